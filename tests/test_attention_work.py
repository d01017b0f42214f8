"""The host-side work list of the prefill attention kernel (no GPU): every item exactly once, the
longest first on each CTA, loads even."""
import ctypes

import numpy as np

from xinfer_b200.native import host_lib


def work_list(counts, starts, dec_max, window, head_pairs, max_ctas):
    counts, starts = np.asarray(counts, dtype=np.int32), np.asarray(starts, dtype=np.int32)
    cap = max_ctas + 1 + 3 * int(((counts + 127) // 128).sum()) * head_pairs + 8
    out = np.full(cap, -9, dtype=np.int32)
    ctas = ctypes.c_int(0)
    used = host_lib().xb_attn_prefill_work(len(counts), counts.ctypes.data, starts.ctypes.data, dec_max, window, head_pairs,
                                           max_ctas, out.ctypes.data, cap, ctypes.byref(ctas))
    c = ctas.value
    offs = out[: c + 1]
    items = out[c + 1: used].reshape(-1, 3)
    return c, offs, items, used


def cost(b, tile, counts, starts, window):
    p0 = starts[b] + tile * 128
    rows = min(128, counts[b] - tile * 128)
    last, first = p0 + rows - 1, (max(0, p0 - window + 1) if window else 0)
    return last // 64 - first // 64 + 1


def test_every_item_once_and_loads_even():
    counts, starts = [2048, 3, 700, 1, 129], [0, 50, 4000, 9, 77]
    for window, head_pairs, max_ctas in ((0, 16, 148), (300, 3, 148), (0, 16, 7), (0, 1, 148)):
        c, offs, items, used = work_list(counts, starts, 4, window, head_pairs, max_ctas)
        want = {(b, t, hp) for b in (0, 2, 4) for t in range((counts[b] + 127) // 128) for hp in range(head_pairs)}
        got = [tuple(r) for r in items.tolist()]
        assert len(got) == len(want) and set(got) == want           # portions of at most 4 tokens are not here
        assert c == min(max_ctas, len(want)) and offs[0] == 0 and offs[-1] == len(want) and (np.diff(offs) >= 1).all()
        loads = []
        for k in range(c):
            mine = [cost(b, t, counts, starts, window) + 3 for b, t, _ in got[offs[k]: offs[k + 1]]]
            assert mine == sorted(mine, reverse=True)                # a CTA's longest item first
            loads.append(sum(mine))
        biggest = max(cost(b, t, counts, starts, window) + 3 for b, t, _ in got)
        assert max(loads) - min(loads) <= biggest                    # what longest-first onto the least loaded guarantees


def test_nothing_to_do_and_too_small_a_buffer():
    c, offs, items, used = work_list([3, 4, 1], [0, 0, 0], 4, 0, 8, 148)
    assert c == 0 and used == 0
    counts, starts = np.asarray([1000], dtype=np.int32), np.asarray([0], dtype=np.int32)
    out = np.zeros(10, dtype=np.int32)
    ctas = ctypes.c_int(0)
    assert host_lib().xb_attn_prefill_work(1, counts.ctypes.data, starts.ctypes.data, 4, 0, 4, 148, out.ctypes.data, 10,
                                           ctypes.byref(ctas)) == -1
