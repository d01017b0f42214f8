"""The host-side work list of the prefill attention kernel (no GPU): every item exactly once, the
longest first on each CTA, loads even."""
import ctypes

import numpy as np

from xinfer_b200.native import host_lib


def work_list(counts, starts, dec_max, window, heads, kv_heads, max_ctas):
    counts, starts = np.asarray(counts, dtype=np.int32), np.asarray(starts, dtype=np.int32)
    cap = max_ctas + 1 + 4 * int(((counts + 127) // 128).sum()) * heads + 8
    out = np.full(cap, -9, dtype=np.int32)
    ctas = ctypes.c_int(0)
    used = host_lib().xb_attn_prefill_work(len(counts), counts.ctypes.data, starts.ctypes.data, dec_max, window, heads, kv_heads,
                                           max_ctas, out.ctypes.data, cap, ctypes.byref(ctas))
    c = ctas.value
    offs = out[: c + 1]
    items = out[c + 1: used].reshape(-1, 4)
    return c, offs, items, used


def cost(b, tile, counts, starts, window):
    p0 = starts[b] + tile * 128
    rows = min(128, counts[b] - tile * 128)
    last, first = p0 + rows - 1, (max(0, p0 - window + 1) if window else 0)
    return last // 64 - first // 64 + 1


def test_every_head_of_every_tile_once_and_loads_even():
    counts, starts = [2048, 3, 700, 1, 129], [0, 50, 4000, 9, 77]
    for window, heads, kv_heads, max_ctas in ((0, 32, 8, 148), (300, 6, 2, 148), (0, 32, 8, 7), (0, 5, 1, 148), (0, 2, 2, 148)):
        c, offs, items, used = work_list(counts, starts, 4, window, heads, kv_heads, max_ctas)
        G = heads // kv_heads
        got = [tuple(r) for r in items.tolist()]
        # every (portion, tile, head) is covered exactly once; portions of at most 4 tokens are not here
        covered = [(b, t, h) for b, t, h0, n in got for h in range(h0, h0 + n)]
        want = {(b, t, h) for b in (0, 2, 4) for t in range((counts[b] + 127) // 128) for h in range(heads)}
        assert len(covered) == len(want) and set(covered) == want
        for b, t, h0, n in got:
            assert n in (1, 2) and h0 // G == (h0 + n - 1) // G           # the heads of an item share their key/value head
        assert c == min(max_ctas, len(got)) and offs[0] == 0 and offs[-1] == len(got) and (np.diff(offs) >= 1).all()
        loads = []
        for k in range(c):
            mine = [cost(b, t, counts, starts, window) * (6 if n == 2 else 4) + 18 for b, t, _, n in got[offs[k]: offs[k + 1]]]
            loads.append(sum(mine))
        biggest = max(cost(b, t, counts, starts, window) * (6 if n == 2 else 4) + 18 for b, t, _, n in got)
        assert max(loads) - min(loads) <= biggest                    # what longest-first onto the least loaded guarantees
    # few items: single heads, so that the SMs have something to do
    c, offs, items, used = work_list([512], [0], 4, 0, 16, 8, 148)
    assert c == 4 * 16 and (items[:, 3] == 1).all()
    c, offs, items, used = work_list([1536], [0], 4, 0, 32, 8, 148)       # 192 pairs fill 148 CTAs: pairs stay
    assert c == 148 and (items[:, 3] == 2).all()
    # many items: pairs
    c, offs, items, used = work_list([4096], [0], 4, 0, 32, 8, 148)
    assert c == 148 and (items[:, 3] == 2).all() and len(items) == 32 * 16
    # two heads per group and a long context: 128 pairs on 128 CTAs end before 256 single heads on 148
    c, offs, items, used = work_list([2048], [30000], 4, 0, 16, 8, 148)
    assert c == 128 and (items[:, 3] == 2).all()
    c, offs, items, used = work_list([2048], [0], 4, 0, 16, 8, 148)       # the same from position 0: short items, single heads
    assert c == 148 and (items[:, 3] == 1).all()


def test_nothing_to_do_and_too_small_a_buffer():
    c, offs, items, used = work_list([3, 4, 1], [0, 0, 0], 4, 0, 32, 8, 148)
    assert c == 0 and used == 0
    counts, starts = np.asarray([1000], dtype=np.int32), np.asarray([0], dtype=np.int32)
    out = np.zeros(10, dtype=np.int32)
    ctas = ctypes.c_int(0)
    assert host_lib().xb_attn_prefill_work(1, counts.ctypes.data, starts.ctypes.data, 4, 0, 8, 2, 148, out.ctypes.data, 10,
                                           ctypes.byref(ctas)) == -1
