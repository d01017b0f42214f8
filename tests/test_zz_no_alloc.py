"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through its
exported C symbol and compared with the ordinary entry point, twice in a row.

Embedders that may not allocate device memory (fixed memory budgets, someone else's allocator
discipline, moments when a cudaMalloc is not acceptable) use it; its scratch is a fixed array inside
the loaded library.  This file sorts last so that a run stopping at the first failure has already
run every other test."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build_case(seed, tokens_ctx, nh=8, nkv=2, d=128, ps=16, dense=True):
    """A batch of single-token requests with contexts `tokens_ctx`, keys/values on shuffled pages
    of a cache that holds NaN wherever no key or value was written.  ``dense``: also the float64
    attention of every request over its own keys, computed without pages."""
    g = torch.Generator().manual_seed(seed)
    B = len(tokens_ctx)
    pages_per = [(c + ps - 1) // ps for c in tokens_ctx]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    stride = max(pages_per) + 1
    table = np.full((B, stride), -1, np.int32)
    kc = torch.full((num_pages, nkv, ps, d), float("nan"), dtype=torch.bfloat16)
    vc = torch.full_like(kc, float("nan"))
    q = torch.randn(B, nh, d, generator=g).to(torch.bfloat16)
    want = torch.zeros(B, nh, d, dtype=torch.float64)
    for b, c in enumerate(tokens_ctx):
        k = torch.randn(c, nkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(c, nkv, d, generator=g).to(torch.bfloat16)
        for i in range(pages_per[b]):
            table[b, i] = perm.pop()
        for i in range(pages_per[b]):
            n = min(ps, c - i * ps)
            kc[table[b, i], :, :n] = k[i * ps:i * ps + n].transpose(0, 1)
            vc[table[b, i], :, :n] = v[i * ps:i * ps + n].transpose(0, 1)
        if dense:
            for h in range(nh):
                kv = h // (nh // nkv)
                s = (k[:, kv].double() @ q[b, h].double()) * d ** -0.5
                want[b, h] = torch.softmax(s, 0) @ v[:, kv].double()
    to = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), positions=to([c - 1 for c in tokens_ctx]), req=to(list(range(B))),
                q_start=to(list(range(B + 1))), table=to(table.reshape(-1)), stride=stride, B=B, nh=nh, nkv=nkv, d=d, ps=ps,
                num_pages=num_pages, bound=max(tokens_ctx), want=want)


def run_both(case, split):
    from xinfer_b200 import kernels
    from xinfer_b200.native import kernels_lib
    lib = kernels_lib()
    c = case
    B, nh, nkv, d = c["B"], c["nh"], c["nkv"], c["d"]
    num_splits = (c["bound"] + split - 1) // split
    scale = d ** -0.5
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    # the ordinary entry point, with scratch from the caller
    ref = torch.zeros(B, nh, d, dtype=torch.bfloat16, device=DEV)
    part_o = torch.zeros(B * nh * num_splits * d, dtype=torch.float32, device=DEV)
    part_ml = torch.zeros(B * nh * num_splits * 2, dtype=torch.float32, device=DEV)
    tickets = torch.zeros(B * nkv, dtype=torch.int32, device=DEV)
    kernels.attn_decode_bf16(ref, part_o, part_ml, c["q"], c["kc"], c["vc"], c["positions"], c["req"], c["q_start"], B,
                             c["table"], c["stride"], None, scale, 4, True, split, num_splits, B, err, tickets)
    # the entry point that allocates nothing, through its C symbol
    fn = lib.xb_attn_decode_bf16_noalloc
    fn.restype = ctypes.c_int
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, I, I, I, I, P, P]
    out = torch.zeros(B, nh, d, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    # free device memory as the driver counts it: an allocation inside the library, by any route,
    # would show here (torch's own counter only sees torch's allocator)
    free_before, _ = torch.cuda.mem_get_info()
    rc = fn(out.data_ptr(), c["q"].data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(), c["positions"].data_ptr(),
            c["req"].data_ptr(), c["q_start"].data_ptr(), B, c["table"].data_ptr(), c["stride"], nh, nkv, d, c["ps"],
            c["num_pages"], 0, scale, 4, 1, split, num_splits, B, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    return rc, out, ref, int(err), free_before - free_after


def test_no_alloc_entry_matches_the_ordinary_one_twice_in_a_row():
    # two different calls back to back: the second finds the first one's leftovers in the array
    for n, (seed, ctxs, split) in enumerate(((0, [700, 65, 1300, 64], 128), (1, [2000, 1, 333], 64))):
        case = build_case(seed, ctxs)
        rc, out, ref, err, taken = run_both(case, split)
        assert rc == 0 and err == 0
        # the same kernel with the same key ranges, merged in the same order: the same bits
        assert torch.equal(out, ref)
        # and both are right: dense float64 attention over each request's own keys (the cache holds
        # NaN wherever nothing was written, so a key read from outside a request shows)
        assert torch.isfinite(out.float()).all()
        diff = (out.double().cpu() - case["want"]).abs().max().item()
        assert diff <= 1.6e-2, diff          # the bfloat16 kernel tolerance of the other attention tests
        if n > 0:      # the first call on a device resolves the array's address; from then on nothing may be taken
            assert taken == 0, f"{taken} bytes of device memory went missing during the call"


def test_no_alloc_entry_refuses_what_does_not_fit():
    from xinfer_b200.native import kernels_lib
    lib = kernels_lib()
    need = lib.xb_attn_decode_bf16_noalloc_need
    need.restype = ctypes.c_longlong
    need.argtypes = [ctypes.c_int] * 5
    assert need(8, 2, 128, 16, 4) == 256 + 4 * 8 * 16 * 2 * 4 + 4 * 8 * 16 * 128 * 4
    assert need(32, 8, 128, 64, 64) > (8 << 20)
    case = build_case(2, [4096] * 64, nh=32, nkv=8, dense=False)
    rc, out, ref, err, _ = run_both(case, 64)
    assert rc == -2                                           # XB_NOALLOC_TOO_LARGE, and nothing was written
    assert torch.count_nonzero(out) == 0
