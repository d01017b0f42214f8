"""Each CUDA kernel alone against a plain PyTorch float32 restatement of the same operation, at
sizes other than the engine's tiny models (odd widths, head sizes in steps of 16, groups of
2/4/6/8, vocabularies that are no power of two)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


@pytest.fixture(params=[True, False], ids=["vectorized", "plain"])
def both_families(request):
    """Norm, gate and q/k preparation exist as plain kernels and as 16-byte-access bfloat16
    kernels; the tests that use this fixture check both."""
    from xinfer_b200 import kernels
    old = kernels.vectorized
    kernels.vectorized = request.param
    yield request.param
    kernels.vectorized = old


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=dev())


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(dev())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 24, 5), (37, 100, 331), (64, 4096, 1000)])
def test_embedding(dtype, T, H, V):
    from xinfer_b200 import kernels
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=dev())
    out = torch.empty(T, H, dtype=dtype, device=dev())
    e = err_word()
    kernels.embedding(out, table, ids, e)
    assert torch.equal(out, table[ids.long()]) and int(e) == 0
    ids[T // 2] = V  # out of range: flagged, never read
    kernels.embedding(out, table, ids, e)
    assert int(e) == kernels.ERR_BAD_TOKEN and torch.count_nonzero(out[T // 2]) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,dim,eps,offset", [(1, 16, 1e-6, 0.0), (33, 100, 1e-5, 0.0), (7, 5120, 3e-6, 1.0), (5, 8200, 1e-6, 0.0),
                                                 (3, 20000, 1e-6, 0.0), (700, 4096, 1e-6, 0.0)])
def test_rmsnorm_plain_fused_and_gathered(dtype, rows, dim, eps, offset, both_families):
    from xinfer_b200 import kernels
    x, br = rnd(rows, dim, dtype=dtype, seed=1), rnd(rows, dim, dtype=dtype, seed=2)
    w = rnd(dim, seed=3) * 0.1 + 1
    e = err_word()

    def ref(s):
        s = s.float()
        return s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * (offset + w)
    out = torch.empty_like(x)
    kernels.rmsnorm(out, x, w, eps, e, weight_offset=offset)
    assert (out.float() - ref(x)).abs().max() <= tol(dtype, 4)
    # fused residual sum: the sum is formed in float32, rounded to the storage type, then normed
    xs = x.clone()
    kernels.rmsnorm(out, xs, w, eps, e, branch=br, sum_out=xs, weight_offset=offset)
    s = (x.float() + br.float()).to(dtype)
    assert torch.equal(xs, s)
    assert (out.float() - ref(s)).abs().max() <= tol(dtype, 4)
    # gathered rows (with the sum, as the final norm uses it)
    idx = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device=dev())
    g = torch.empty(3, dim, dtype=dtype, device=dev())
    kernels.rmsnorm(g, x, w, eps, e, branch=br, rows=idx, weight_offset=offset)
    assert (g.float() - ref(s[idx.long()])).abs().max() <= tol(dtype, 4)
    assert int(e) == 0
    idx[1] = rows
    kernels.rmsnorm(g, x, w, eps, e, rows=idx)
    assert int(e) == kernels.ERR_BAD_ROW


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (33, 100, 70), (130, 257, 129), (3, 1000, 4096)])
def test_gemm_plain_is_true_float32_and_row_independent(M, N, K):
    from xinfer_b200 import kernels
    a, w = rnd(M, K, seed=4), rnd(N, K, seed=5)
    out = torch.empty(M, N, device=dev())
    kernels.gemm_plain(out, a, w)
    ref = (a.double() @ w.double().t())
    assert (out.double() - ref).abs().max() <= 1e-6 * K ** 0.5 * float(ref.abs().max())
    # a row's result does not depend on the other rows of the batch
    one = torch.empty(1, N, device=dev())
    kernels.gemm_plain(one, a[M // 2: M // 2 + 1].contiguous(), w)
    assert torch.equal(one[0], out[M // 2])
    # mixed storage types
    ab, wb = a.bfloat16(), w.bfloat16()
    o2 = torch.empty(M, N, device=dev())
    kernels.gemm_plain(o2, ab, wb)
    assert (o2.double() - ab.double() @ wb.double().t()).abs().max() <= 1e-6 * K ** 0.5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 8), (13, 48), (37, 11008 // 16 + 3), (5, 12288), (600, 8200)])
def test_swiglu(dtype, T, I, both_families):
    from xinfer_b200 import kernels
    gu = rnd(T, 2 * I, dtype=dtype, scale=3.0)
    out = torch.empty(T, I, dtype=dtype, device=dev())
    kernels.swiglu(out, gu)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    ref = (g / (1 + torch.exp(-g)) * u).to(dtype)
    # within one unit in the last place of the storage type (the reference's own probe bound,
    # tests/probes/compare_attention_misc_probe.py:73-87)
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -22
    assert ((out.float() - ref.float()).abs() <= ulp * ref.float().abs().clamp_min(1e-3)).all()


def make_cache(num_pages, nkv, ps, d, dtype):
    k = torch.zeros(num_pages, nkv, ps, d, dtype=dtype, device=dev())
    return k, torch.zeros_like(k)


def meta(entries, ps, num_pages, seed=0):
    """entries: list of (start, count).  Pages are dealt in a shuffled order."""
    rng = np.random.default_rng(seed)
    pages = rng.permutation(num_pages).tolist()
    B = len(entries)
    stride = max((s + c + ps - 1) // ps for s, c in entries) + 1
    table = np.full((B, stride), -1, np.int32)
    pos, req = [], []
    for b, (s, c) in enumerate(entries):
        for i in range((s + c + ps - 1) // ps):
            table[b, i] = pages.pop()
        pos += list(range(s, s + c))
        req += [b] * c
    to = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev())
    return to(pos), to(req), to(table.reshape(-1)), stride, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot,inter,ps", [(4, 2, 16, 16, False, 16), (6, 1, 48, 48, False, 8), (8, 8, 128, 64, True, 4), (10, 5, 80, 80, False, 16), (32, 8, 128, 128, False, 16), (3, 3, 256, 256, True, 16), (5, 1, 64, 32, False, 16)])
def test_qk_norm_rope_write(dtype, nh, nkv, d, rot, inter, ps, both_families):
    from xinfer_b200 import kernels
    entries = [(0, 9), (21, 1), (5, 14)]
    T = sum(c for _, c in entries)
    num_pages, max_pos, eps, theta = 30, 64, 1e-5, 10000.0
    pos, req, table, stride, table_np = meta(entries, ps, num_pages)
    qkv = rnd(T, (nh + 2 * nkv) * d, dtype=dtype, seed=6)
    qw, kw = rnd(d, seed=7) * 0.2 + 1, rnd(d, seed=8) * 0.2 + 1
    inv = torch.tensor((1.0 / theta ** (np.arange(0, rot, 2) / rot)).astype(np.float32), device=dev())
    cos, sin = torch.empty(max_pos, rot // 2, device=dev()), torch.empty(max_pos, rot // 2, device=dev())
    kernels.rope_table(cos, sin, inv)
    ang = torch.arange(max_pos, device=dev()).float()[:, None] * inv[None, :]
    assert (cos - torch.cos(ang)).abs().max() < 2e-6 and (sin - torch.sin(ang)).abs().max() < 2e-6
    kc, vc = make_cache(num_pages, nkv, ps, d, dtype)
    q_out = torch.empty(T, nh, d, dtype=dtype, device=dev())
    e = err_word()
    kernels.qk_norm_rope_write(q_out, kc, vc, qkv, qw, kw, cos, sin, pos, req, table, stride, nh, nkv, d, rot, inter, eps, True, e)
    assert int(e) == 0

    def ref_rot(x, w):  # x [T, heads, d] float32
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
        c, s = torch.cos(ang[pos.long()])[:, None, :], torch.sin(ang[pos.long()])[:, None, :]
        y = x.clone()
        if inter:
            a, b = x[..., 0:rot:2], x[..., 1:rot:2]
            y[..., 0:rot:2], y[..., 1:rot:2] = a * c - b * s, a * s + b * c
        else:
            a, b = x[..., : rot // 2], x[..., rot // 2: rot]
            y[..., : rot // 2], y[..., rot // 2: rot] = a * c - b * s, a * s + b * c
        return y
    x = qkv.float()
    q_ref = ref_rot(x[:, : nh * d].view(T, nh, d), qw)
    k_ref = ref_rot(x[:, nh * d:(nh + nkv) * d].view(T, nkv, d), kw)
    v_ref = x[:, (nh + nkv) * d:].view(T, nkv, d)
    t_ = tol(dtype, 4)
    assert (q_out.float() - q_ref).abs().max() <= t_
    posl, reql = pos.tolist(), req.tolist()
    for t in range(T):
        page, off = table_np[reql[t], posl[t] // ps], posl[t] % ps
        assert (kc[page, :, off].float() - k_ref[t]).abs().max() <= t_
        assert torch.equal(vc[page, :, off].float(), v_ref[t])
    # nothing else in the cache was touched
    written = kc.float().abs().sum(-1).ne(0).sum().item()
    assert written == T * nkv
    # a table entry outside the pool is flagged and skipped, never written through
    bad = table.clone()
    bad[0] = num_pages + 3
    before = kc.clone()
    kernels.qk_norm_rope_write(q_out, kc, vc, qkv, qw, kw, cos, sin, pos, req, bad, stride, nh, nkv, d, rot, inter, eps, True, e)
    assert int(e) == kernels.ERR_BAD_PAGE


def attention_ref(q, k_all, v_all, start, window, scale):
    """q [n, nh, d] at positions start..start+n-1 over keys [ctx, nkv, d] (float64)."""
    n, nh, d = q.shape
    nkv = k_all.shape[1]
    out = torch.zeros(n, nh, d, dtype=torch.float64)
    for i in range(n):
        p = start + i
        lo = 0 if not window else max(0, p - window + 1)
        for h in range(nh):
            g = h // (nh // nkv)
            s = (k_all[lo:p + 1, g] @ q[i, h]) * scale
            out[i, h] = torch.softmax(s, 0) @ v_all[lo:p + 1, g]
    return out


def attention_case(kernel, dtype, nh, nkv, d, ps, entries, window, plant=None, seed=0, want_out=False):
    """Fill a cache through shuffled pages, run `kernel`, compare with the dense reference."""
    from xinfer_b200 import kernels
    num_pages = sum((s + c + ps - 1) // ps for s, c in entries) + 3
    pos, req, table, stride, table_np = meta(entries, ps, num_pages, seed)
    kc, vc = make_cache(num_pages, nkv, ps, d, dtype)
    kc.fill_(float("nan"))   # anything read beyond a request's keys poisons the result
    vc.fill_(float("nan"))
    T = sum(c for _, c in entries)
    q = rnd(T, nh, d, dtype=dtype, seed=seed + 9)
    ks, vs = [], []
    for b, (s, c) in enumerate(entries):
        k = rnd(s + c, nkv, d, dtype=dtype, seed=seed + 20 + b)
        v = rnd(s + c, nkv, d, dtype=dtype, seed=seed + 40 + b)
        if plant is not None:
            plant(b, s, c, q, k, v)
        ks.append(k)
        vs.append(v)
        for j in range(s + c):
            kc[table_np[b, j // ps], :, j % ps] = k[j]
            vc[table_np[b, j // ps], :, j % ps] = v[j]
    out = torch.full((T, nh, d), float("nan"), dtype=dtype, device=dev())
    e = err_word()
    scale = 1.0 / math.sqrt(d)
    kernel(out, q, kc, vc, pos, req, table, stride, window, scale, e, entries)
    assert int(e) == 0
    t0 = 0
    worst = 0.0
    for b, (s, c) in enumerate(entries):
        ref = attention_ref(q[t0:t0 + c].double().cpu(), ks[b].double().cpu(), vs[b].double().cpu(), s, window, scale)
        diff = (out[t0:t0 + c].double().cpu() - ref).abs().max().item()
        assert diff == diff, f"entry {b}: NaN in the output (a key beyond the request's range was read)"
        worst = max(worst, diff)
        t0 += c
    return (worst, out) if want_out else worst


def plain_kernel(out, q, kc, vc, pos, req, table, stride, window, scale, e, entries):
    from xinfer_b200 import kernels
    kernels.attention_plain(out, q, kc, vc, pos, req, table, stride, window, scale, e)


CASES = [
    # nh, nkv, d, page, entries (start, count), window
    (4, 2, 16, 16, [(0, 1)], None),
    (4, 2, 16, 16, [(0, 17), (16, 1), (15, 2)], None),
    (6, 1, 32, 8, [(0, 40), (63, 1), (5, 7), (64, 1)], None),
    (8, 2, 64, 16, [(33, 31), (0, 3)], 20),
    (8, 1, 128, 16, [(300, 1), (0, 70)], None),
    (6, 3, 48, 4, [(10, 25), (36, 1)], 5),
    (16, 2, 80, 16, [(0, 33)], 16),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,ps,entries,window", CASES)
def test_attention_plain(dtype, nh, nkv, d, ps, entries, window):
    worst = attention_case(plain_kernel, dtype, nh, nkv, d, ps, entries, window)
    assert worst <= tol(dtype, 2), worst


def far_key_checks(kernel, dtype):
    """One key far back gets a score that dominates and a value unlike all others: if a kernel
    skipped it (or read past the window's edge) the output would be wrong by O(1), not by
    rounding.  Checked for a key far behind, for the oldest key inside a window and for the
    newest key outside it."""
    window = 50
    nh, nkv, d, ps = 2, 1, 32, 16
    for win, start, far, visible in ((None, 300, 3, True), (window, 120, 120 - window + 1, True),
                                     (window, 120, 120 - window, False)):
        def plant(b, s, c, q, k, v, far=far):
            qd = q[0, 0, :].float()
            k[far] = 0
            k[far, 0] = (qd / qd.norm() * 60).to(k.dtype)     # head 0's query points at it
            v[far] = 7.0
        worst, out = attention_case(kernel, dtype, nh, nkv, d, ps, [(start, 1)], win, plant=plant, seed=5, want_out=True)
        assert worst <= tol(dtype, 8), (win, far, worst)
        if visible:
            assert (out[0, 0].float() - 7.0).abs().max() < 0.1, "the planted key must decide head 0"
        else:
            assert (out[0, 0].float() - 7.0).abs().min() > 3.0, "a key behind the window must not be seen"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_plain_sees_one_far_key_and_the_windows_edge(dtype):
    far_key_checks(plain_kernel, dtype)


# ---- the tensor-core attention kernels (bfloat16) through the backend that picks them -------------
def tiled_kernel(out, q, kc, vc, pos, req, table, stride, window, scale, e, entries):
    from types import SimpleNamespace
    from xinfer_b200.parts import LayerCache, Workspace
    from xinfer_b200.parts import attention_backend
    counts = [c for _, c in entries]
    q_start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    to = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev())
    ctx = SimpleNamespace(positions=pos, req_of_token=req, q_start=to(q_start), start_pos=to([s for s, _ in entries]),
                          num_entries=len(entries), num_tokens=int(q_start[-1]), h_q_start=q_start, real_entries=len(entries),
                          h_start_pos=np.asarray([s for s, _ in entries], dtype=np.int32),
                          max_context=max(s + c for s, c in entries), fixed_shapes=False, scratch={},
                          workspace=Workspace(dev()), err=e)
    cache = LayerCache.of_keys_and_values(kc, vc, 0, kc.shape[2])
    attention_backend.attend(out, q, cache, ctx, table, stride, window, scale)


TILED_CASES = CASES + [
    (32, 8, 128, 16, [(0, 200), (1000, 1), (130, 3), (64, 64), (511, 2)], None),     # 8B head layout, mixed batch
    (16, 8, 128, 16, [(0, 70), (700, 1)], 100),
    (4, 4, 16, 8, [(0, 65), (3, 130)], None),
    (12, 2, 96, 16, [(250, 1), (256, 1), (255, 1), (0, 1)], None),                  # range edges of the decode kernel
    (40, 2, 32, 16, [(513, 1), (20, 150)], 300),                                   # 20 query heads per kv head: two row tiles
    (5, 5, 256, 16, [(0, 90), (300, 1)], None),
    (8, 2, 112, 32, [(77, 4), (0, 5), (1023, 1)], 512),
]


@pytest.fixture(params=[True, False], ids=["tcgen05", "mma_sync"])
def prefill_family(request, monkeypatch):
    """Long portions and single tokens run on the tcgen05 kernels where they take the sizes, else
    on the mma.sync kernels; tests with this fixture run both."""
    from xinfer_b200.parts import attention_backend
    monkeypatch.setattr(attention_backend, "PREFILL_TC", request.param)
    monkeypatch.setattr(attention_backend, "DECODE_TC", request.param)
    return request.param


@pytest.mark.parametrize("nh,nkv,d,ps,entries,window", TILED_CASES)
def test_attention_tiled_bf16(nh, nkv, d, ps, entries, window, prefill_family):
    worst = attention_case(tiled_kernel, torch.bfloat16, nh, nkv, d, ps, entries, window)
    assert worst <= tol(torch.bfloat16, 2), worst


@pytest.mark.parametrize("nh,nkv,d,ps,entries,window", [
    (2, 1, 128, 16, [(0, 128)], None), (2, 1, 128, 16, [(0, 200)], None), (4, 2, 64, 8, [(37, 300), (0, 129)], None),
    (4, 4, 96, 32, [(1000, 260)], 200), (2, 2, 16, 64, [(5, 150)], None), (8, 2, 128, 128, [(100, 500), (0, 6)], 333),
    (3, 1, 48, 16, [(600, 700)], None), (6, 1, 80, 16, [(0, 1300), (2000, 131)], None), (4, 1, 128, 8, [(4000, 257)], 1000),
    (5, 5, 128, 16, [(0, 300), (900, 140)], None), (10, 2, 64, 32, [(50, 500)], 300)])
def test_attention_prefill_tcgen05(nh, nkv, d, ps, entries, window, monkeypatch):
    """Even and odd numbers of query heads per key/value head (the kernel takes them two at a time)."""
    from xinfer_b200.parts import attention_backend
    monkeypatch.setattr(attention_backend, "PREFILL_TC", True)
    worst = attention_case(tiled_kernel, torch.bfloat16, nh, nkv, d, ps, entries, window)
    assert worst <= tol(torch.bfloat16, 2), worst


@pytest.mark.parametrize("window", [None, 5000])
def test_attention_prefill_tcgen05_after_a_long_prefix(window, monkeypatch):
    """A portion of 300 tokens after 20,000 cached ones: some 320 key tiles go through the four-stage
    rings and the two score buffers of a CTA, with and without a window that starts inside a tile."""
    from xinfer_b200.parts import attention_backend
    monkeypatch.setattr(attention_backend, "PREFILL_TC", True)
    worst = attention_case(tiled_kernel, torch.bfloat16, 4, 2, 128, 16, [(20000, 300)], window)
    assert worst <= tol(torch.bfloat16, 2), worst


def test_attention_tiled_sees_one_far_key_and_the_windows_edge(prefill_family):
    far_key_checks(tiled_kernel, torch.bfloat16)


@pytest.mark.parametrize("nh,nkv,d,ps,entries,window", [
    (4, 1, 128, 16, [(0, 1)], None),                                            # a single key
    (32, 8, 128, 16, [(4095, 1), (63, 1), (64, 1), (65, 1), (1, 1), (2049, 1), (700, 1), (127, 1)], None),
    (8, 2, 64, 8, [(1000, 1), (999, 2), (1001, 3), (5, 4)], None),             # several tokens per small portion
    (6, 1, 48, 16, [(3000, 1), (129, 1)], 700),                                 # window over several ranges
    (6, 1, 48, 16, [(3000, 1), (129, 1)], 64),                                  # window of one tile
    (12, 1, 96, 32, [(513, 1)], None),                                          # 12 heads share the keys: both row sets
    (16, 1, 16, 64, [(200, 1), (77, 2)], 100),                                  # a full 16-row group, page = tile
    (3, 3, 112, 128, [(2500, 1), (130, 1)], None),                              # page larger than a tile
    (2, 2, 80, 16, [(9000, 1)], None),
])
def test_attention_decode_tcgen05(nh, nkv, d, ps, entries, window, monkeypatch):
    """Single tokens (and portions of up to four) over long contexts: ranges, their merge, range
    edges at multiples of the tile, windows."""
    from xinfer_b200.parts import attention_backend
    from xinfer_b200 import kernels

    def not_this_one(*a, **k):
        raise AssertionError("the mma.sync decode kernel was called")
    monkeypatch.setattr(attention_backend, "DECODE_TC", True)
    monkeypatch.setattr(kernels, "attn_decode_bf16", not_this_one)
    assert attention_backend.decode_tc_takes(nh, nkv, d, ps)
    worst = attention_case(tiled_kernel, torch.bfloat16, nh, nkv, d, ps, entries, window)
    assert worst <= tol(torch.bfloat16, 2), worst


def test_attention_decode_tcgen05_never_reads_a_poisoned_page(monkeypatch):
    """Pages the request does not own hold NaN: ranges end inside pages and tiles, and nothing of
    what lies behind may reach a result."""
    from xinfer_b200.parts import attention_backend
    monkeypatch.setattr(attention_backend, "DECODE_TC", True)
    for start in (0, 15, 16, 63, 64, 100, 1023, 1024):
        worst = attention_case(tiled_kernel, torch.bfloat16, 8, 2, 128, 16, [(start, 1), (start + 7, 1)], None)
        assert worst <= tol(torch.bfloat16, 2), (start, worst)


def test_attention_tiled_far_key_in_a_long_prompt_portion(prefill_family):
    """The same planted key, but seen from the prefill kernel: a 70-token portion starting at 400."""
    nh, nkv, d, ps = 4, 2, 64, 16
    for win, far, visible in ((None, 5, True), (128, 400 + 69 - 128 + 1, True), (128, 400 + 69 - 128, False)):
        def plant(b, s, c, q, k, v, far=far):
            qd = q[69, 0, :].float()                   # the last query of the portion, head 0
            k[far] = 0
            k[far, 0] = (qd / qd.norm() * 60).to(k.dtype)
            v[far] = 7.0
        worst, out = attention_case(tiled_kernel, torch.bfloat16, nh, nkv, d, ps, [(400, 70)], win, plant=plant, seed=11, want_out=True)
        assert worst <= tol(torch.bfloat16, 8), (win, far, worst)
        if visible:
            assert (out[69, 0].float() - 7.0).abs().max() < 0.1
        else:
            assert (out[69, 0].float() - 7.0).abs().min() > 3.0


def test_attention_tiled_refuses_what_it_cannot_do():
    from xinfer_b200 import kernels
    assert not kernels.attn_tiled_supported(torch.bfloat16, 40)
    assert not kernels.attn_tiled_supported(torch.bfloat16, 272)
    assert not kernels.attn_tiled_supported(torch.float32, 64)
    q = torch.zeros(2, 4, 40, dtype=torch.bfloat16, device=dev())
    kc = torch.zeros(4, 2, 16, 40, dtype=torch.bfloat16, device=dev())
    z = torch.zeros(4, dtype=torch.int32, device=dev())
    with pytest.raises(kernels.KernelError, match="head size"):
        kernels.attn_prefill_bf16(q.clone(), q, kc, kc.clone(), z, z, 1, z, 4, None, 1.0, 4, 1, 64, err_word())
    # head size 40 still runs: the backend hands it to the plain kernel
    worst = attention_case(tiled_kernel, torch.bfloat16, 4, 2, 40, 16, [(0, 30), (50, 1)], None)
    assert worst <= tol(torch.bfloat16, 2)


@pytest.mark.parametrize("warps", [4, 8])
def test_attention_prefill_tile_sizes(warps, monkeypatch):
    from xinfer_b200.parts import attention_backend
    monkeypatch.setattr(attention_backend, "PREFILL_WARPS", warps)
    for nh, nkv, d, ps, entries, window in [(8, 2, 128, 16, [(0, 300), (100, 129), (5, 64)], None), (4, 1, 64, 8, [(37, 200)], 90)]:
        worst = attention_case(tiled_kernel, torch.bfloat16, nh, nkv, d, ps, entries, window)
        assert worst <= tol(torch.bfloat16, 2), worst


def test_decode_tcgen05_launch_figures():
    from xinfer_b200 import kernels
    from xinfer_b200.parts.attention_backend import DECODE_TC_CTAS, decode_tc_launch
    assert decode_tc_launch(1, 1, 1) == (1, 1)
    assert decode_tc_launch(4096, 8, 8)[0] == DECODE_TC_CTAS            # enough work for every slot
    assert decode_tc_launch(300, 1, 2) == (3, 2)                        # 5 tiles x 2 heads, 4 tiles per piece at least
    assert kernels.attn_decode_plan_size(8, 296, 8) == 4 + 8 * (8 + 37 + 2)
    for bound, tokens, heads in [(4096, 1, 8), (100000, 3, 2), (64, 500, 8), (5000, 64, 1)]:
        ctas, splits = decode_tc_launch(bound, tokens, heads)
        assert 1 <= ctas <= DECODE_TC_CTAS and splits >= 1
        # what the kernel does with the longest context: pieces = max(1, tiles / share)
        tiles = (bound + 63) // 64
        for total in (tiles * heads, tokens * heads * tiles):            # alone, or every token as long
            share = max(4, -(-total // ctas))
            assert splits >= max(1, tiles // share)
        assert splits == kernels.decode_tc_splits_max(ctas, heads, bound, 256)


def test_decode_split_choice():
    from xinfer_b200.parts.attention_backend import decode_split
    for bound, pairs in [(1, 1), (4096, 8), (4096, 64), (4096, 512), (40000, 8), (100, 4096)]:
        split, n = decode_split(bound, pairs)
        assert split % 64 == 0 and split >= 64 and (n - 1) * split < bound <= n * split
    assert decode_split(4096, 8)[1] >= 16              # few pairs: cut finely
    assert decode_split(4096, 64)[1] * 64 <= 444       # one wave holds every CTA
    assert decode_split(64, 5000) == (64, 1)


@pytest.mark.parametrize("shape", [(1, 7), (3, 1000), (64, 1016), (5, 151936), (2, 9)])
def test_widen_bf16_is_exact(shape):
    from xinfer_b200 import kernels
    x = rnd(*shape, dtype=torch.bfloat16, seed=31, scale=30.0)
    out = torch.full(shape, float("nan"), device=dev())
    kernels.widen_bf16(out, x)
    assert torch.equal(out, x.float())
    # a view that starts off a 16-byte boundary takes the element-wise kernel
    flat = rnd(4099, dtype=torch.bfloat16, seed=32)
    part = flat[3:]
    o2 = torch.empty(4096, device=dev())
    kernels.widen_bf16(o2, part)
    assert torch.equal(o2, part.float())


# ---------------------------------------------------------------------------------------------
# the many-row form of the SiLU gate against its few-row form: the same bits
# ---------------------------------------------------------------------------------------------
DEV = "cuda:0"


def _both_forms(fn):
    """Run ``fn`` with the few-row kernels, then with the many-row ones."""
    from xinfer_b200 import kernels
    was = kernels.many_rows
    try:
        kernels.many_rows = 1 << 30
        before = dict(kernels.launch_counts())
        few = fn()
        kernels.many_rows = 1
        many = fn()
        after = kernels.launch_counts()
    finally:
        kernels.many_rows = was
    return few, many, {k: after[k] - before.get(k, 0) for k in after if after[k] != before.get(k, 0)}


@pytest.mark.parametrize("tokens,inter", [(300, 12288), (1111, 176), (600, 3072), (2, 25600)])
def test_swiglu_many_rows_equals_few_rows(tokens, inter):
    from xinfer_b200 import kernels
    g = torch.Generator().manual_seed(tokens)
    gu = (torch.randn(tokens, 2 * inter, generator=g) * 3).to(torch.bfloat16).to(DEV)

    def run():
        out = torch.zeros(tokens, inter, dtype=torch.bfloat16, device=DEV)
        kernels.swiglu(out, gu)
        return out

    o1, o2, ran = _both_forms(run)
    assert ran.get("swiglu_rows_bf16") == 1 and ran.get("swiglu_bf16") == 1
    assert torch.equal(o1, o2)
    gate, up = gu[:, :inter].float(), gu[:, inter:].float()
    assert (o2.float() - torch.nn.functional.silu(gate) * up).abs().max().item() <= 0.02 * (gate.abs() * up.abs()).max().item()


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(4))
def test_attention_tiled_random_layouts_and_batches(seed):
    """Random head layouts (1 to 16 query heads per key/value head), head sizes, page sizes, windows and
    mixed batches of decode tokens and prompt portions, through the backend's choice of kernels."""
    rng = np.random.default_rng(500 + seed)
    for case in range(10):
        nkv = int(rng.choice([1, 2, 3, 4, 8]))
        G = int(rng.choice([1, 2, 3, 4, 5, 8, 16]))
        if nkv * G > 40:
            nkv = max(1, 40 // G)
        d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128]))
        ps = int(rng.choice([8, 16, 32, 64, 128]))
        window = None if rng.random() < 0.6 else int(rng.integers(3, 900))
        entries = []
        for _ in range(int(rng.integers(1, 6))):
            kind = rng.random()
            if kind < 0.45:
                entries.append((int(rng.integers(0, 1500)), int(rng.integers(1, 5))))      # decode tokens behind a context
            elif kind < 0.9:
                entries.append((int(rng.integers(0, 700)), int(rng.integers(5, 400))))      # a portion behind a prefix
            else:
                entries.append((0, int(rng.integers(1, 300))))                              # the start of a prompt
        worst = attention_case(tiled_kernel, torch.bfloat16, nkv * G, nkv, d, ps, entries, window, seed=case)
        assert worst <= tol(torch.bfloat16, 2), (nkv * G, nkv, d, ps, window, entries, worst)
