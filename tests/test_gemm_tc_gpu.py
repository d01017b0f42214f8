"""The tcgen05 matrix product for few tokens against a float64 product of the same bfloat16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def check(M, N, K, out_dtype, splits=0, seed=0):
    from xinfer_b200 import kernels
    g = torch.Generator().manual_seed(seed + M + N + K)
    x = (torch.randn(M, K, generator=g)).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    took = kernels.gemm_skinny_tc(out, x, w, err, splits)
    torch.cuda.synchronize()
    assert int(err) == 0, kernels.describe_error(int(err))
    if not took:
        return False
    ref = x.double() @ w.double().t()
    scale = float(ref.abs().max())
    tol = 2e-6 * scale * K ** 0.5 + (0 if out_dtype == torch.float32 else scale * 2 ** -8)
    diff = (out.double() - ref).abs().max().item()
    assert diff <= tol, (M, N, K, out_dtype, splits, diff, tol)
    return True


@pytest.mark.parametrize("M", [1, 5, 8, 16, 17, 64, 100, 256])
@pytest.mark.parametrize("N,K", [(128, 64), (100, 72), (384, 4096), (4096, 1000), (331, 200)])
def test_shapes(M, N, K):
    assert check(M, N, K, torch.bfloat16)


@pytest.mark.parametrize("splits", [1, 2, 3, 4, 8])
def test_split_k_through_the_cluster(splits):
    assert check(8, 512, 4096, torch.bfloat16, splits)
    assert check(33, 200, 12288, torch.float32, splits)


def test_float32_output_and_model_shapes():
    for M, N, K in [(1, 6144, 4096), (8, 4096, 12288), (64, 24576, 4096), (3, 151936, 1024)]:
        assert check(M, N, K, torch.float32)


def test_refuses_what_it_cannot_do():
    assert not check(4, 64, 60, torch.bfloat16)      # K not a multiple of 8
    assert not check(4, 64, 32, torch.bfloat16)      # K below one tile
    assert not check(300, 64, 128, torch.bfloat16)   # too many tokens


# ---- tiles finished inside the product ---------------------------------------------------------------
@pytest.mark.parametrize("splits", [0, 1, 2, 4])
@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (8, 12288, 4096), (5, 200, 136), (32, 3072, 1024), (17, 100, 4096), (3, 88, 320)])
def test_gate_finished_in_the_product_equals_the_two_kernels(M, I, K, splits):
    """silu(gate) * up from the packed projection's kernel: bit for bit what the product followed by
    the gate kernel gives, at widths that are and are not multiples of the tile's 64 features."""
    from xinfer_b200 import kernels
    g = torch.Generator().manual_seed(M + I + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_skinny_tc(gu, x, w, err, splits)
    two = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    kernels.swiglu(two, gu)
    one = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_skinny_swiglu(one, x, w, err, splits)
    torch.cuda.synchronize()
    assert int(err) == 0, kernels.describe_error(int(err))
    assert torch.equal(one, two)
    # and both follow the plain formula on a float64 product of the same inputs
    ref = x.double() @ w.double().t()
    gate, up = ref[:, :I], ref[:, I:]
    want = gate / (1 + torch.exp(-gate)) * up
    scale = float(ref.abs().max())
    assert (one.double() - want).abs().max() <= 3 * 2 ** -8 * max(scale, 1.0) * max(scale, 1.0)


@pytest.mark.parametrize("splits", [0, 1, 2, 8])
@pytest.mark.parametrize("M,nh,nkv,K,inter,norm", [(1, 4, 2, 256, False, True), (8, 32, 8, 4096, False, True), (5, 3, 1, 136, True, True),
                                                  (32, 16, 8, 1024, False, False), (23, 2, 2, 512, False, True)])
def test_heads_finished_in_the_product_equal_the_two_kernels(M, nh, nkv, K, inter, norm, splits):
    """q/k norm, rotation and the cache write from the packed q/k/v projection's kernel: bit for bit what
    the product followed by the head kernel gives; no other cache slot is touched."""
    from xinfer_b200 import kernels
    import numpy as np
    d, ps, num_pages, max_pos, eps = 128, 4, 40, 96, 1e-6
    g = torch.Generator().manual_seed(M + nh + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((nh + 2 * nkv) * d, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    qw = (torch.randn(d, generator=g) * 0.2 + 1).to(DEV) if norm else None
    kw = (torch.randn(d, generator=g) * 0.2 + 1).to(DEV) if norm else None
    inv = torch.tensor((1.0 / 10000.0 ** (np.arange(0, d, 2) / d)).astype(np.float32), device=DEV)
    cos, sin = torch.empty(max_pos, d // 2, device=DEV), torch.empty(max_pos, d // 2, device=DEV)
    kernels.rope_table(cos, sin, inv)
    # requests: token t belongs to request t % 3 (the last one is padding when there are more than four)
    rng = np.random.default_rng(M)
    reqs = [t % 3 for t in range(M)]
    starts = {0: 7, 1: 0, 2: 30}
    seen = {0: 0, 1: 0, 2: 0}
    pos = []
    for r in reqs:
        pos.append(starts[r] + seen[r])
        seen[r] += 1
    if M > 4:
        reqs[-1] = -1     # a padding token: q is written, nothing is cached
    stride = 24
    table = rng.permutation(num_pages)[:3 * 12].reshape(3, 12)
    full = np.full((3, stride), -1, np.int32)
    full[:, :12] = table
    to = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    pos_d, req_d, table_d = to(pos), to(reqs), to(full.reshape(-1))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)

    def caches():
        k = torch.zeros(num_pages, nkv, ps, d, dtype=torch.bfloat16, device=DEV)
        return k, torch.zeros_like(k)

    qkv = torch.empty(M, (nh + 2 * nkv) * d, dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_skinny_tc(qkv, x, w, err, splits)
    k2, v2 = caches()
    q2 = torch.empty(M, nh, d, dtype=torch.bfloat16, device=DEV)
    kernels.qk_norm_rope_write(q2, k2, v2, qkv, qw, kw, cos, sin, pos_d, req_d, table_d, stride, nh, nkv, d, d, inter, eps, True, err)
    k1, v1 = caches()
    q1 = torch.full((M, nh, d), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_skinny_qkv(q1, k1, v1, x, w, qw, kw, cos, sin, pos_d, req_d, table_d, stride, nh, nkv, d, d, inter, eps,
                                   True, err, splits)
    torch.cuda.synchronize()
    assert int(err) == 0, kernels.describe_error(int(err))
    assert torch.equal(q1, q2) and torch.equal(k1, k2) and torch.equal(v1, v2)
    live = sum(1 for r in reqs if r >= 0)
    assert int(k1.float().abs().sum(-1).ne(0).sum()) == live * nkv
    # a page outside the pool is flagged and skipped
    bad = table_d.clone()
    bad[pos[0] // ps] = num_pages + 2
    assert kernels.gemm_skinny_qkv(q1, k1, v1, x, w, qw, kw, cos, sin, pos_d, req_d, bad, stride, nh, nkv, d, d, inter, eps,
                                   True, err, splits)
    torch.cuda.synchronize()
    assert int(err) == kernels.ERR_BAD_PAGE
    assert torch.equal(k1, k2)


def test_heads_of_other_widths_are_left_to_the_two_kernels():
    from xinfer_b200 import kernels
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(4 * 64, 64, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(2, 2, 64, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(4, 1, 4, 64, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(8, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert not kernels.gemm_skinny_qkv(q, k, k.clone(), x, w, None, None, None, None, z, z, z, 4, 2, 1, 64, 0, False, 1e-6, True, err)
