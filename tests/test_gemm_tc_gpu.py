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
