"""Dense projection ``y = x . W^T`` with ``W`` stored ``[out, in]`` (src/models/layers/linear.rs:76-124).

float32: the engine's own FMA kernel (true 32-bit, no tensor-core mode).  bfloat16: the engine's
tcgen05 kernel for steps of few tokens, else the library matrix product, as in the reference
(cuBLAS through its tensor library); see ``gemm_backend``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


def linear(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] . weight[N, K]^T.  ``out`` may be float32 for bfloat16 inputs.
    ``err``: the step's device error word (kernels with bounded waits report there)."""
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        from . import gemm_backend
        if gemm_backend.try_fast(out, x, weight, err):
            return out
        if out.dtype == torch.bfloat16:
            torch.mm(x, weight.t(), out=out)
        else:
            tmp = torch.mm(x, weight.t())
            kernels.widen_bf16(out, tmp)
        return out
    kernels.gemm_plain(out, x, weight)
    return out
