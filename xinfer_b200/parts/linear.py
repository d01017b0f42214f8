"""Dense projection ``y = x . W^T`` with ``W`` stored ``[out, in]`` (src/models/layers/linear.rs:76-124).

float32: the engine's own FMA kernel (true 32-bit, no tensor-core mode).  bfloat16: the engine's
tcgen05 kernel for steps of few tokens, else the library matrix product, as in the reference
(cuBLAS through its tensor library); see ``gemm_backend``.  Both write float32 accumulators
straight into a float32 ``out`` (the logits).
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
            # float32 out of the library product too: its accumulators are never rounded to bfloat16, so a
            # row's logits are the same numbers whichever kernel the size of the batch selects
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        return out
    kernels.gemm_plain(out, x, weight)
    return out
