"""Which hand-written bfloat16 matrix-product kernel takes a given shape, if any.

``try_fast(out, x, w)`` runs one of the engine's own tensor-core kernels and returns True, or
returns False to leave the shape to the library product.  Steps with few tokens (decode) are
bound by reading the weights once; they go to the TMA-fed tcgen05 kernel that streams W through
a ring of shared-memory stages and shares K over a thread-block cluster.
"""
from __future__ import annotations

import torch

from .. import kernels

# most tokens for which the streaming kernel is used (above, the library product is faster)
SKINNY_MAX_TOKENS = 32

_enabled = True
_err = {}


def set_enabled(flag: bool) -> None:
    global _enabled
    _enabled = bool(flag)


def _err_word(device) -> torch.Tensor:
    e = _err.get(device)
    if e is None:
        e = torch.zeros(1, dtype=torch.int32, device=device)
        _err[device] = e
    return e


def try_fast(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, err: torch.Tensor = None) -> bool:
    if not _enabled:
        return False
    M, K = x.shape
    if M <= SKINNY_MAX_TOKENS and K % 8 == 0 and K >= 64:
        return kernels.gemm_skinny_tc(out, x, w, err if err is not None else _err_word(x.device))
    return False
