"""Which hand-written bfloat16 matrix-product kernel takes a given shape, if any.

``try_fast(out, x, w)`` runs one of the engine's own tensor-core kernels and returns True, or
returns False to leave the shape to the library product.  Steps with few tokens (decode) are
bound by reading the weights once; they go to the TMA-fed tcgen05 kernel that streams W through
a ring of shared-memory stages and shares K over a thread-block cluster.  The same kernel can
finish its tile in place of the kernel that would follow: ``try_fused_gate`` (the SiLU gate of a
packed gate/up projection) and ``try_fused_qkv`` (per-head q/k norm, rotation and cache write of
a packed q/k/v projection) return False where the separate kernels have to run.
"""
from __future__ import annotations

import torch

from .. import kernels

# most tokens for which the streaming kernel is used (above, the library product is faster)
SKINNY_MAX_TOKENS = 32

# Finish a tile inside the product where that replaces a kernel.  Off: measured on a B200 at the
# Qwen3-8B layer sizes, a decode step of 8 requests took 4 % longer with it.  Under programmatic
# dependent launch the small kernel between two large ones is where the next large kernel's blocks
# become resident and run their prologue (tensor memory, barriers, page tables, the first ring of
# weight tiles); without it that prologue waits for the product's blocks to leave and shows.
FUSE_EPILOGUES = False

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


def try_fused_gate(act: torch.Tensor, x: torch.Tensor, w_gate_up: torch.Tensor, err: torch.Tensor) -> bool:
    """act = silu(gate(x)) * up(x) in the kernel of the packed projection."""
    if not (_enabled and FUSE_EPILOGUES):
        return False
    M, K = x.shape
    if M <= SKINNY_MAX_TOKENS and K % 8 == 0 and K >= 64 and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
        return kernels.gemm_skinny_swiglu(act, x, w_gate_up, err)
    return False


def try_fused_qkv(q_out, k_cache, v_cache, x, w_qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token, block_table,
                  table_stride, nh, nkv, d, rot, interleaved, eps, write_kv, err) -> bool:
    """The packed q/k/v projection with its heads finished (norm, rotation, cache write) in the same kernel."""
    if not (_enabled and FUSE_EPILOGUES):
        return False
    M, K = x.shape
    if (M <= SKINNY_MAX_TOKENS and K % 8 == 0 and K >= 64 and d == 128 and x.dtype == torch.bfloat16
            and w_qkv.dtype == torch.bfloat16 and (cos_t is None or interleaved or rot == d)):
        return kernels.gemm_skinny_qkv(q_out, k_cache, v_cache, x, w_qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token,
                                       block_table, table_stride, nh, nkv, d, rot, interleaved, eps, write_kv, err)
    return False
