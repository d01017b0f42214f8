"""Python faces of the CUDA kernels.  Each wrapper checks devices, dtypes, shapes and contiguity,
launches on the current torch stream and raises on a launch error.  Nothing here computes on the
CPU or through a library: a missing extension or a CPU tensor is an error.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np
import torch

from .native import kernels_lib

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    """The checks every wrapper makes on its tensors; the message is only put together on failure
    (these run a few thousand times in a step of a small model)."""
    try:
        ok = t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype)
    except AttributeError:
        ok = False
    if ok and shape is not None:
        ts = t.shape
        if len(ts) != len(shape):
            ok = False
        else:
            for want, have in zip(shape, ts):
                if want is not None and want != have:
                    ok = False
                    break
    if not ok:
        _need_failed(t, name, dtype, shape)


def _need_failed(t, name, dtype, shape) -> None:
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


try:    # the raw handle of the current stream without building a Stream object for every launch
    _raw_stream, _device_index = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:  # pragma: no cover - other torch builds
    _raw_stream = None


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(_device_index())
    return torch.cuda.current_stream().cuda_stream


_launches = 0
_by_name: dict = {}

# Use the 16-byte-access bfloat16 kernels for norm / gate / q-k preparation where sizes allow;
# tests switch this off to compare them with the plain kernels.
vectorized = True
# From this many rows (tokens) on, the SiLU gate runs in its many-row form (blocks that stay on
# their SM and walk over rows with the next row's loads in flight); below, in the form shaped for a
# decode step's few rows.  The two forms give the same bits; tests move this bound to compare them.
many_rows = int(os.environ.get("XINFER_B200_MANY_ROWS", "256"))


def launch_count() -> int:
    """Kernels of this engine launched so far by this process (captured launches included)."""
    return _launches


def launch_counts() -> dict:
    """Launches so far by wrapper name (a copy): which kernels a step really ran."""
    return dict(_by_name)


def _ok(status: int, what: str, n: int = 1) -> None:
    global _launches
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status} at launch")
    _launches += n
    _by_name[what] = _by_name.get(what, 0) + n


# device-side error word -------------------------------------------------------------------------
ERR_BAD_TOKEN, ERR_BAD_PAGE, ERR_WAIT, ERR_BAD_ROW, ERR_SCRATCH, ERR_BAD_POSITION = 1, 2, 4, 8, 16, 32


def describe_error(word: int) -> str:
    parts = []
    if word & ERR_BAD_TOKEN:
        parts.append("a token id outside the vocabulary")
    if word & ERR_BAD_PAGE:
        parts.append("a block-table entry outside the page pool")
    if word & ERR_WAIT:
        parts.append("a bounded wait inside a kernel gave up")
    if word & ERR_BAD_ROW:
        parts.append("a requested row outside the step's tokens")
    if word & ERR_BAD_POSITION:
        parts.append("a token position outside the position table")
    if word & ERR_SCRATCH:
        parts.append("scratch memory that a kernel must find zeroed was not")
    return "; ".join(parts) or "no error"


# ---- wrappers --------------------------------------------------------------------------------------
def embedding(out, table, ids, err, sampled=None, scale=None):
    """out[t] = table[ids[t]] (times ``scale``, if given, rounded to the table's dtype); an id -1 - i
    is replaced on the device by ``sampled[i]`` (int32 ids a sampler left there)."""
    T, H = out.shape
    _need(out, "out", table.dtype, (T, H))
    _need(table, "table", None, (None, H))
    _need(ids, "ids", torch.int32)
    if ids.numel() < T:
        raise KernelError(f"ids holds {ids.numel()} entries for {T} tokens")
    _need(err, "err", torch.int32)
    if sampled is not None:
        _need(sampled, "sampled", torch.int32)
    _ok(kernels_lib().xb_embedding(dtype_code(table.dtype), out.data_ptr(), table.data_ptr(), ids.data_ptr(),
                                   _ptr(sampled), sampled.numel() if sampled is not None else 0,
                                   T, H, table.shape[0], 1.0 if scale is None else float(scale), err.data_ptr(),
                                   _stream()), "embedding")


def logits_post(logits, scale=None, softcap=None):
    """In place on float32 logits: ``logits *= scale``, then ``logits = softcap * tanh(logits / softcap)``."""
    _need(logits, "logits", torch.float32)
    _ok(kernels_lib().xb_logits_post(logits.data_ptr(), logits.numel(), 1.0 if scale is None else float(scale),
                                     0.0 if softcap is None else float(softcap), _stream()), "logits_post")


def rmsnorm(out, x, weight, eps, err, *, branch=None, sum_out=None, rows=None, weight_offset=0.0):
    """out = norm(s) * (offset + w) with s = x (+ branch), optionally gathered at ``rows``;
    ``sum_out`` receives s (it may be x itself when no rows are given)."""
    dim = x.shape[-1]
    n = out.shape[0]
    _need(x, "x", None, (None, dim))
    _need(out, "out", x.dtype, (n, dim))
    _need(weight, "weight", torch.float32, (dim,))
    if branch is not None:
        _need(branch, "branch", x.dtype, tuple(x.shape))
    if sum_out is not None:
        _need(sum_out, "sum_out", x.dtype, (n, dim))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError(f"rows holds {rows.numel()} entries for {n} output rows")
    elif n != x.shape[0]:
        raise KernelError(f"out has {n} rows, x has {x.shape[0]} and no row list was given")
    if vectorized and x.dtype == torch.bfloat16 and dim % 8 == 0 and dim <= 32768:
        _ok(kernels_lib().xb_rmsnorm_bf16(out.data_ptr(), _ptr(sum_out), x.data_ptr(), _ptr(branch), _ptr(rows),
                                          weight.data_ptr(), n, dim, x.shape[0], float(eps), float(weight_offset),
                                          err.data_ptr(), _stream()), "rmsnorm_bf16")
        return
    _ok(kernels_lib().xb_rmsnorm(dtype_code(x.dtype), out.data_ptr(), _ptr(sum_out), x.data_ptr(), _ptr(branch),
                                 _ptr(rows), weight.data_ptr(), n, dim, x.shape[0], float(eps),
                                 float(weight_offset), err.data_ptr(), _stream()), "rmsnorm")


def add(out, x, branch):
    _need(x, "x")
    _need(branch, "branch", x.dtype, tuple(x.shape))
    _need(out, "out", x.dtype, tuple(x.shape))
    _ok(kernels_lib().xb_add(dtype_code(x.dtype), out.data_ptr(), x.data_ptr(), branch.data_ptr(), x.numel(), _stream()), "add")


def gemm_plain(out, a, w):
    """out[M, N] = a[M, K] . w[N, K]^T with float32 FMA accumulation (no tensor cores)."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", None, (M, K))
    _need(w, "w", None, (N, K))
    _need(out, "out", None, (M, N))
    _ok(kernels_lib().xb_gemm_plain(dtype_code(a.dtype), dtype_code(w.dtype), dtype_code(out.dtype), out.data_ptr(),
                                    a.data_ptr(), w.data_ptr(), M, N, K, _stream()), "gemm_plain")


def rope_table(cos_t, sin_t, inv_freq):
    max_pos, half = cos_t.shape
    _need(cos_t, "cos", torch.float32, (max_pos, half))
    _need(sin_t, "sin", torch.float32, (max_pos, half))
    _need(inv_freq, "inv_freq", torch.float32, (half,))
    _ok(kernels_lib().xb_rope_table(cos_t.data_ptr(), sin_t.data_ptr(), inv_freq.data_ptr(), max_pos, half, _stream()), "rope_table")


def qk_norm_rope_write(q_out, k_cache, v_cache, qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token,
                       block_table, table_stride, nh, nkv, d, rot, interleaved, eps, write_kv, err):
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (nh + 2 * nkv) * d))
    _need(q_out, "q_out", qkv.dtype, (T, nh, d))
    if write_kv:
        _need(k_cache, "k_cache", qkv.dtype, (None, nkv, None, d))
        _need(v_cache, "v_cache", qkv.dtype, tuple(k_cache.shape))
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    page_size = k_cache.shape[2] if k_cache is not None else 1
    for name, w_ in (("q_norm", q_w), ("k_norm", k_w)):
        if w_ is not None:
            _need(w_, name, torch.float32, (d,))
    max_pos = 0
    if cos_t is not None:
        _need(cos_t, "cos", torch.float32, (None, rot // 2))
        _need(sin_t, "sin", torch.float32, tuple(cos_t.shape))
        max_pos = cos_t.shape[0]
    if (vectorized and qkv.dtype == torch.bfloat16 and d % 16 == 0 and d <= 512
            and (cos_t is None or interleaved or rot == d)):
        _ok(kernels_lib().xb_qk_norm_rope_write_bf16(
            q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), qkv.data_ptr(), _ptr(q_w), _ptr(k_w), _ptr(cos_t), _ptr(sin_t),
            positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride), T, nh, nkv, d, rot,
            int(bool(interleaved)), page_size, num_pages, max_pos, float(eps), int(bool(write_kv)), err.data_ptr(),
            _stream()), "qk_norm_rope_write_bf16")
        return
    _ok(kernels_lib().xb_qk_norm_rope_write(
        dtype_code(qkv.dtype), q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), qkv.data_ptr(), _ptr(q_w), _ptr(k_w),
        _ptr(cos_t), _ptr(sin_t), positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(),
        int(table_stride), T, nh, nkv, d, rot, int(bool(interleaved)), page_size, num_pages, max_pos, float(eps),
        int(bool(write_kv)), err.data_ptr(), _stream()), "qk_norm_rope_write")


def attention_plain(out, q, k_cache, v_cache, positions, req_of_token, block_table, table_stride, window, scale, err):
    T, nh, d = q.shape
    _need(q, "q", None, (T, nh, d))
    _need(out, "out", q.dtype, (T, nh, d))
    _need(k_cache, "k_cache", q.dtype, (None, None, None, d))
    _need(v_cache, "v_cache", q.dtype, tuple(k_cache.shape))
    num_pages, nkv, page_size, _ = k_cache.shape
    if nh % nkv:
        raise KernelError(f"{nh} query heads do not divide into {nkv} key/value heads")
    if d > 512:
        raise KernelError(f"head size {d} is larger than the plain attention kernel's limit of 512")
    _ok(kernels_lib().xb_attention_plain(
        dtype_code(q.dtype), out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
        req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride), T, nh, nkv, d, page_size, num_pages,
        int(window or 0), float(scale), err.data_ptr(), _stream()), "attention_plain")


def swiglu(out, gate_up):
    T, two_i = gate_up.shape
    _need(gate_up, "gate_up", None, (T, two_i))
    _need(out, "out", gate_up.dtype, (T, two_i // 2))
    if vectorized and gate_up.dtype == torch.bfloat16 and two_i % 16 == 0:
        if T >= many_rows:
            _ok(kernels_lib().xb_swiglu_rows_bf16(out.data_ptr(), gate_up.data_ptr(), T, two_i // 2, _stream()), "swiglu_rows_bf16")
            return
        _ok(kernels_lib().xb_swiglu_bf16(out.data_ptr(), gate_up.data_ptr(), T, two_i // 2, _stream()), "swiglu_bf16")
        return
    _ok(kernels_lib().xb_swiglu(dtype_code(gate_up.dtype), out.data_ptr(), gate_up.data_ptr(), T, two_i // 2, _stream()), "swiglu")


def widen_bf16(out, x):
    _need(x, "x", torch.bfloat16)
    _need(out, "out", torch.float32, tuple(x.shape))
    _ok(kernels_lib().xb_widen_bf16(out.data_ptr(), x.data_ptr(), x.numel(), _stream()), "widen_bf16")


SAMPLE_PARAMS = np.dtype([
    ("temperature", np.float32), ("top_k", np.int32), ("top_p", np.float32),
    ("seed_lo", np.uint32), ("seed_hi", np.uint32), ("draw", np.uint32),
    ("frequency_penalty", np.float32), ("presence_penalty", np.float32),
    ("history_offset", np.int32), ("history_len", np.int32),
])


def sample_scratch_bytes(capacity: int) -> int:
    """Bytes of scratch for a sampler that sees at most ``capacity`` rows in one call."""
    return int(kernels_lib().xb_sample_scratch_bytes(int(capacity)))


def sample(out_tokens, logits, params_dev, history_dev, apply_penalties: bool, scratch, err_word=None, *,
           capacity: Optional[int] = None):
    """One token per logits row into ``out_tokens``; with ``err_word`` (a device int32) its value is
    written to ``out_tokens[R]``, so that one copy brings tokens and error word to the host.
    ``scratch``: uint8 device buffer of ``sample_scratch_bytes(capacity)``, zero before its first use
    and laid out by ``capacity`` (default: the rows of this call): calls that share a buffer must
    give the same capacity, whatever their rows."""
    R, V = logits.shape
    capacity = R if capacity is None else int(capacity)
    if R > capacity:
        raise KernelError(f"{R} rows exceed the sampler scratch's capacity {capacity}")
    _need(logits, "logits", torch.float32, (R, V))
    _need(out_tokens, "out_tokens", torch.int32)
    _need(params_dev, "params", torch.uint8)
    lib = kernels_lib()
    if lib.xb_sample_params_size() != SAMPLE_PARAMS.itemsize:
        raise KernelError("the sampler's parameter record differs between Python and CUDA")
    _need(scratch, "scratch", torch.uint8)
    if (params_dev.numel() < R * SAMPLE_PARAMS.itemsize or out_tokens.numel() < R + (err_word is not None)
            or scratch.numel() < lib.xb_sample_scratch_bytes(capacity)):
        raise KernelError("sampler buffers are smaller than the number of rows")
    _ok(lib.xb_sample(out_tokens.data_ptr(), logits.data_ptr(), params_dev.data_ptr(), _ptr(history_dev), R, capacity, V,
                      int(bool(apply_penalties)), scratch.data_ptr(), _ptr(err_word), _stream()), "sample",
        2 if apply_penalties else 1)


# ---- bfloat16 attention on tensor cores ------------------------------------------------------------
def attn_tiled_supported(dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def attn_prefill_queries(head_dim: int, warps: int = 8) -> int:
    """Queries one CTA of the prefill kernel takes (256-wide heads always use 4 warps)."""
    return 16 * (4 if head_dim > 128 else warps)


def attn_prefill_bf16(out, q, k_cache, v_cache, q_start, start_pos, num_entries, block_table, table_stride,
                      window, scale, dec_max, tiles, max_context, err, warps: int = 8):
    """Portions of more than ``dec_max`` tokens; ``tiles`` = sum over them of
    ceil(tokens / attn_prefill_queries(head_dim, warps)); ``max_context`` = their longest
    start + tokens."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    num_pages, nkv, ps, _ = k_cache.shape
    if not attn_tiled_supported(q.dtype, d) or nh % nkv:
        raise KernelError(f"tiled attention needs bfloat16, a head size in steps of 16 up to 256 and heads divisible "
                          f"by key/value heads; got head size {d}, {nh}/{nkv} heads")
    _ok(kernels_lib().xb_attn_prefill_bf16(
        out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q_start.data_ptr(), start_pos.data_ptr(),
        int(num_entries), block_table.data_ptr(), int(table_stride), nh, nkv, d, ps, num_pages, int(window or 0),
        float(scale), int(dec_max), int(tiles), int(max_context), 4 if d > 128 else int(warps), err.data_ptr(),
        _stream()), "attn_prefill_bf16")


def attn_decode_bf16(out, part_o, part_ml, q, k_cache, v_cache, positions, req_of_token, q_start, num_entries,
                     block_table, table_stride, window, scale, dec_max, direct, split, num_splits, tokens, err, tickets=None):
    """Tokens of portions of at most ``dec_max`` tokens (``tokens`` of them); keys are cut into
    ``num_splits`` ranges of ``split`` positions (a multiple of 64).  ``tickets``: int32 scratch of
    tokens * kv_heads * ceil(group / 16) zeros (left zero), needed with ``num_splits`` > 1.  ``part_o`` /
    ``part_ml``: float32 scratch of at least tokens*heads*num_splits*head_dim and
    tokens*heads*num_splits*2 elements when ``num_splits`` > 1."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    num_pages, nkv, ps, _ = k_cache.shape
    if not attn_tiled_supported(q.dtype, d) or nh % nkv:
        raise KernelError(f"tiled attention needs bfloat16, a head size in steps of 16 up to 256 and heads divisible "
                          f"by key/value heads; got head size {d}, {nh}/{nkv} heads")
    if tokens > 65535:
        raise KernelError(f"{tokens} small-portion tokens exceed the decode kernel's grid limit of 65535")
    if num_splits > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < tokens * nh * num_splits * d or part_ml.numel() < tokens * nh * num_splits * 2:
            raise KernelError("attention scratch buffers are too small for the number of key ranges")
        _need(tickets, "tickets", torch.int32)
        if tickets.numel() < tokens * nkv * ((nh // nkv + 15) // 16):
            raise KernelError("the attention ticket buffer is too small")
    _ok(kernels_lib().xb_attn_decode_bf16(
        out.data_ptr(), _ptr(part_o), _ptr(part_ml), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        positions.data_ptr(), req_of_token.data_ptr(), q_start.data_ptr(), int(num_entries), block_table.data_ptr(),
        int(table_stride), nh, nkv, d, ps, num_pages, int(window or 0), float(scale), int(dec_max), int(bool(direct)),
        int(split), int(num_splits), int(tokens), _ptr(tickets), err.data_ptr(), _stream()), "attn_decode_bf16")


ERR_NOT_SUPPORTED = 801  # cudaErrorNotSupported


def attn_decode_plan_size(tokens: int, ctas: int, kv_heads: int) -> int:
    return int(kernels_lib().xb_attn_decode_plan_size(int(tokens), int(ctas), int(kv_heads)))


def attn_decode_plan(plan, positions, req_of_token, q_start, num_entries, window, dec_max, direct, tokens, min_keys,
                     ctas, kv_heads, err) -> bool:
    """Decide how the attention of the step's ``tokens`` small tokens is shared out (pieces of about
    1 / ``ctas`` of all keys, at least ``min_keys`` each) and write it to ``plan`` (int32,
    ``attn_decode_plan_size`` elements).  It must run before the step's first kernel when
    ``attn_decode_tc`` is to overlap with its predecessor.  False: more tokens than a plan takes."""
    _need(plan, "plan", torch.int32)
    if plan.numel() < attn_decode_plan_size(tokens, ctas, kv_heads):
        raise KernelError("the attention plan buffer is too small")
    rc = kernels_lib().xb_attn_decode_plan(plan.data_ptr(), positions.data_ptr(), req_of_token.data_ptr(), q_start.data_ptr(),
                                           int(num_entries), int(window or 0), int(dec_max), int(bool(direct)), int(tokens),
                                           int(min_keys), int(ctas), int(kv_heads), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "attn_decode_plan")
    return True


def attn_decode_tc(out, part_o, part_ml, q, k_cache, v_cache, plan, block_table, table_stride, scale, dec_max,
                   splits_max, tokens, ctas, err, tickets=None, overlap: bool = True) -> bool:
    """The step's small tokens on tcgen05 tensor cores with TMA-fed pages, shared out as ``plan``
    says (``attn_decode_plan`` with the same tokens, ctas and kv heads).  A token and head in several
    pieces is merged through ``part_o`` / ``part_ml`` (float32, tokens*heads*splits_max*head_dim
    and tokens*heads*splits_max*2 elements) and ``tickets`` (int32, tokens * kv_heads zeros, left
    zero); ``decode_tc_splits_max`` gives the ``splits_max`` that is always enough.  ``overlap``:
    start while the kernel before drains - only with a plan made before the step's first kernel.
    Returns False, having done nothing, for shapes the kernel does not take (a head size over
    128, a page size that is no power of two >= 8, more than 16 query heads per key/value head)."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(plan, "plan", torch.int32)
    num_pages, nkv, ps, _ = k_cache.shape
    if nh % nkv or d % 16:
        raise KernelError(f"tiled attention needs a head size in steps of 16 and heads divisible by key/value heads; "
                          f"got head size {d}, {nh}/{nkv} heads")
    if plan.numel() < attn_decode_plan_size(tokens, ctas, nkv):
        raise KernelError("the attention plan buffer is too small")
    if splits_max > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < tokens * nh * splits_max * d or part_ml.numel() < tokens * nh * splits_max * 2:
            raise KernelError("attention scratch buffers are too small for the number of pieces per token")
        _need(tickets, "tickets", torch.int32)
        if tickets.numel() < tokens * nkv:
            raise KernelError("the attention ticket buffer is too small")
    rc = kernels_lib().xb_attn_decode_tc(
        out.data_ptr(), _ptr(part_o), _ptr(part_ml), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), plan.data_ptr(),
        block_table.data_ptr(), int(table_stride), T, nh, nkv, d, ps, num_pages, float(scale), int(dec_max),
        int(splits_max), int(tokens), int(ctas), _ptr(tickets), int(bool(overlap)), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "attn_decode_tc")
    return True


def decode_tc_splits_max(ctas: int, kv_heads: int, bound: int, min_keys: int) -> int:
    """Most pieces one token of ``attn_decode_tc`` can be cut into when no context is longer than
    ``bound``: a (token, head) pair holds at most 1 / kv_heads of all tiles (so it gets at most
    ctas / kv_heads shares), and a piece at least ``min_keys``."""
    tiles = (max(int(bound), 1) + 63) // 64
    per = max(int(min_keys) // 64, 1)
    return max(1, min(int(ctas) // int(kv_heads) + 1, tiles // per + 1))


# ---- matrix product for few tokens on tcgen05 tensor cores ---------------------------------------------


def gemm_skinny_tc(out, x, w, err, splits: int = 0) -> bool:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 256 with TMA-fed tcgen05 MMAs (bfloat16 in, float32
    accumulation; ``out`` bfloat16 or float32).  Returns False, having done nothing, for shapes the
    kernel does not take (K not a multiple of 8, K < 64, M > 256)."""
    M, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16, (M, K))
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", None, (M, N))
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"out must be bfloat16 or float32, not {out.dtype}")
    rc = kernels_lib().xb_gemm_skinny_tc(out.data_ptr(), int(out.dtype == torch.float32), x.data_ptr(), w.data_ptr(),
                                         M, N, K, int(splits), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "gemm_skinny_tc")
    return True


def gemm_skinny_swiglu(out, x, w_gate_up, err, splits: int = 0) -> bool:
    """out[M, I] = silu(x . Wg^T) * (x . Wu^T) for w_gate_up = [Wg; Wu] of [2 I, K]: the packed gate/up
    product of few tokens and the SiLU gate in one kernel, with the values that ``gemm_skinny_tc``
    followed by ``swiglu`` gives.  Returns False, having done nothing, for shapes it does not take."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x, "x", torch.bfloat16, (M, K))
    _need(w_gate_up, "w_gate_up", torch.bfloat16, (2 * I, K))
    _need(out, "out", torch.bfloat16, (M, I))
    rc = kernels_lib().xb_gemm_skinny_swiglu(out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), M, I, K, int(splits),
                                             err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "gemm_skinny_swiglu")
    return True


def gemm_skinny_qkv(q_out, k_cache, v_cache, x, w_qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token, block_table,
                    table_stride, nh, nkv, d, rot, interleaved, eps, write_kv, err, splits: int = 0) -> bool:
    """The packed q/k/v product of few tokens finished per head in the same kernel: what
    ``gemm_skinny_tc`` followed by ``qk_norm_rope_write`` gives (q to ``q_out``, k and v into their
    pages).  Heads must be 128 wide; returns False, having done nothing, for what it does not take."""
    M, K = x.shape
    _need(x, "x", torch.bfloat16, (M, K))
    _need(w_qkv, "w_qkv", torch.bfloat16, ((nh + 2 * nkv) * d, K))
    _need(q_out, "q_out", torch.bfloat16, (M, nh, d))
    if write_kv:
        _need(k_cache, "k_cache", torch.bfloat16, (None, nkv, None, d))
        _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    page_size = k_cache.shape[2] if k_cache is not None else 1
    for name, w_ in (("q_norm", q_w), ("k_norm", k_w)):
        if w_ is not None:
            _need(w_, name, torch.float32, (d,))
    max_pos = 0
    if cos_t is not None:
        _need(cos_t, "cos", torch.float32, (None, rot // 2))
        _need(sin_t, "sin", torch.float32, tuple(cos_t.shape))
        max_pos = cos_t.shape[0]
    rc = kernels_lib().xb_gemm_skinny_qkv(
        q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), x.data_ptr(), w_qkv.data_ptr(), M, K, int(splits), _ptr(q_w), _ptr(k_w),
        _ptr(cos_t), _ptr(sin_t), positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride),
        nh, nkv, d, rot, int(bool(interleaved)), page_size, num_pages, max_pos, float(eps), int(bool(write_kv)),
        err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "gemm_skinny_qkv")
    return True


PREFILL_TC_MAX_CTAS = 148   # one CTA of the tcgen05 prefill kernel per SM


def attn_prefill_work(counts, starts, dec_max: int, window, heads: int, kv_heads: int, max_ctas: int = PREFILL_TC_MAX_CTAS,
                      host_buffer=None):
    """The work list of ``attn_prefill_tc`` for a step whose entries bring ``counts`` tokens after
    ``starts`` cached ones (host arrays): the portions of more than ``dec_max`` tokens cut into items of
    128 queries of a pair of query heads (of single heads where pairs would be too few) and shared out among at most ``max_ctas`` CTAs, longest first
    onto the least loaded.  ``host_buffer(n)``: gives a pinned int32 tensor of at least n elements to write
    into (default: a fresh one).  Returns (pinned int32 host tensor, number of CTAs); no CTAs: nothing to do."""
    from .native import host_lib
    counts = np.ascontiguousarray(counts, dtype=np.int32)
    starts = np.ascontiguousarray(starts, dtype=np.int32)
    tiles = int(((counts[counts > dec_max] + 127) // 128).sum())
    cap = max_ctas + 1 + 4 * tiles * heads + 4
    host = host_buffer(cap) if host_buffer is not None else torch.empty(cap, dtype=torch.int32).pin_memory()
    ctas = ctypes.c_int(0)
    used = host_lib().xb_attn_prefill_work(len(counts), counts.ctypes.data, starts.ctypes.data, int(dec_max), int(window or 0),
                                           int(heads), int(kv_heads), int(max_ctas), host.data_ptr(), cap, ctypes.byref(ctas))
    if used < 0:
        raise KernelError("the prefill work list does not fit its buffer")
    return host[:max(int(used), 1)], int(ctas.value)


def attn_prefill_tc(out, q, k_cache, v_cache, q_start, start_pos, block_table, table_stride, window, scale, work, ctas, err) -> bool:
    """Prefill attention on tcgen05 (TMA-fed; scores, probabilities and accumulators in tensor memory):
    128 queries of two query heads of a key/value head per work item; ``work`` (int32, on the device)
    and ``ctas`` come from ``attn_prefill_work`` for the same step, heads and window.  Returns False,
    having done nothing, for sizes it does not take (head size over 128, page size not a power of two
    from 8)."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(work, "work", torch.int32)
    num_pages, nkv, ps, _ = k_cache.shape
    if ctas <= 0:
        return True
    if work.numel() < ctas + 1:
        raise KernelError("the prefill work list is shorter than its table of CTAs")
    rc = kernels_lib().xb_attn_prefill_tc(
        out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q_start.data_ptr(), start_pos.data_ptr(),
        block_table.data_ptr(), int(table_stride), T, nh, nkv, d, ps, num_pages, int(window or 0), float(scale),
        work.data_ptr(), int(ctas), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "attn_prefill_tc")
    return True
