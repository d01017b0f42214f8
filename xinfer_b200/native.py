"""Loads the two native libraries (building them at first use) and declares their C signatures.

There is no fallback: if the kernels cannot be built or loaded the engine raises.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import (POINTER, c_char_p, c_float, c_int, c_int32, c_longlong, c_void_p)

_lock = threading.Lock()
_host = None
_kernels = None

_I32P = POINTER(c_int32)
_I64P = POINTER(c_longlong)


def host_lib():
    """Host runtime: cache manager, scheduler, step metadata assembly (no CUDA needed)."""
    global _host
    with _lock:
        if _host is None:
            from .csrc.build import build_host
            lib = ctypes.CDLL(build_host())
            _declare_host(lib)
            _host = lib
    return _host


def kernels_lib():
    """CUDA kernels for sm_100a."""
    global _kernels
    with _lock:
        if _kernels is None:
            from .csrc.build import build_kernels
            lib = ctypes.CDLL(build_kernels())
            _declare_kernels(lib)
            _kernels = lib
    return _kernels


def _sig(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes


def _declare_host(lib):
    _sig(lib, "xb_cm_create", c_void_p, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), c_int])
    _sig(lib, "xb_cm_destroy", None, [c_void_p])
    for name in ("xb_cm_open", "xb_cm_live_requests"):
        _sig(lib, name, c_int, [c_void_p])
    for name in ("xb_cm_close", "xb_cm_is_live", "xb_cm_length", "xb_cm_free_pages"):
        _sig(lib, name, c_int, [c_void_p, c_int])
    for name in ("xb_cm_can_extend", "xb_cm_extend", "xb_cm_advance", "xb_cm_table_size"):
        _sig(lib, name, c_int, [c_void_p, c_int, c_int])
    _sig(lib, "xb_cm_copy_table", c_int, [c_void_p, c_int, c_int, _I32P, c_int])
    _sig(lib, "xb_cm_consistent", c_int, [c_void_p, c_char_p, c_int])
    _sig(lib, "xb_attn_prefill_work", c_longlong,
         [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p])
    _sig(lib, "xb_cm_log_freed", None, [c_void_p, c_int])
    _sig(lib, "xb_cm_drain_freed", c_int, [c_void_p, c_void_p, c_void_p, c_int])
    _sig(lib, "xb_assemble", c_longlong,
         [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
          c_void_p, c_void_p, c_longlong, c_void_p])
    _sig(lib, "xb_sched_create", c_void_p, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int])
    _sig(lib, "xb_sched_destroy", None, [c_void_p])
    _sig(lib, "xb_sched_add", c_int, [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int])
    _sig(lib, "xb_sched_abort", c_int, [c_void_p, c_longlong])
    _sig(lib, "xb_sched_schedule", c_int,
         [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _sig(lib, "xb_sched_commit", None, [c_void_p, c_void_p, c_int])
    _sig(lib, "xb_sched_schedule_ahead", c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _sig(lib, "xb_sched_fail_steps", c_int, [c_void_p])
    _sig(lib, "xb_sched_drain_finished", c_int, [c_void_p, c_void_p, c_int])
    for name in ("xb_sched_num_waiting", "xb_sched_num_running", "xb_sched_preemptions"):
        _sig(lib, name, c_int, [c_void_p])
    for name in ("xb_sched_finish_reason", "xb_sched_output_length", "xb_sched_prompt_length",
                 "xb_sched_num_drawn", "xb_sched_release"):
        _sig(lib, name, c_int, [c_void_p, c_longlong])
    _sig(lib, "xb_sched_copy_output", c_int, [c_void_p, c_longlong, c_void_p, c_int])
    _sig(lib, "xb_sched_copy_tail", c_int, [c_void_p, c_longlong, c_void_p, c_int])


def _declare_kernels(lib):
    P, I, F, L = c_void_p, c_int, c_float, c_longlong
    _sig(lib, "xb_embedding", I, [I, P, P, P, P, I, I, I, I, F, P, P])
    _sig(lib, "xb_logits_post", I, [P, L, F, F, P])
    _sig(lib, "xb_rmsnorm", I, [I, P, P, P, P, P, P, I, I, I, F, F, P, P])
    _sig(lib, "xb_add", I, [I, P, P, P, L, P])
    _sig(lib, "xb_gemm_plain", I, [I, I, I, P, P, P, I, I, I, P])
    _sig(lib, "xb_rope_table", I, [P, P, P, I, I, P])
    _sig(lib, "xb_qk_norm_rope_write", I,
         [I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P])
    _sig(lib, "xb_attention_plain", I, [I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P])
    _sig(lib, "xb_swiglu", I, [I, P, P, I, I, P])
    _sig(lib, "xb_widen_bf16", I, [P, P, L, P])
    _sig(lib, "xb_sample", I, [P, P, P, P, I, I, I, I, P, P, P])
    _sig(lib, "xb_sample_scratch_bytes", c_longlong, [I])
    _sig(lib, "xb_sample_params_size", I, [])
    _sig(lib, "xb_rmsnorm_bf16", I, [P, P, P, P, P, P, I, I, I, F, F, P, P])
    _sig(lib, "xb_swiglu_bf16", I, [P, P, I, I, P])
    _sig(lib, "xb_qk_norm_rope_write_bf16", I,
         [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P])
    _sig(lib, "xb_swiglu_rows_bf16", I, [P, P, I, I, P])
    _sig(lib, "xb_attn_prefill_tc", I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, I, P, P])
    _sig(lib, "xb_gemm_skinny_tc", I, [P, I, P, P, I, I, I, I, P, P])
    _sig(lib, "xb_gemm_skinny_swiglu", I, [P, P, P, I, I, I, I, P, P])
    _sig(lib, "xb_gemm_skinny_qkv", I,
         [P, P, P, P, P, I, I, I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P])
    _sig(lib, "xb_attn_prefill_bf16", I, [P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, I, I, I, P, P])
    _sig(lib, "xb_attn_decode_bf16", I,
         [P, P, P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, I, I, I, I, P, P, P])
    _sig(lib, "xb_attn_decode_plan_size", c_longlong, [I, I, I])
    _sig(lib, "xb_attn_decode_plan", I, [P, P, P, P, I, I, I, I, I, I, I, I, P, P])
    _sig(lib, "xb_attn_decode_tc", I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, I, P, I, P, P])
