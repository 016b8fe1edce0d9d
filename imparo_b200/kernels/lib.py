"""Loads the native libraries (compiling them at first use) and declares their C entry points.

There is no other path: if the kernel library cannot be built or loaded, every GPU
operation raises.  The libraries live in the source tree (imparo_b200/_build/).
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, c_float, c_int, c_int64, c_size_t, c_void_p

from . import build

_lock = threading.Lock()
_kernels = None
_host = None

P = c_void_p
I = c_int


class NativeError(RuntimeError):
    pass


def _declare(lib, name, argtypes, restype=c_int):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def kernels():
    """The CUDA kernel library (sm_100a)."""
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                path = build.build_kernels()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise NativeError(f"cannot load the CUDA kernel library {path}: {e}") from None
                _declare_kernels(lib)
                _kernels = lib
    return _kernels


def host():
    """The host runtime library (cache manager, scheduler)."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                path = build.build_host()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise NativeError(f"cannot load the host runtime library {path}: {e}") from None
                _declare_host(lib)
                _host = lib
    return _host


def _declare_kernels(lib):
    S = c_void_p  # cudaStream_t
    _declare(lib, "imparo_timeline_start", [P, c_int64])
    _declare(lib, "imparo_timeline_launches", [], c_int64)
    _declare(lib, "imparo_timeline_name", [c_int64, ctypes.c_char_p, I])
    _declare(lib, "imparo_embed_gather", [P, I, P, P, I, I, I, P, S])
    _declare(lib, "imparo_rmsnorm", [P, P, P, c_float, P, I, I, I, S])
    _declare(lib, "imparo_add_partials_rmsnorm", [P, P, I, c_int64, P, c_float, P, I, I, I, S])
    _declare(lib, "imparo_swiglu_act", [P, P, I, I, I, S])
    _declare(lib, "imparo_add_bias", [P, I, P, I, I, S])
    _declare(lib, "imparo_gated_act", [P, P, P, I, I, I, I, c_float, S])
    _declare(lib, "imparo_sgemm_nt", [P, P, P, I, I, I, I, I, I, S])
    _declare(lib, "imparo_gemm_lib_init", [P, c_size_t])
    _declare(lib, "imparo_gemm_bf16_nt", [P, P, P, I, I, I, I, I, I, I, S])
    _declare(lib, "imparo_gemm_tc_plan", [I, I, I, I, POINTER(c_int), POINTER(c_int), POINTER(c_int64), POINTER(c_int)])
    _declare(lib, "imparo_gemm_tc_max_clusters", [I, I])
    _declare(lib, "imparo_gemm_tc", [P, I, I, P, P, I, I, I, I, I, P, P, P, S])
    _declare(lib, "imparo_gemm_tc_gated", [P, I, I, P, P, I, I, I, I, I, c_float, P, P, P, P, S])
    _declare(lib, "imparo_gemm_tc_combine", [P, P, I, I, I, P, P, I, I, I, I, I, P, P, S])
    _declare(lib, "imparo_gemm_prefill", [P, I, I, P, P, I, I, I, I, I, I, c_float, P, P, S])
    _declare(lib, "imparo_qk_norm_rope_store",
             [P, I, P, P, P, P, P, I, c_float, P, P, P, P, I, I, I, I, I, I, I, I, c_int64, P, S])
    _declare(lib, "imparo_paged_attention",
             [P, P, P, I, P, P, P, I, I, I, I, c_float, P, I, I, I, I, P, S])
    _declare(lib, "imparo_paged_attention_split",
             [P, P, P, I, P, P, P, I, I, I, I, c_float, P, P, P, I, I, I, I, I, I, P, S])
    _declare(lib, "imparo_attention_split_combine", [P, P, P, I, I, I, I, I, S])
    _declare(lib, "imparo_attention_decode_mma",
             [P, P, P, P, P, P, I, I, I, I, c_float, P, P, P, I, I, I, I, I, I, I, I, P, S])
    _declare(lib, "imparo_attention_decode_mma_capped",
             [P, P, P, P, P, P, I, I, I, I, c_float, P, P, P, I, I, I, I, I, I, I, I, c_float, P, S])
    _declare(lib, "imparo_attention_decode_mma_grouped",
             [P, P, P, P, P, P, I, I, I, I, c_float, P, P, I, I, I, I, I, I, I, I, c_float, P, S])
    _declare(lib, "imparo_attention_split_combine_sinks", [P, P, P, I, I, I, I, P, I, S])
    _declare(lib, "imparo_attention_prefill_tc_sinks",
             [P, P, P, P, P, I, P, I, I, I, I, c_float, c_float, P, P, I, I, I, I, I, P, S])
    _declare(lib, "imparo_gemm_bf16_heads", [P, P, P, I, I, I, I, I, I, I, I, S])
    _declare(lib, "imparo_sigmoid_gate", [P, c_int64, P, c_int64, I, I, I, I, S])
    _declare(lib, "imparo_attention_decode_mma_qkv",
             [P, I, c_int64, P, P, P, I, c_float, P, P, P, P, P, I, I, I, I, c_float, P, P, P, I, I, I, I, I, I, P, S])
    _declare(lib, "imparo_attention_prefill",
             [P, P, P, P, P, I, P, I, I, I, I, c_float, P, I, I, I, I, P, S])
    _declare(lib, "imparo_attention_prefill_tc",
             [P, P, P, P, P, I, P, I, I, I, I, c_float, c_float, P, I, I, I, I, I, P, S])
    _declare(lib, "imparo_gated_conv", [P, I, P, P, P, P, P, P, P, I, I, I, I, I, c_int64, P, S])
    _declare(lib, "imparo_fold_partials", [P, I, c_int64, P, I, c_int64, S])
    _declare(lib, "imparo_gather_rows_f32", [P, P, P, I, I, S])
    _declare(lib, "imparo_argmax_rows", [P, P, P, P, I, I, I, S])
    _declare(lib, "imparo_sample_rows", [P, P, P, P, I, I, I, S])
    _declare(lib, "imparo_gemm_tc_configure", [])
    _declare(lib, "imparo_sample_rows_parts", [P, P, P, P, P, P, I, I, I, S])
    _declare(lib, "imparo_take_sampled_tokens", [P, P, P, I, I, S])
    _declare(lib, "imparo_selftest_wait_limit", [P, I, P, S])
    _declare(lib, "imparo_zero_state_slots", [P, P, I, c_int64, P, I, I, P, S])
    _declare(lib, "imparo_act_rows", [P, P, I, c_int64, I, S])
    _declare(lib, "imparo_gated_rmsnorm", [P, P, c_float, P, c_int64, P, I, I, I, S])
    _declare(lib, "imparo_norm_mean_add", [P, I, P, P, c_float, c_float, P, c_float, I, I, S])
    _declare(lib, "imparo_norm_mean_add_rmsnorm", [P, I, P, P, c_float, c_float, P, c_float, P, c_float, P, I, I, I, S])
    _declare(lib, "imparo_add_scaled", [P, P, c_float, c_int64, S])
    _declare(lib, "imparo_add_weighted", [P, P, P, P, P, I, c_float, c_float, c_float, c_float, c_int64, S])
    _declare(lib, "imparo_stream_inject", [P, P, I, P, P, I, I, I, P, S])
    _declare(lib, "imparo_softcap", [P, c_int64, c_float, S])
    _declare(lib, "imparo_qkv_rotate_store", [P, I, P, P, P, I, I, c_float, P, P, P, P, I, I, I, I, I, I, I, I, c_int64, P, S])
    _declare(lib, "imparo_act_rows_strided", [P, c_int64, P, I, I, I, I, S])
    _declare(lib, "imparo_attention_any", [P, P, P, I, P, P, P, I, I, I, I, c_float, I, P, c_float, P, I, I, I, I, I, P, S])
    _declare(lib, "imparo_qkv_prepare_store", [P, c_int64, P, I, P, P, P, I, c_float, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, S])
    _declare(lib, "imparo_out_norm_add", [P, P, P, c_float, P, I, I, I, S])
    _declare(lib, "imparo_cast_rows", [P, P, I, c_int64, S])
    _declare(lib, "imparo_scale_rows", [P, c_int64, c_float, S])
    _declare(lib, "imparo_mamba2_conv", [P, I, c_int64, I, I, I, I, I, P, P, P, P, P, P, P, I, I, I, P, P, P, S])
    _declare(lib, "imparo_mamba2_scan", [P, P, P, P, P, P, P, I, I, P, I, I, I, I, P, S])
    _declare(lib, "imparo_mamba2_scan_chunked", [P, P, P, P, P, P, P, I, I, P, I, I, I, I, I, I, P, P, P, P, S])
    _declare(lib, "imparo_gate_group_rmsnorm", [P, P, I, c_int64, P, c_float, P, I, I, I, I, S])
    _declare(lib, "imparo_moe_route", [P, I, P, I, I, I, I, I, I, I, I, c_float, c_float, I, P, P, P, S])
    _declare(lib, "imparo_moe_rows", [P, P, P, I, P, P, I, I, I, I, I, I, I, c_float, P, P, S])
    _declare(lib, "imparo_moe_pick", [P, I, I, I, I, I, I, I, I, c_float, c_float, I, P, P, S])
    _declare(lib, "imparo_moe_tiles", [P, P, P, P, P, I, I, I, I, I, I, I, c_float, P, P, P, P, P, P, S])
    _declare(lib, "imparo_moe_grouped", [P, P, P, I, P, P, I, I, I, I, I, I, I, c_float, P, P, P, P, S])
    _declare(lib, "imparo_linear_attention_recurrent", [P, P, P, c_int64, I, I, P, P, P, P, I, I, P, I, I, I, P, S])
    _declare(lib, "imparo_streams_norm", [P, P, I, P, P, c_float, P, I, I, I, S])
    _declare(lib, "imparo_streams_mix_add", [P, I, P, P, P, P, P, c_float, P, I, I, I, S])
    _declare(lib, "imparo_embed_copies", [P, I, P, c_float, I, P, P, I, P, I, I, I, P, S])
    _declare(lib, "imparo_channel_conv", [P, c_int64, I, I, I, P, P, P, P, P, P, I, I, P, c_int64, I, P, S])
    _declare(lib, "imparo_channel_conv_state", [P, c_int64, I, I, I, P, P, P, P, I, I, S])
    _declare(lib, "imparo_delta_prepare", [P, c_int64, I, I, P, c_int64, I, P, P, P, P, I, I, I, I, c_float, c_float, S])
    _declare(lib, "imparo_delta_scan", [P, c_int64, I, I, I, P, P, P, P, P, I, I, P, I, I, I, I, P, S])
    _declare(lib, "imparo_head_norm_gate", [P, P, c_float, P, c_int64, P, I, I, I, I, I, S])
    _declare(lib, "imparo_latent_norm_store", [P, c_int64, I, I, I, I, P, P, c_float, P, P, P, P, I, P, I, I, I, I, P, S])
    _declare(lib, "imparo_latent_rot_store", [P, c_int64, I, I, I, I, P, c_float, P, I, P, P, P, P, P, I, P, I, I, I, I, P, S])
    _declare(lib, "imparo_mlstm_scan", [P, c_int64, I, I, I, I, I, P, P, c_float, c_float, P, P, P, P, P, I, I, I, P, I, I, I, I, P, P, P,
                                        P, S])
    _declare(lib, "imparo_heads_linear", [P, c_int64, P, P, c_int64, P, c_int64, I, I, I, I, I, I, I, I, S])
    _declare(lib, "imparo_linear_attention_chunked", [P, P, P, c_int64, I, I, P, P, P, I, I, P, P, I, I, P, I, I, I, P, S])


def _declare_host(lib):
    from . import host_api
    host_api.declare(lib, _declare)
