"""The native kernel library, loaded once through its C ABI.

There is no fallback: if the library cannot be built or loaded, or a kernel
returns a non-zero status, a `CudaError` is raised.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional

from ..errors import CudaError

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_longlong = ctypes.c_longlong

_SIGNATURES = {
    "rfx_embed": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p],
    "rfx_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int,
                    c_void_p, c_int, c_int, c_void_p],
    "rfx_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_add": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "rfx_gather_dot": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_gemm_bf16_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                         c_int, c_int, c_float, c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_glu_clamped": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                     c_float, c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_relu2": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_xielu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                               c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_residual": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                  c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_qkv": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p,
                             c_float, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemv_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_qkv_post": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int,
                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                     c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "rfx_attention_plain": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                            c_void_p],
    "rfx_attention_decode_kf": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p],
    "rfx_attention_prefill_kf": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_void_p, c_void_p, c_void_p],
    "rfx_attention_prefill_tc_kf": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "rfx_qkv_post_kv": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "rfx_short_conv_act": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong,
                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_sigmoid_gate_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_hyper_expand": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_hyper_step": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                       c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_hyper_collapse": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                           c_int, c_void_p],
    "rfx_mamba_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                       c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_int,
                       c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                             c_void_p, c_longlong, c_void_p, c_void_p],
    "rfx_attention_decode_cluster": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                     c_void_p, c_longlong, c_void_p, c_void_p],
    "rfx_attention_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_void_p, c_void_p, c_void_p],
    "rfx_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "rfx_layernorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p,
                      c_int, c_int, c_void_p],
    "rfx_bigram_add": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                       c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p],
    "rfx_sinusoid_add": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "rfx_latent_post": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                        c_void_p],
    "rfx_heads_linear": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                         c_int, c_void_p],
    "rfx_scale_heads": [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p],
    "rfx_mlstm_scan": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                       c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                       c_void_p],
    "rfx_mlstm_chunk": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                        c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_void_p],
    "rfx_mlstm_out": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_int,
                      c_int, c_int, c_void_p],
    "rfx_moe_route": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_moe_up": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_float, c_float, c_void_p],
    "rfx_moe_down": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_void_p],
    "rfx_moe_group": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "rfx_moe_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_moe_activation": [c_void_p, c_int, c_longlong, c_int, c_void_p],
    "rfx_moe_combine": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_moe_route_scaled": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                             c_void_p],
    "rfx_sandwich_norm": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_float, c_void_p, c_int, c_int,
                          c_int, c_void_p],
    "rfx_group_norm_gate": [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                            c_void_p],
    "rfx_xielu": [c_void_p, c_int, c_longlong, c_float, c_float, c_void_p],
    "rfx_loop_input": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "rfx_tanh_cols": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_scaled_sum": [c_void_p, c_void_p, c_float, c_float, c_longlong, c_void_p],
    "rfx_sig_qkv_post": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_attention_sigmoid_plain": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "rfx_attention_sigmoid_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_void_p, c_void_p],
    "rfx_ssd_scan": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_void_p],
    "rfx_delta_rule": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_float,
                       c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                       c_void_p],
    "rfx_short_conv": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong,
                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "rfx_conv_qkv_post": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "rfx_conv_state_update": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p,
                              c_int, c_int, c_void_p],
    "rfx_rglru_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                       c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int,
                       c_int, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_void_p],
    "rfx_branch_norm_mean": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                             c_void_p],
    "rfx_glu_clamped": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "rfx_row_gate_add": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
    "rfx_stream_concat": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_logit_finish": [c_void_p, c_longlong, c_float, c_float, c_void_p],
    "rfx_wait_probe": [c_longlong, c_void_p, c_void_p],
    "rfx_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "rfx_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p, c_void_p],
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc import build

        try:
            path = build.ensure_built()
            handle = ctypes.CDLL(path)
        except (RuntimeError, OSError) as e:
            raise CudaError(f"the native kernel library is not available: {e}") from e
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as e:
                raise CudaError(f"native library {path} lacks symbol {name}") from e
            fn.argtypes = argtypes
            fn.restype = c_int
        handle.rfx_gemm_bf16_tc_max_parts.argtypes = [c_int]
        handle.rfx_gemm_bf16_tc_max_parts.restype = c_int
        handle.rfx_mlstm_state_floats.argtypes = [c_int, c_int]
        handle.rfx_mlstm_state_floats.restype = c_int
        handle.rfx_mamba_scan_scratch.argtypes = [c_int, c_int, c_int, c_int]
        handle.rfx_mamba_scan_scratch.restype = c_longlong
        handle.rfx_sm_count.argtypes = []
        handle.rfx_sm_count.restype = c_int
        handle.rfx_sample_work_bytes.argtypes = [c_int, c_int]
        handle.rfx_sample_work_bytes.restype = c_longlong
        handle.rfx_error_string.argtypes = [c_int]
        handle.rfx_error_string.restype = ctypes.c_char_p
        _lib = handle
        return _lib


def register_signature(name: str, argtypes) -> None:
    """Declare one more exported function (used by kernels added later)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


LAUNCHES = 0  # kernels of this library launched (or captured into a graph) so far


ERR_UNSUPPORTED = -2  # a kernel's answer for sizes it does not take


def check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status != 0:
        msg = lib().rfx_error_string(status).decode("utf-8", "replace")
        raise CudaError(f"{what} failed: {msg} (status {status})")
