"""Loads the compiled CUDA library with ctypes and declares its entry points.

There is no other implementation behind these names: if the library cannot be built or
loaded the engine stops with an error rather than compute on the CPU or through a
framework op.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_size_t, c_void_p

_lib = None
_lock = threading.Lock()
LAUNCHES = 0    # entry points called since the counter was last reset (each launches at least one kernel)

P, I, F = c_void_p, c_int, c_float

_SIGNATURES = {
    # name: argtypes (all return int)
    "nhv_embed": [I, P, P, P, I, I, I, P],
    "nhv_feed_tokens": [P, P, P, I, I, I, P],
    "nhv_rmsnorm": [I, P, P, P, P, P, I, I, F, I, F, P],
    "nhv_silu_mul": [I, P, P, I, I, P],
    "nhv_to_f32": [I, P, P, c_size_t, P],
    "nhv_qk_norm_rope_store": [I, P, I, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, P],
    "nhv_attention_simt": [I, P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, I, I, F, P],
    "nhv_gemm_nt_simt": [I, P, P, P, I, I, I, I, I, I, I, P],
    "nhv_sample": [P, P, I, P, P, P, I, I, P, P, P, I, P, P],
    "nhv_gemm_small_m": [P, P, P, I, I, I, I, I, I, I, P],
    "nhv_gemm_stream_k": [P, P, P, I, I, I, I, I, I, I, P, P, I, I, P],
    "nhv_gemm_slab": [P, P, P, I, I, I, I, I, I, I, P],
    "nhv_gemm_slab_hint": [P, P, P, I, I, I, I, I, I, I, P, ctypes.c_longlong, I, I, P],
    "nhv_gemm_slab_geometry": [I, I, I, I, P, P, P, P, P],
    "nhv_gemm_tcgen05": [P, P, P, I, I, I, I, I, I, I, P, P, I, I, P],
    "nhv_gelu_tanh_mul": [I, P, P, I, I, P],
    "nhv_gemm_rows_f32": [P, I, P, I, P, I, I, I, I, P],
    "nhv_embed_scaled_f32": [I, P, P, P, I, I, I, F, P],
    "nhv_rmsnorm_stream": [I, P, P, P, P, F, F, F, P, P, P, I, I, F, I, F, I, P],
    "nhv_scaled_sum": [I, P, P, P, F, F, c_size_t, P],
    "nhv_short_conv_silu": [I, I, P, I, P, I, P, P, P, ctypes.c_long, P, P, P, I, I, I, I, P],
    "nhv_delta_rule": [I, P, P, I, P, P, P, P, ctypes.c_long, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, I, P],
    "nhv_ssd_scan": [I, P, P, I, P, I, P, P, P, P, ctypes.c_long, P, P, P, I, I, I, I, I, I, I, I, P],
    "nhv_gated_rmsnorm": [I, P, I, P, P, I, P, I, I, I, I, F, I, I, P],
    "nhv_rope_norm_store": [I, P, I, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, I, P, P, I, I, P],
    "nhv_dyntanh": [I, I, I, P, P, P, P, P, I, I, P],
    "nhv_embed_dyntanh": [I, P, P, P, P, P, P, I, I, I, P],
    "nhv_dyntanh_stream": [I, P, P, P, P, P, P, P, P, P, P, I, I, I, P],
    "nhv_sigmoid_mul": [I, P, I, P, I, P, I, I, I, P],
    "nhv_add_row_bias": [I, P, P, I, I, P],
    "nhv_clamped_glu": [I, P, P, I, I, F, F, P],
    "nhv_mlstm_scan": [I, P, P, I, P, I, P, F, P, ctypes.c_long, P, P, P, I, I, I, I, I, I, P],
    "nhv_moe_route": [P, P, P, I, P, I, I, I, I, I, I, I, P],
    "nhv_moe_align": [P, I, I, I, P, P, P, P],
    "nhv_moe_gemm_simt": [I, I, P, P, I, P, P, P, P, I, I, I, I, F, F, F, P, P],
    "nhv_moe_gemm_mma": [I, I, P, P, I, P, P, P, P, I, I, I, I, F, F, F, P, P],
    "nhv_moe_gather_rows": [P, P, P, I, I, I, P],
    "nhv_moe_gemm_tcgen05": [I, P, P, P, P, I, P, P, I, I, I, F, F, F, P, P],
    "nhv_moe_combine": [I, P, P, P, P, P, I, P, P, P, I, I, I, I, P],
    "nhv_attention_simt_ex": [I, P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P, I, I, P],
    "nhv_causal_filter_add": [I, P, P, I, P, I, P, P, P, ctypes.c_long, P, P, P, I, I, I, I, P],
    "nhv_latent_rope_store": [I, P, I, P, I, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "nhv_gemm_nt_simt_batched": [I, P, P, P, I, I, I, I, I, I, I, I, ctypes.c_long, ctypes.c_long, ctypes.c_long, P],
    "nhv_general_delta": [I, P, P, I, P, I, P, P, P, P, ctypes.c_long, P, P, P, P, P, P, I, I, I, I, F, P],
    "nhv_general_delta_tanh": [I, P, P, I, I, I, P],
    "nhv_sigmoid_mul_heads": [I, P, I, P, I, P, I, I, I, I, I, P],
    "nhv_latent_gather": [I, P, P, P, P, I, P, P, I, I, I, I, I, I, I, P],
    "nhv_latent_assemble": [I, P, P, P, P, P, I, P, I, ctypes.c_long, I, I, I, I, I, I, I, P],
    "nhv_latent_decode_supports": [I, I, I],
    "nhv_latent_decode": [P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, I, F, P, I, P, P, P],
    "nhv_relu_squared": [I, P, c_size_t, P],
    "nhv_scale_softcap": [P, F, F, c_size_t, P],
    "nhv_gelu_tanh": [I, P, c_size_t, P],
    "nhv_postnorm_stream": [I, P, P, P, P, F, P, P, F, P, P, I, I, F, F, P],
    "nhv_stream_round": [I, P, P, c_size_t, P],
    "nhv_token_shift_mix": [I, P, P, P, P, ctypes.c_long, P, P, P, I, I, I, I, P],
    "nhv_decay_scan": [I, P, P, P, P, I, P, P, P, P, ctypes.c_long, P, P, P, I, I, I, I, I, I, I, P],
    "nhv_decay_lowrank": [I, P, P, I, P, P, I, I, I, P],
}


class KernelError(RuntimeError):
    pass


def load_library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import ensure_built
                path = ensure_built()
                lib = ctypes.CDLL(path)
                lib.nhv_last_error.restype = ctypes.c_char_p
                lib.nhv_last_error.argtypes = []
                for name, argtypes in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.argtypes = argtypes
                    fn.restype = c_int
                _lib = lib
    return _lib


def declare(name: str, argtypes) -> None:
    """Declare one more entry point (used by kernels added in their own files)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def call(name: str, *args) -> None:
    global LAUNCHES
    LAUNCHES += 1
    lib = load_library()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(lib.nhv_last_error().decode(errors="replace"))
