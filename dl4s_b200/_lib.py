"""Loader of libdl4s_cuda.so (the C ABI declared in include/dl4s_cuda.h).

The shared object is built in-tree by dl4s_b200.build. There is no fallback: if
it is missing, or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DL4S_CUDA_LIB") or os.path.join(_HERE, "libdl4s_cuda.so")

c_f32p = ctypes.POINTER(ctypes.c_float)
c_i32p = ctypes.POINTER(ctypes.c_int32)
c_i64p = ctypes.POINTER(ctypes.c_int64)
c_vp = ctypes.c_void_p
c_i64 = ctypes.c_int64
c_i32 = ctypes.c_int32
c_f32 = ctypes.c_float
c_sz = ctypes.c_size_t

PREC_FP32 = 0
PREC_F16 = 1
PREC_F16_SPLIT = 2
ACT_GELU_SIGMOID = 0
ACT_RELU = 1

# name -> argtypes; every function returns int32 status unless listed in _SPECIAL.
_SIGNATURES = {
    "dl4s_cuda_device_count": [c_i32p],
    "dl4s_cuda_init": [c_i32p, c_i32],
    "dl4s_cuda_shutdown": [],
    "dl4s_cuda_set_device": [c_i32],
    "dl4s_cuda_get_device": [c_i32p],
    "dl4s_cuda_sync": [],
    "dl4s_cuda_set_stream": [c_vp],
    "dl4s_cuda_get_stream": [ctypes.POINTER(c_vp)],
    "dl4s_cuda_device_status": [c_i32p],
    "dl4s_cuda_set_timing": [c_i32],
    "dl4s_cuda_get_timing": [c_f32p],
    "dl4s_cuda_set_trace": [c_i32],
    "dl4s_cuda_trace_read": [ctypes.c_char_p, c_sz],
    "dl4s_cuda_inject_failure": [c_i32, c_i32],
    "dl4s_cuda_launch_count": [ctypes.POINTER(ctypes.c_uint64)],
    "dl4s_cuda_graph_begin": [],
    "dl4s_cuda_graph_end": [ctypes.POINTER(c_vp)],
    "dl4s_cuda_graph_launch": [c_vp],
    "dl4s_cuda_graph_destroy": [c_vp],
    "dl4s_cuda_profile_begin": [],
    "dl4s_cuda_profile_end": [ctypes.c_char_p, c_sz],
    "dl4s_cuda_malloc": [c_sz, ctypes.POINTER(c_vp)],
    "dl4s_cuda_free": [c_vp],
    "dl4s_cuda_memcpy_h2d": [c_vp, c_vp, c_sz],
    "dl4s_cuda_memcpy_d2h": [c_vp, c_vp, c_sz],
    "dl4s_cuda_memcpy_d2d": [c_vp, c_vp, c_sz],
    "dl4s_cuda_memcpy_h2d_async": [c_vp, c_vp, c_sz],
    "dl4s_cuda_memcpy_d2h_async": [c_vp, c_vp, c_sz],
    "dl4s_cuda_memcpy_h2d_async_on": [c_vp, c_vp, c_sz, c_vp],
    "dl4s_cuda_memcpy_d2h_async_on": [c_vp, c_vp, c_sz, c_vp],
    "dl4s_cuda_host_alloc": [c_sz, ctypes.POINTER(c_vp)],
    "dl4s_cuda_host_free": [c_vp],
    "dl4s_cuda_get_value_f32": [c_vp, c_f32p],
    "dl4s_cuda_set_value_f32": [c_vp, c_f32],
    "dl4s_cuda_copy_strided_f32": [c_vp, c_i64p, c_i64, c_vp, c_i64p, c_i64, c_i64p, c_i32],
    "dl4s_cuda_fill_f32": [c_f32, c_vp, c_i64],
    "dl4s_cuda_fill_i32": [c_i32, c_vp, c_i64],
    "dl4s_cuda_vadd": [c_vp, c_vp, c_vp, c_i64],
    "dl4s_cuda_vsub": [c_vp, c_vp, c_vp, c_i64],
    "dl4s_cuda_vmul": [c_vp, c_vp, c_vp, c_i64],
    "dl4s_cuda_vdiv": [c_vp, c_vp, c_vp, c_i64],
    "dl4s_cuda_vneg": [c_vp, c_vp, c_i64],
    "dl4s_cuda_broadcast_add": [c_vp, c_i64p, c_i32, c_vp, c_i64p, c_i32, c_vp],
    "dl4s_cuda_broadcast_sub": [c_vp, c_i64p, c_i32, c_vp, c_i64p, c_i32, c_vp],
    "dl4s_cuda_broadcast_mul": [c_vp, c_i64p, c_i32, c_vp, c_i64p, c_i32, c_vp],
    "dl4s_cuda_broadcast_div": [c_vp, c_i64p, c_i32, c_vp, c_i64p, c_i32, c_vp],
    "dl4s_cuda_exp": [c_vp, c_vp, c_i64],
    "dl4s_cuda_log": [c_vp, c_vp, c_i64],
    "dl4s_cuda_sqrt": [c_vp, c_vp, c_i64],
    "dl4s_cuda_relu": [c_vp, c_vp, c_i64],
    "dl4s_cuda_heaviside": [c_vp, c_vp, c_i64],
    "dl4s_cuda_sin": [c_vp, c_vp, c_i64],
    "dl4s_cuda_cos": [c_vp, c_vp, c_i64],
    "dl4s_cuda_tanh": [c_vp, c_vp, c_i64],
    "dl4s_cuda_reduce_sum": [c_vp, c_i64p, c_i32, c_i32p, c_i32, c_vp],
    "dl4s_cuda_reduce_max": [c_vp, c_i64p, c_i32, c_i32p, c_i32, c_vp, c_vp],
    "dl4s_cuda_permute_axes": [c_vp, c_i64p, c_i32, c_i32p, c_vp],
    "dl4s_cuda_stack": [ctypes.POINTER(c_vp), c_i64p, c_i32, c_i32, c_i32, c_vp],
    "dl4s_cuda_unstack": [c_vp, ctypes.POINTER(c_vp), c_i64p, c_i32, c_i32, c_i32],
    "dl4s_cuda_unstack_add": [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), c_i64p, c_i32, c_i32, c_i32],
    "dl4s_cuda_dropout": [c_vp, c_vp, c_i64, c_f32, ctypes.c_uint64, ctypes.c_uint32],
    "dl4s_cuda_set_dropout": [c_f32, ctypes.c_uint64],
    "dl4s_cuda_dropout_counter": [ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32)],
    "dl4s_cuda_band": [c_vp, c_i64, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp],
    "dl4s_cuda_gemm": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_f32, c_f32, c_i32, c_i32, c_i32],
    "dl4s_cuda_sdpa_forward": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f32, c_vp, c_i32,
                               c_vp, c_i64p, c_vp, c_i32],
    "dl4s_cuda_sdpa_backward": [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f32, c_vp, c_i32, c_vp,
                                c_i64p, c_vp, c_vp, c_vp, c_i32],
    "dl4s_cuda_sdpa_decode": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_f32, c_vp, c_vp],
    "dl4s_cuda_sdpa_decode_noalloc": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_f32, c_vp, c_vp],
    "dl4s_cuda_layernorm_backward": [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp],
    "dl4s_cuda_layernorm": [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp],
    "dl4s_cuda_mha_forward": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp,
                              c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_i64p, c_vp, c_i32],
    "dl4s_cuda_mha_heads_forward": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp,
                                    c_vp, c_i32, c_vp, c_i32, c_i32],
    "dl4s_cuda_mha_heads_half_supported": [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i32p],
    "dl4s_cuda_mha_output_forward": [c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i64,
                                     c_i64],
    "dl4s_cuda_comm_unique_id": [c_vp],
    "dl4s_cuda_comm_init": [c_i32, c_i32, c_vp],
    "dl4s_cuda_comm_destroy": [],
    "dl4s_cuda_comm_info": [c_i32p, c_i32p, c_i32p],
    "dl4s_cuda_comm_timing": [c_f32p, c_f32p],
    "dl4s_cuda_mha_forward_sharded": [c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32,
                                      c_vp, c_i32, c_i32],
    "dl4s_cuda_mha_sharded_plan": [c_i64, c_i32, c_i32, c_i32, c_i64p, c_i64p],
    "dl4s_cuda_mha_decode_step": [c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64,
                                  c_vp, c_vp],
    "dl4s_cuda_decoder_forward": [c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_i32,
                                  c_vp, c_i32],
    "dl4s_cuda_mha_kv_project": [c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_i64],
    "dl4s_cuda_decoder_cache_create": [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, ctypes.POINTER(c_vp)],
    "dl4s_cuda_decoder_cache_set_encoder": [c_vp, c_vp, c_vp],
    "dl4s_cuda_decoder_cache_lengths": [c_vp, ctypes.POINTER(c_vp)],
    "dl4s_cuda_decoder_step": [c_vp, c_vp, c_i32, c_vp],
    "dl4s_cuda_decoder_cache_destroy": [c_vp],
    "dl4s_cuda_embed_at": [c_vp, c_i64, c_i64, c_i64, c_i64, c_vp, c_i64, c_i32, c_vp],
    "dl4s_cuda_transformer_greedy_decode": [c_i32p, c_i64, c_i32, c_i32, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64,
                                            c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32p, c_i64p],
    "dl4s_cuda_output_head": [c_vp, c_i64, c_i64, c_vp, c_i64, c_vp, c_vp, c_i32],
    "dl4s_cuda_log_softmax_rows": [c_vp, c_i64, c_i64, c_vp],
    "dl4s_cuda_ffn_forward": [c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_i32],
    "dl4s_cuda_encoder_forward": [c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_i32,
                                  c_vp, c_i32],
    "dl4s_cuda_encoder_prepare": [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, c_i32, ctypes.POINTER(c_vp)],
    "dl4s_cuda_encoder_prepared_refresh": [c_vp],
    "dl4s_cuda_encoder_prepared_destroy": [c_vp],
    "dl4s_cuda_encoder_forward_prepared": [c_vp, c_vp, c_i64, c_i64, c_vp, c_i32, c_vp],
    "dl4s_cuda_embed_positional": [c_vp, c_i64, c_i64, c_i64, c_vp, c_i64, c_i32, c_vp],
}
_SPECIAL = {
    "dl4s_cuda_last_error": (ctypes.c_char_p, []),
    "dl4s_cuda_version": (c_i32, []),
}

EXPORTS = tuple(_SIGNATURES) + tuple(_SPECIAL)


class DL4SCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libdl4s_cuda status {status}: {message}")
        self.status = status


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared object and bind every declared symbol. Raises if the
    library was not built (python -m dl4s_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `python -m dl4s_b200.build`; "
                                "there is no fallback implementation")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_i32
    for name, (restype, argtypes) in _SPECIAL.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        msg = load().dl4s_cuda_last_error()
        raise DL4SCudaError(status, msg.decode() if msg else "")


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args))
