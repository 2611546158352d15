"""ctypes bindings of libingot_cuda.so (include/ingot_cuda.h).

Loading fails loudly when the library has not been built: there is no CPU or
framework fallback for any operator.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libingot_cuda.so")

OK, INVALID, UNSUPPORTED, DEVICE, EOF, INTERRUPTED, TIMEOUT = range(7)
OPT_PDL, OPT_FORCE_PLAIN, OPT_NO_MMA, OPT_TCGEN05_GEMV, OPT_EP_WORLD, OPT_GROUP_SCOPE, OPT_WIDE_ROWS = 1, 2, 3, 4, 5, 6, 7
X_PACKED = 256
X_DIGITS = 258
X_PACKED_HI = 259

vp, u32, u64, i32, f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float
sz = C.c_size_t

# name -> argument types (every function returns ingot_status unless noted)
SIGNATURES = {
    "ingot_geometry": [u32, C.POINTER(u32), C.POINTER(u32)],
    "ingot_tensor_layout": [u32, u64, u64, u64, C.POINTER(u64), C.POINTER(u64)],
    "ingot_gpu_create": [i32, C.POINTER(vp)],
    "ingot_gpu_set_stream": [vp, vp],
    "ingot_gpu_set_option": [vp, i32, i32],
    "ingot_synchronize": [vp],
    "ingot_buffer_alloc": [vp, sz, C.POINTER(vp)],
    "ingot_buffer_free": [vp, vp],
    "ingot_buffer_upload": [vp, vp, vp, sz],
    "ingot_buffer_read": [vp, vp, vp, sz],
    "ingot_buffer_zero": [vp, vp, sz],
    "ingot_host_alloc": [vp, sz, C.POINTER(vp)],
    "ingot_host_free": [vp, vp],
    "ingot_weight_upload": [vp, vp, u32, u64, u64, u64, sz, C.POINTER(vp)],
    "ingot_dequant_rows": [vp, vp, u32, u64, u32, u32, vp],
    "ingot_matmul": [vp, vp, u32, u32, u32, u32, u32, vp, u32, u32, vp],
    "ingot_gemm": [vp, vp, u32, u32, u32, u32, u32, vp, u32, u32, vp],
    "ingot_gate_up": [vp, vp, vp, u32, u32, u32, u32, vp, u32, u32, u32, vp],
    "ingot_routed": [vp, vp, u32, u32, u32, u32, u32, vp, u32, vp, u32, u32, u32, vp],
    "ingot_routed_gate_up": [vp, vp, vp, u32, u32, u32, u32, u32, vp, u32, vp, u32, u32, vp],
    "ingot_route_topk": [vp, vp, u32, u32, u32, vp, vp],
    "ingot_moe_sum": [vp, vp, vp, u32, u32, u32, vp],
    "ingot_activation": [vp, vp, vp, u64, u32, vp],
    "ingot_merge": [vp, vp, vp, vp, vp, u32, u32, vp],
    "ingot_add_rms": [vp, vp, vp, vp, vp, vp, vp, u32, u32, f32, u32],
    "ingot_add_rms_packed": [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, f32, u32],
    "ingot_expert_layout": [vp, vp, u32, u32, u32, vp, vp, vp, vp],
    "ingot_combine_packed": [vp, vp, vp, vp, u32, u32, u32, vp],
    "ingot_ep_localize": [vp, vp, vp, u32, u32, u32, vp, vp],
    "ingot_convert_bf16": [vp, vp, u64, vp],
    "ingot_packed_x_bytes": [u32, C.POINTER(u64)],
    "ingot_pack_x": [vp, vp, u32, u32, u32, vp],
    "ingot_matmul_normed": [vp, vp, u32, u32, u32, u32, u32, vp, vp, vp, vp, C.c_float, u32, u32, vp],
    "ingot_gate_up_normed": [vp, vp, vp, u32, u32, u32, u32, vp, vp, vp, vp, C.c_float, u32, u32, u32, vp],
    "ingot_independent_begin": [vp],
    "ingot_independent_end": [vp],
    "ingot_packed_hi_bytes": [u32, C.POINTER(u64)],
    "ingot_pack_x_hi": [vp, vp, u32, u32, vp],
    "ingot_packed_digits_bytes": [u32, C.POINTER(u64)],
    "ingot_pack_digits": [vp, vp, u32, u32, u32, vp],
    "ingot_matvec_static": [vp, u32, u32, u32, u32, u32, vp, vp, vp, i32],
    "ingot_expert_project": [vp, vp, u32, u32, u32, u32, u32, vp, vp, vp, u32, u32, u32, u32, vp],
    "ingot_expert_gate_up": [vp, vp, vp, u32, u32, u32, u32, u32, vp, vp, vp, u32, u32, u32, vp],
    "ingot_embedding_batch": [vp, vp, vp, u32, u32, u32, u32, u32, vp],
    "ingot_qk_rope_cache": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32],
    "ingot_attention_decode": [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32],
    "ingot_gather_rows": [vp, vp, vp, u32, u32, u32, vp],
    "ingot_expert_gemm": [vp, vp, u32, u32, u32, u32, u32, vp, vp, u32, vp],
    "ingot_expert_gemm_gate_up": [vp, vp, vp, u32, u32, u32, u32, u32, vp, vp, u32, u32, vp],
    "ingot_scale_rows": [vp, vp, u64, f32, vp],
    "ingot_softcap_rows": [vp, vp, u64, f32, vp],
    "ingot_swiglu_fused": [vp, vp, u32, u32, vp],
    "ingot_copy_columns": [vp, vp, u32, u32, u32, u32, vp],
    "ingot_attention_prefill": [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32],
    "ingot_greedy_select": [vp, vp, vp, u32, u32, vp, vp],
    "ingot_gguf_open": [C.c_char_p, C.POINTER(vp)],
    "ingot_gguf_tensor_at": [vp, u64, C.POINTER(C.c_char_p), vp],
    "ingot_gguf_tensor": [vp, C.c_char_p, vp],
    "ingot_gguf_integer": [vp, C.c_char_p, C.POINTER(u64)],
    "ingot_gguf_float": [vp, C.c_char_p, C.POINTER(f32)],
    "ingot_gguf_string": [vp, C.c_char_p, C.POINTER(C.c_char_p)],
    "ingot_gguf_array_length": [vp, C.c_char_p, C.POINTER(u64)],
    "ingot_gguf_array_integer": [vp, C.c_char_p, u64, C.POINTER(u64)],
    "ingot_gguf_array_string": [vp, C.c_char_p, u64, C.POINTER(C.c_char_p)],
    "ingot_gguf_read_range": [vp, vp, u64, vp, u64],
    "ingot_gguf_rows": [vp, C.c_char_p, vp, u64, vp],
    "ingot_gguf_matrix": [vp, C.c_char_p, vp, u32, vp, u64, vp],
    "ingot_weight_load": [vp, vp, C.c_char_p, vp, u32, C.POINTER(vp), vp],
    "ingot_group_create": [vp, u32, u32, sz, u32, C.POINTER(vp), vp],
    "ingot_group_connect": [vp, vp],
    "ingot_group_connect_local": [C.POINTER(vp), u32],
    "ingot_group_window": [vp, u32, C.POINTER(vp)],
    "ingot_group_step": [vp],
    "ingot_group_wait": [vp, u32, vp, u32],
    "ingot_tp_signal_next": [vp, u32],
    "ingot_tp_wait_next": [vp, u32, u32],
    "ingot_ep_dispatch": [vp, u32, vp, vp, vp, u32, u32, u32, u32, u32],
    "ingot_ep_receive": [vp, u32, vp, u32, u32, vp],
    "ingot_ep_return": [vp, u32, vp, vp, vp, u32, u32],
    "ingot_ep_combine": [vp, u32, vp, vp, u32, u32, u32, u32, vp],
    "ingot_chain_begin": [vp],
    "ingot_chain_end": [vp, C.POINTER(vp)],
    "ingot_chain_submit": [vp, vp],
    "ingot_chain_info": [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)],
    "ingot_command_begin": [vp],
    "ingot_command_end": [vp, C.POINTER(vp)],
    "ingot_command_submit": [vp, vp],
    "ingot_gpu_configure_workspace": [vp, sz],
    "ingot_output_alloc": [vp, sz, C.POINTER(vp)],
    "ingot_output_release": [vp, vp],
    "ingot_workspace_statistics": [vp, C.POINTER(u64), C.POINTER(u64), C.POINTER(sz), C.POINTER(sz)],
    "ingot_ffn": [vp, vp, vp, vp, u32, u32, u32, u32, vp, vp, vp, vp],
    "ingot_moe_host": [vp, vp, vp, vp, vp, sz, vp, sz, vp],
    "ingot_dequant_host": [vp, vp, sz, u64, u64, u64, u32, u64, vp],
    "ingot_project_host": [vp, vp, sz, u64, u64, u64, u32, u64, vp, sz, vp],
}
# functions with another return type
OTHER = {
    "ingot_gpu_destroy": (None, [vp]),
    "ingot_last_error": (C.c_char_p, [vp]),
    "ingot_command_destroy": (None, [vp]),
    "ingot_chain_destroy": (None, [vp]),
    "ingot_group_destroy": (None, [vp]),
    "ingot_gguf_close": (None, [vp]),
    "ingot_gguf_last_error": (C.c_char_p, []),
    "ingot_gguf_architecture": (C.c_char_p, [vp]),
    "ingot_gguf_tensor_count": (u64, [vp]),
    "ingot_gguf_bytes_read": (u64, [vp]),
    "ingot_matvec_static_error": (C.c_char_p, []),
}

_lib = None


def load() -> C.CDLL:
    """The shared library, with argument types attached."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m ingot_b200.build` "
            "(needs nvcc). ingot_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = i32
        fn.argtypes = args
    for name, (res, args) in OTHER.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def exported_names() -> list[str]:
    return sorted(list(SIGNATURES) + list(OTHER))
