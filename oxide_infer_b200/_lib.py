"""ctypes binding of liboxi_kv.so.  There is no fallback: if the library is
missing or fails to load, importing the operators raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# OXI_KV_LIB selects another build of the same library (the bounds-checking build of
# oxide_infer_b200.build, for the tests); there is still no fallback if it is missing.
SO_PATH = os.environ.get("OXI_KV_LIB") or os.path.join(HERE, "liboxi_kv.so")

_vp, _u32, _i32, _f32 = C.c_void_p, C.c_uint32, C.c_int32, C.c_float

# name -> argument ctypes (all functions return int32 unless listed in _RESTYPE)
SIGNATURES = {
    "oxi_version": [],
    "oxi_status_string": [_i32],
    "oxi_last_error_string": [],
    "oxi_create": [C.POINTER(_vp), _i32, _u32, _u32, _u32],
    "oxi_destroy": [_vp],
    "oxi_workspace_bytes": [_vp],
    "oxi_device_status": [_vp, _vp, C.POINTER(_u32)],
    "oxi_append": [_vp] * 12 + [_u32, _f32],
    "oxi_decode_attn": [_vp] * 8 + [_u32, _u32],
    "oxi_append_decode": [_vp] * 15 + [_u32, _u32, _f32],
    "oxi_prefill_attn": [_vp] * 8 + [_u32, _u32],
    "oxi_conv_decode": [_vp] * 6 + [_u32],
    "oxi_conv_prefill": [_vp] * 8 + [_u32],
    "oxi_advance_step": [_vp] * 4 + [_u32, _u32],
    "oxi_append_paged": [_vp] * 11 + [_u32, _f32],
    "oxi_decode_attn_paged": [_vp] * 7 + [_u32, _u32],
    "oxi_append_decode_paged": [_vp] * 13 + [_u32, _u32, _f32],
    "oxi_prefill_attn_paged": [_vp] * 8 + [_u32, _u32],
    "oxi_prefill_split_configure": [_vp, _u32, _u32],
    "oxi_register_kv_slab": [_vp, _vp, C.c_uint64],
    "oxi_prefill_split_slot_bytes": [],
    "oxi_embed_lookup": [_vp] * 5 + [_u32, _u32, _u32],
    "oxi_argmax": [_vp] * 4 + [_u32, _u32],
    "oxi_qk_rmsnorm": [_vp, _vp, _vp, _vp, _f32, _u32, _u32],
    "oxi_rope": [_vp] * 6 + [_u32, _u32],
    "oxi_kv_copy": [_vp] * 5 + [_u32],
    "oxi_sigmoid_gate": [_vp] * 4 + [_u32],
    "oxi_decode_step_host": [_vp] * 14 + [_u32, _u32, _u32, _f32],
    "oxi_decode_attn_static": [_vp] * 7 + [_u32, _u32, _u32],
    "oxi_qkvg_create": [C.POINTER(_vp), _vp, _vp, _vp, _vp],
    "oxi_linear_create": [C.POINTER(_vp), _vp, _u32],
    "oxi_linear_destroy": [_vp],
    "oxi_project_append": [_vp] * 14 + [_u32, _f32],
    "oxi_linear_forward": [_vp] * 5 + [_u32],
    "oxi_host_last_error_string": [],
    "oxi_pool_create": [C.POINTER(_vp), _vp, _u32, _u32, C.c_uint64],
    "oxi_pool_destroy": [_vp],
    "oxi_pool_capacity_tokens": [_vp],
    "oxi_pool_free_tokens": [_vp],
    "oxi_pool_free_slots": [_vp],
    "oxi_pool_acquire": [_vp, _vp, C.c_uint64, _vp],
    "oxi_pool_release": [_vp, _vp],
    "oxi_pool_k_ptr": [_vp, _u32, _vp],
    "oxi_pool_v_ptr": [_vp, _u32, _vp],
    "oxi_pool_conv_ptr": [_vp, _u32, _vp],
    "oxi_tables_create": [C.POINTER(_vp), _vp, _u32],
    "oxi_tables_destroy": [_vp],
    "oxi_tables_set_row": [_vp, _u32, _vp, _u32],
    "oxi_tables_upload": [_vp, _vp, _u32],
    "oxi_tables_advance": [_vp, _vp, _vp, _u32],
    "oxi_tables_batch": [_vp],
    "oxi_tables_k_ptrs": [_vp, _u32],
    "oxi_tables_v_ptrs": [_vp, _u32],
    "oxi_tables_conv_ptrs": [_vp, _u32],
    "oxi_tables_pos_ids": [_vp],
    "oxi_tables_seq_lens": [_vp],
    "oxi_debug_arm_wait_fault": [_vp, _u32, _u32, _u32],
    "oxi_static_device_status": [_vp, C.POINTER(_u32)],
    "oxi_debug_stream_read": [_vp, _vp, _vp, C.c_uint64, _u32],
}
_RESTYPE = {"oxi_status_string": C.c_char_p, "oxi_last_error_string": C.c_char_p,
            "oxi_host_last_error_string": C.c_char_p,
            "oxi_pool_capacity_tokens": C.c_uint64, "oxi_pool_free_tokens": C.c_uint64, "oxi_pool_free_slots": _u32,
            "oxi_pool_k_ptr": C.c_uint64, "oxi_pool_v_ptr": C.c_uint64, "oxi_pool_conv_ptr": C.c_uint64,
            "oxi_tables_batch": _u32, "oxi_tables_k_ptrs": _vp, "oxi_tables_v_ptrs": _vp,
            "oxi_tables_conv_ptrs": _vp, "oxi_tables_pos_ids": _vp, "oxi_tables_seq_lens": _vp,
            "oxi_workspace_bytes": C.c_size_t, "oxi_prefill_split_slot_bytes": C.c_uint64}

_lib = None


def load() -> C.CDLL:
    """Load the shared library and bind every declared symbol (raises if any is missing)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise ImportError(
            f"{SO_PATH} is missing: build it with `python -m oxide_infer_b200.build` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
    lib = C.CDLL(SO_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = args
        fn.restype = _RESTYPE.get(name, _i32)
    _lib = lib
    return lib
