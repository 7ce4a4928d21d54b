"""ctypes binding of libpd_b200.so (the C ABI declared in include/pd_b200.h).

There is no fallback: if the shared library has not been built, loading raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PD_B200_LIB") or os.path.join(HERE, "libpd_b200.so")   # PD_B200_LIB: a tuning build elsewhere

PD_OK, PD_INVALID_ARGUMENT, PD_LENGTH_ERROR, PD_CUDA_ERROR, PD_OUT_OF_PAGES, PD_KERNEL_TIMEOUT, PD_INTERNAL = range(7)


class InvalidArgument(ValueError):
    """std::invalid_argument in the reference."""


class LengthError(ValueError):
    """std::length_error in the reference."""


class CudaError(RuntimeError):
    """The reference prints and aborts on a CUDA failure; here it is an exception."""


class KernelTimeout(RuntimeError):
    """A bounded device-side wait expired."""


class pd_params(C.Structure):
    """decode::DecodeParams (src/decode/decode_types.hpp:14-45), field for field."""
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("block_table", C.c_void_p), ("seq_lens", C.c_void_p), ("slot_ids", C.c_void_p),
        ("block_table_stride", C.c_int), ("batch", C.c_int), ("num_q_heads", C.c_int), ("num_kv_heads", C.c_int),
        ("head_dim", C.c_int), ("page_size", C.c_int), ("sm_scale", C.c_float), ("k_scale", C.c_float),
        ("v_scale", C.c_float), ("segments", C.c_void_p), ("cta_seg_begin", C.c_void_p),
        ("item_seg_begin", C.c_void_p), ("num_ctas", C.c_int), ("needs_merge", C.c_int),
        ("partial_out", C.c_void_p), ("partial_lse", C.c_void_p),
    ]


class pd_cache_config(C.Structure):
    """PagedKVCache::Config (src/decode/paged_kv_cache.hpp:19-29)."""
    _fields_ = [
        ("num_pages", C.c_int), ("page_size", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int),
        ("max_slots", C.c_int), ("max_pages_per_slot", C.c_int), ("dtype", C.c_int), ("k_scale", C.c_float),
        ("v_scale", C.c_float),
    ]


_i32p = C.POINTER(C.c_int)
_vp = C.c_void_p

# name -> (restype, argtypes); the full list of symbols include/pd_b200.h declares
SIGNATURES = {
    "pd_last_error": (C.c_char_p, []),
    "pd_version": (C.c_char_p, []),
    "pd_kv_dtype_bytes": (C.c_int, [C.c_int]),
    "pd_kv_dtype_name": (C.c_char_p, [C.c_int]),
    "pd_tile_tokens": (C.c_int, [C.c_int, C.c_int, C.c_int, _i32p]),
    "pd_wave_ctas": (C.c_int, [C.c_int, C.c_int, C.c_int, _i32p]),
    "pd_default_ctas": (C.c_int, [C.c_int, C.c_int, C.c_int, _i32p]),
    "pd_set_adaptive_cut": (C.c_int, [C.c_int]),
    "pd_adaptive_cut": (C.c_int, []),
    "pd_adaptive_cut_reset": (C.c_int, []),
    "pd_adaptive_cut_refresh": (C.c_int, [_vp]),
    "pd_adaptive_cut_table": (C.c_int, [C.c_int, _vp, _vp, C.c_int]),
    "pd_set_head_fused": (C.c_int, [C.c_int]),
    "pd_head_fused": (C.c_int, []),
    "pd_make_plan": (C.c_int, [C.c_int, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(_vp)]),
    "pd_make_plan_tiled": (C.c_int, [C.c_int, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(_vp)]),
    "pd_make_plan_weighted": (C.c_int, [C.c_int, _i32p, C.c_int, C.c_int, C.c_int, _vp, C.c_int, C.POINTER(_vp)]),
    "pd_plan_from_arrays": (C.c_int, [C.c_int, C.c_int, _i32p, C.c_int, _i32p, _i32p, C.c_int, C.POINTER(_vp)]),
    "pd_plan_free": (None, [_vp]),
    "pd_plan_num_ctas": (C.c_int, [_vp]),
    "pd_plan_tile": (C.c_int, [_vp]),
    "pd_plan_num_segments": (C.c_int, [_vp]),
    "pd_plan_num_items": (C.c_int, [_vp]),
    "pd_plan_segments": (_i32p, [_vp]),
    "pd_plan_cta_seg_begin": (_i32p, [_vp]),
    "pd_plan_item_seg_begin": (_i32p, [_vp]),
    "pd_device_plan_create": (C.c_int, [C.POINTER(_vp)]),
    "pd_device_plan_destroy": (None, [_vp]),
    "pd_device_plan_upload": (C.c_int, [_vp, _vp, C.c_int, C.c_int, _vp]),
    "pd_device_plan_bind": (C.c_int, [_vp, C.POINTER(pd_params)]),
    "pd_device_plan_reset": (C.c_int, [_vp, _vp]),
    "pd_describe_launch": (C.c_int, [C.c_int, C.POINTER(pd_params), _i32p]),
    "pd_device_plan_build": (C.c_int, [_vp, C.c_int, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "pd_device_plan_info": (C.c_int, [_vp, _i32p, _vp]),
    "pd_device_plan_fetch": (C.c_int, [_vp, C.POINTER(_vp), _vp]),
    "pd_paged_decode": (C.c_int, [C.c_int, C.POINTER(pd_params), _vp]),
    "pd_paged_decode_bounded": (C.c_int, [C.c_int, C.POINTER(pd_params), C.c_int, _vp]),
    "pd_paged_decode_static": (C.c_int, [C.c_int, C.POINTER(pd_params), C.c_int, C.c_int, _vp, _vp]),
    "pd_kernel_status": (C.c_int, [_vp, C.POINTER(C.c_uint)]),
    "pd_gather_create": (C.c_int, [C.c_int, C.c_int, C.c_size_t, C.POINTER(_vp)]),
    "pd_gather_destroy": (None, [_vp]),
    "pd_gather_handle_bytes": (C.c_int, []),
    "pd_gather_export": (C.c_int, [_vp, C.c_char_p]),
    "pd_gather_connect": (C.c_int, [_vp, C.c_char_p]),
    "pd_gather_buffer": (_vp, [_vp, C.c_int]),
    "pd_gather_epoch": (C.c_uint, [_vp]),
    "pd_paged_decode_gather": (C.c_int, [C.c_int, C.POINTER(pd_params), C.c_int, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "pd_paged_decode_gather_sync": (C.c_int, [C.c_int, C.POINTER(pd_params), C.c_int, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "pd_gather_wait": (C.c_int, [_vp, _vp]),
    "pd_gather_wait_epoch": (C.c_int, [_vp, C.c_uint, _vp]),
    "pd_stream_read": (C.c_int, [_vp, C.c_size_t, C.c_int, _vp]),
    "pd_append_tokens": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_float, C.c_float, _vp]),
    "pd_append_tokens_scaled": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_float, C.c_float, _vp, _vp, _vp]),
    "pd_paged_decode_scaled": (C.c_int, [C.c_int, C.POINTER(pd_params), C.c_int, _vp, _vp, _vp]),
    "pd_cache_set_head_scales": (C.c_int, [_vp, _vp, _vp]),
    "pd_cache_bytes_per_page": (C.c_size_t, [C.POINTER(pd_cache_config)]),
    "pd_cache_pages_for_budget": (C.c_int, [C.POINTER(pd_cache_config), C.c_size_t]),
    "pd_cache_create": (C.c_int, [C.POINTER(pd_cache_config), C.POINTER(_vp)]),
    "pd_cache_destroy": (None, [_vp]),
    "pd_cache_admit": (C.c_int, [_vp]),
    "pd_cache_append": (C.c_int, [_vp, C.c_int, _vp, _vp, C.c_int, _vp]),
    "pd_cache_append_batch": (C.c_int, [_vp, C.c_int, _i32p, C.POINTER(_vp), C.POINTER(_vp), _i32p, _vp]),
    "pd_cache_release": (C.c_int, [_vp, C.c_int]),
    "pd_cache_shuffle_free_pages": (None, [_vp, C.c_uint]),
    "pd_cache_plan": (C.c_int, [_vp, _i32p, C.c_int, C.c_int, C.c_int, _vp]),
    "pd_cache_plan_device": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "pd_cache_run": (C.c_int, [_vp, _vp, _vp, _vp]),
    "pd_cache_decode": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "pd_cache_describe_launch": (C.c_int, [_vp, _i32p]),
    "pd_cache_last_plan": (_vp, [_vp]),
    "pd_cache_params": (C.c_int, [_vp, C.POINTER(pd_params)]),
    "pd_cache_seq_len": (C.c_int, [_vp, C.c_int]),
    "pd_cache_occupied": (C.c_int, [_vp, C.c_int]),
    "pd_cache_free_pages": (C.c_int, [_vp]),
    "pd_cache_max_seq_len": (C.c_int, [_vp]),
    "pd_cache_total_bytes": (C.c_size_t, [_vp]),
    "pd_cache_config_of": (C.c_int, [_vp, C.POINTER(pd_cache_config)]),
    "pd_cache_block_table": (C.c_int, [_vp, C.c_int, _i32p, C.c_int]),
    "pd_cache_free_list": (C.c_int, [_vp, _i32p, C.c_int]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m paged_attention_b200.build` "
                "(there is no CPU or PyTorch fallback for this engine)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc):
    """Turn a pd_status into the exception the reference would raise."""
    if rc == PD_OK:
        return
    msg = lib().pd_last_error().decode()
    if rc == PD_INVALID_ARGUMENT:
        raise InvalidArgument(msg)
    if rc == PD_LENGTH_ERROR:
        raise LengthError(msg)
    if rc == PD_KERNEL_TIMEOUT:
        raise KernelTimeout(msg)
    if rc == PD_CUDA_ERROR:
        raise CudaError(msg)
    raise RuntimeError(f"pd status {rc}: {msg}")
