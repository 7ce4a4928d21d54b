"""ctypes access to the CPU oracle (oracle/liboracle.so) and, when it has been
built, to the reference compiled from its own sources (oracle/_ref/libpd_ref.so).

Checker code: only the tests, the smoke test and the benchmark's CPU-baseline
leg may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libpd_ref.so")

_i32p = C.POINTER(C.c_int)
_u16p = C.POINTER(C.c_uint16)
_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)


def _ptr(a, ty):
    return a.ctypes.data_as(ty)


def build_oracle():
    """Compile oracle/liboracle.so if it is missing or older than its source."""
    src = os.path.join(ORACLE_DIR, "pd_oracle.cpp")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "all"], stdout=subprocess.DEVNULL)


_oracle = None
_ref = None


def oracle():
    global _oracle
    if _oracle is None:
        build_oracle()
        L = C.CDLL(ORACLE_SO)
        L.orc_half_to_float.restype = C.c_float
        L.orc_half_to_float.argtypes = [C.c_uint16]
        L.orc_float_to_half.restype = C.c_uint16
        L.orc_float_to_half.argtypes = [C.c_float]
        L.orc_e4m3_from_float.restype = C.c_uint8
        L.orc_e4m3_from_float.argtypes = [C.c_float]
        L.orc_e4m3_to_float.restype = C.c_float
        L.orc_e4m3_to_float.argtypes = [C.c_uint8]
        L.orc_quantize_e4m3.argtypes = [_u16p, C.c_long, C.c_float, _u8p]
        L.orc_make_plan.argtypes = [C.c_int, C.c_int, _i32p, C.c_int, C.c_int, C.c_int, _i32p, _i32p, C.c_int,
                                    _i32p, _i32p, C.c_int, _i32p]
        L.orc_pool_create.restype = C.c_void_p
        L.orc_pool_create.argtypes = [C.c_int] * 4
        for n in ("destroy", "admit", "free_pages"):
            getattr(L, "orc_pool_" + n).argtypes = [C.c_void_p]
        L.orc_pool_append.argtypes = [C.c_void_p, C.c_int, C.c_int, _i32p]
        L.orc_pool_release.argtypes = [C.c_void_p, C.c_int]
        L.orc_pool_shuffle.argtypes = [C.c_void_p, C.c_uint]
        L.orc_pool_seq_len.argtypes = [C.c_void_p, C.c_int]
        L.orc_pool_occupied.argtypes = [C.c_void_p, C.c_int]
        L.orc_pool_table.argtypes = [C.c_void_p, C.c_int, _i32p, C.c_int]
        L.orc_pool_free_list.argtypes = [C.c_void_p, _i32p, C.c_int]
        L.orc_append.argtypes = [C.c_int, _u16p, _u16p, C.c_int, C.c_void_p, C.c_void_p, _i32p, C.c_int, C.c_int,
                                 C.c_int, C.c_int, C.c_float, C.c_float]
        L.orc_cpu_attention.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int]
        L.orc_paged_decode.argtypes = [C.c_int, C.c_int, _u16p, C.c_void_p, C.c_void_p, _i32p, C.c_int, _i32p,
                                       _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                       C.c_float, _f32p, C.c_int]
        L.orc_merge.argtypes = [_f32p, _f32p, C.c_int, C.c_int, _f32p]
        _oracle = L
    return _oracle


def have_ref():
    return os.path.exists(REF_SO)


def ref():
    """The reference compiled from its own sources; None when it was not built."""
    global _ref
    if _ref is None and have_ref():
        L = C.CDLL(REF_SO)
        L.ref_last_error.restype = C.c_char_p
        L.ref_e4m3_from_float.restype = C.c_uint8
        L.ref_e4m3_from_float.argtypes = [C.c_float]
        L.ref_e4m3_to_float.restype = C.c_float
        L.ref_e4m3_to_float.argtypes = [C.c_uint8]
        L.ref_half_to_float.restype = C.c_float
        L.ref_half_to_float.argtypes = [C.c_uint16]
        L.ref_float_to_half.restype = C.c_uint16
        L.ref_float_to_half.argtypes = [C.c_float]
        L.ref_quantize_e4m3.argtypes = [_u16p, C.c_long, C.c_float, _u8p]
        L.ref_cpu_attention.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int]
        L.ref_paged_cpu_decode.argtypes = [C.c_int, _u16p, C.c_void_p, C.c_void_p, _i32p, C.c_int, _i32p, _i32p,
                                           C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                           _f32p, C.c_int, C.POINTER(C.c_double)]
        L.ref_tile_tokens.argtypes = [C.c_int, C.c_int, C.c_int, _i32p]
        L.ref_default_ctas.argtypes = [C.c_int, C.c_int, C.c_int, _i32p]
        L.ref_make_plan.argtypes = [C.c_int, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p,
                                    _i32p, C.c_int, _i32p, _i32p, C.c_int, _i32p]
        L.ref_cache_create.restype = C.c_void_p
        L.ref_cache_create.argtypes = [C.c_int] * 7 + [C.c_float, C.c_float]
        L.ref_cache_destroy.argtypes = [C.c_void_p]
        L.ref_cache_admit.argtypes = [C.c_void_p]
        L.ref_cache_append.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.ref_cache_release.argtypes = [C.c_void_p, C.c_int]
        L.ref_cache_shuffle.argtypes = [C.c_void_p, C.c_uint]
        L.ref_cache_free_pages.argtypes = [C.c_void_p]
        L.ref_cache_seq_len.argtypes = [C.c_void_p, C.c_int]
        L.ref_cache_table.argtypes = [C.c_void_p, C.c_int, _i32p, C.c_int]
        L.ref_cache_pointers.argtypes = [C.c_void_p] + [C.POINTER(C.c_void_p)] * 4
        L.ref_cache_plan.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, C.c_int]
        L.ref_cache_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.ref_cache_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.ref_cache_plan_info.argtypes = [C.c_void_p, _i32p, _i32p, _i32p]
        L.ref_decoder_create.restype = C.c_void_p
        L.ref_decoder_destroy.argtypes = [C.c_void_p]
        L.ref_decoder_plan.argtypes = [C.c_void_p, C.c_int, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.ref_decoder_run.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_float, C.c_float, C.c_void_p]
        L.ref_decoder_info.argtypes = [C.c_void_p, _i32p, _i32p]
        _ref = L
    return _ref


# ---- numpy-level helpers over the oracle -------------------------------------------

def make_plan(tile, num_ctas, seq_lens, hq, hkv, lib=None):
    """(num_ctas, segments[n,4], cta_seg_begin, item_seg_begin) from the oracle planner."""
    L = lib or oracle()
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    batch = len(lens)
    total = int(sum((int(x) + tile - 1) // tile for x in lens) * hkv) if batch else 0
    seg_cap = total + 1 if num_ctas > total else num_ctas + batch * hkv + 1
    seg = np.zeros((max(seg_cap, 1), 4), np.int32)
    cta = np.zeros(num_ctas + 2, np.int32)
    item = np.zeros(batch * hkv + 1, np.int32)
    nc, ns = C.c_int(), C.c_int()
    rc = L.orc_make_plan(tile, num_ctas, _ptr(lens, _i32p), batch, hq, hkv, C.byref(nc), _ptr(seg, _i32p),
                         seg_cap, C.byref(ns), _ptr(cta, _i32p), len(cta), _ptr(item, _i32p))
    if rc == 1:
        raise ValueError("make_plan: invalid argument")
    if rc != 0:
        raise RuntimeError("make_plan: capacity")
    return nc.value, seg[:ns.value].copy(), cta[:nc.value + 1].copy(), item


def ref_make_plan(dtype, seq_lens, hq, hkv, head_dim, num_ctas):
    """Same tuple (+tile) from the reference's own make_plan; num_ctas must be > 0 without a GPU."""
    L = ref()
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    batch = len(lens)
    seg_cap = num_ctas + batch * hkv + 8
    seg = np.zeros((seg_cap, 4), np.int32)
    cta = np.zeros(num_ctas + 2, np.int32)
    item = np.zeros(batch * hkv + 1, np.int32)
    nc, tile, ns = C.c_int(), C.c_int(), C.c_int()
    rc = L.ref_make_plan(dtype, _ptr(lens, _i32p), batch, hq, hkv, head_dim, num_ctas, C.byref(nc), C.byref(tile),
                         _ptr(seg, _i32p), seg_cap, C.byref(ns), _ptr(cta, _i32p), len(cta), _ptr(item, _i32p))
    if rc == 1:
        raise ValueError(L.ref_last_error().decode())
    if rc != 0:
        raise RuntimeError(L.ref_last_error().decode())
    return nc.value, tile.value, seg[:ns.value].copy(), cta[:nc.value + 1].copy(), item


def quantize_e4m3(half_bits, scale, lib_fn=None):
    h = np.ascontiguousarray(half_bits, dtype=np.uint16)
    out = np.empty(h.shape, np.uint8)
    fn = lib_fn or oracle().orc_quantize_e4m3
    fn(_ptr(h, _u16p), h.size, C.c_float(scale), _ptr(out, _u8p))
    return out


def e4m3_to_float_table():
    L = oracle()
    return np.array([L.orc_e4m3_to_float(b) for b in range(256)], np.float32)


class PoolModel:
    """The oracle's allocator model (host half of the reference's PagedKVCache)."""

    def __init__(self, num_pages, page_size, max_slots, max_pages_per_slot):
        self.L = oracle()
        self.h = self.L.orc_pool_create(num_pages, page_size, max_slots, max_pages_per_slot)
        if not self.h:
            raise ValueError("all sizes must be positive")
        self.num_pages, self.max_pages = num_pages, max_pages_per_slot

    def __del__(self):
        if getattr(self, "h", None):
            self.L.orc_pool_destroy(self.h)
            self.h = None

    def admit(self):
        return self.L.orc_pool_admit(self.h)

    def append(self, slot, n):
        rc = self.L.orc_pool_append(self.h, slot, n, None)
        if rc == -1:
            raise ValueError("slot is not admitted")
        if rc == -2:
            raise OverflowError("sequence exceeds max_pages_per_slot")
        return rc == 1

    def release(self, slot):
        if self.L.orc_pool_release(self.h, slot) != 0:
            raise ValueError("slot is not admitted")

    def shuffle(self, seed):
        self.L.orc_pool_shuffle(self.h, seed)

    def free_pages(self):
        return self.L.orc_pool_free_pages(self.h)

    def seq_len(self, slot):
        return self.L.orc_pool_seq_len(self.h, slot)

    def table(self, slot):
        out = np.zeros(self.max_pages, np.int32)
        n = self.L.orc_pool_table(self.h, slot, _ptr(out, _i32p), len(out))
        return out[:n].copy()

    def free_list(self):
        out = np.zeros(self.num_pages, np.int32)
        n = self.L.orc_pool_free_list(self.h, _ptr(out, _i32p), len(out))
        return out[:n].copy()


def append(dtype, k_half, v_half, k_cache, v_cache, table_row, start_pos, hkv, d, ps, k_scale=1.0, v_scale=1.0):
    """Scatter n tokens ([n][hkv][d] fp16 bits) into numpy caches in place (oracle append)."""
    k = np.ascontiguousarray(k_half, np.uint16)
    v = np.ascontiguousarray(v_half, np.uint16)
    row = np.ascontiguousarray(table_row, np.int32)
    n = k.size // (hkv * d)
    oracle().orc_append(dtype, _ptr(k, _u16p), _ptr(v, _u16p), n, k_cache.ctypes.data, v_cache.ctypes.data,
                        _ptr(row, _i32p), start_pos, hkv, d, ps, C.c_float(k_scale), C.c_float(v_scale))


def paged_decode(precision, dtype, q_half, k_cache, v_cache, block_table, seq_lens, hq, hkv, d, ps,
                 sm_scale=None, k_scale=1.0, v_scale=1.0, slot_ids=None, threads=0):
    """Oracle decode over the cache bytes as stored. precision 0 = fp32 cpu_attention, 1 = double.
    q_half: uint16 [B][hq][d]. Returns float32 [B][hq][d]."""
    q = np.ascontiguousarray(q_half, np.uint16)
    bt = np.ascontiguousarray(block_table, np.int32)
    lens = np.ascontiguousarray(seq_lens, np.int32)
    B = q.size // (hq * d)
    out = np.zeros((B, hq, d), np.float32)
    sid = None
    if slot_ids is not None:
        sid_arr = np.ascontiguousarray(slot_ids, np.int32)
        sid = _ptr(sid_arr, _i32p)
    if sm_scale is None:
        sm_scale = 1.0 / np.sqrt(np.float32(d))
    oracle().orc_paged_decode(precision, dtype, _ptr(q, _u16p), k_cache.ctypes.data, v_cache.ctypes.data,
                              _ptr(bt, _i32p), bt.shape[1], _ptr(lens, _i32p), sid, B, hq, hkv, d, ps,
                              C.c_float(sm_scale), C.c_float(k_scale), C.c_float(v_scale), _ptr(out, _f32p), threads)
    return out


def cpu_attention(q, K, V, use_ref=False):
    q = np.ascontiguousarray(q, np.float32)
    K = np.ascontiguousarray(K, np.float32)
    V = np.ascontiguousarray(V, np.float32)
    T, d = K.shape
    out = np.zeros(d, np.float32)
    fn = ref().ref_cpu_attention if use_ref else oracle().orc_cpu_attention
    fn(_ptr(q, _f32p), _ptr(K, _f32p), _ptr(V, _f32p), _ptr(out, _f32p), T, d)
    return out
