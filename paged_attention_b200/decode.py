"""Python mirror of the reference's `decode::` interface over the C ABI.

Same names, argument meaning and error behaviour as src/decode/decode.hpp and
src/decode/paged_kv_cache.hpp of the reference; every call goes straight into
libpd_b200.so.  Device buffers are passed as integers (device pointers) or as
any object with a `data_ptr()` method (torch tensors); streams as an integer
cudaStream_t handle (0 = default stream).
"""
import ctypes as C
import enum

import numpy as np

from . import _lib
from ._lib import InvalidArgument, LengthError, check, pd_cache_config, pd_params

DecodeParams = pd_params


class KVDtype(enum.IntEnum):
    """decode::KVDtype (src/decode/decode_types.hpp:8)."""
    FP16 = 0
    FP8_E4M3 = 1


def kv_dtype_bytes(t):
    return _lib.lib().pd_kv_dtype_bytes(int(t))


def kv_dtype_name(t):
    return _lib.lib().pd_kv_dtype_name(int(t)).decode()


def _ptr(x):
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return int(x)


def _out_int(fn, *args):
    v = C.c_int()
    check(fn(*args, C.byref(v)))
    return v.value


def tile_tokens(dtype, head_dim, group):
    """decode::tile_tokens (src/decode/decode.hpp:30)."""
    return _out_int(_lib.lib().pd_tile_tokens, int(dtype), head_dim, group)


def wave_ctas(dtype, head_dim, group):
    """decode::wave_ctas (src/decode/decode.hpp:33)."""
    return _out_int(_lib.lib().pd_wave_ctas, int(dtype), head_dim, group)


def default_ctas(dtype, head_dim, group):
    """decode::default_ctas (src/decode/decode.hpp:35)."""
    return _out_int(_lib.lib().pd_default_ctas, int(dtype), head_dim, group)


def set_head_fused(mode):
    """Head-fused schedule of fp16 layers with 8 kv heads: 0 / False never, 1 / True where it wins
    (the default), 2 whenever the layer allows it."""
    check(_lib.lib().pd_set_head_fused(int(mode)))


def head_fused():
    """The current mode: 0, 1 or 2."""
    return int(_lib.lib().pd_head_fused())


def set_adaptive_cut(on):
    """Adaptive cut (not in the reference): device plans are cut in shares proportional to the streaming
    rate each CTA showed in earlier launches.  On by default."""
    check(_lib.lib().pd_set_adaptive_cut(int(bool(on))))


def adaptive_cut():
    return bool(_lib.lib().pd_adaptive_cut())


def adaptive_cut_reset():
    """Forget the rates learned so far."""
    check(_lib.lib().pd_adaptive_cut_reset())


def adaptive_cut_refresh(stream=0):
    """Fold the latest per-CTA readings into the weights; for loops that replay a captured device-side plan."""
    check(_lib.lib().pd_adaptive_cut_refresh(stream))


def adaptive_cut_tables():
    """[(weights, launches)] of every (kernel, grid) the adaptive cut has seen: relative share per CTA."""
    out = []
    for index in range(1 << 16):
        w = np.zeros(4096, np.float32)
        r = np.zeros(2 * 4096 + 1, np.uint64)
        n = _lib.lib().pd_adaptive_cut_table(index, w.ctypes.data, r.ctypes.data, 4096)
        if n <= 0:
            break
        out.append((w[:min(n, 4096)].copy(), int(r[2 * n]) if n <= 4096 else 0))
    return out


class DecodePlan:
    """decode::DecodePlan (src/decode/decode.hpp:21-27). Owns (or borrows) a pd_plan handle."""

    def __init__(self, handle, owned=True):
        self._h = handle
        self._owned = owned

    def __del__(self):
        if getattr(self, "_owned", False) and self._h:
            try:
                _lib.lib().pd_plan_free(self._h)
            except Exception:      # interpreter shutdown: the module is already gone
                pass
            self._h = None

    @property
    def num_ctas(self):
        return _lib.lib().pd_plan_num_ctas(self._h)

    @property
    def tile(self):
        return _lib.lib().pd_plan_tile(self._h)

    @property
    def num_segments(self):
        return _lib.lib().pd_plan_num_segments(self._h)

    @property
    def segments(self):
        n = self.num_segments
        if n == 0:
            return np.zeros((0, 4), np.int32)
        return np.ctypeslib.as_array(_lib.lib().pd_plan_segments(self._h), shape=(n, 4)).copy()

    @property
    def cta_seg_begin(self):
        return np.ctypeslib.as_array(_lib.lib().pd_plan_cta_seg_begin(self._h), shape=(self.num_ctas + 1,)).copy()

    @property
    def item_seg_begin(self):
        n = _lib.lib().pd_plan_num_items(self._h)
        return np.ctypeslib.as_array(_lib.lib().pd_plan_item_seg_begin(self._h), shape=(n + 1,)).copy()


def _lens_arg(seq_lens):
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    return lens, lens.ctypes.data_as(C.POINTER(C.c_int))


def make_plan(dtype, seq_lens, num_q_heads, num_kv_heads, head_dim, num_ctas=0):
    """decode::make_plan (src/decode/decode.hpp:38-39)."""
    lens, p = _lens_arg(seq_lens)
    h = C.c_void_p()
    check(_lib.lib().pd_make_plan(int(dtype), p, len(lens), num_q_heads, num_kv_heads, head_dim, num_ctas, C.byref(h)))
    return DecodePlan(h)


def make_plan_weighted(tile, seq_lens, num_q_heads, num_kv_heads, weights):
    """The planner with one relative share per CTA (the cut of the adaptive schedule); host arithmetic only."""
    lens, p = _lens_arg(seq_lens)
    w = np.ascontiguousarray(weights, dtype=np.float32)
    h = C.c_void_p()
    check(_lib.lib().pd_make_plan_weighted(tile, p, len(lens), num_q_heads, num_kv_heads, w.ctypes.data, len(w), C.byref(h)))
    return DecodePlan(h)


def plan_from_arrays(num_ctas, tile, segments, cta_seg_begin, item_seg_begin):
    """A DecodePlan from the arrays of a decode::DecodePlan made elsewhere (src/decode/decode.hpp:21-27),
    e.g. by the reference's own planner; the tables are checked for consistency."""
    seg = np.ascontiguousarray(segments, dtype=np.int32).reshape(-1, 4)
    cta = np.ascontiguousarray(cta_seg_begin, dtype=np.int32)
    item = np.ascontiguousarray(item_seg_begin, dtype=np.int32)
    ip = C.POINTER(C.c_int)
    h = C.c_void_p()
    check(_lib.lib().pd_plan_from_arrays(num_ctas, tile, seg.ctypes.data_as(ip), len(seg), cta.ctypes.data_as(ip),
                                         item.ctypes.data_as(ip), len(item) - 1, C.byref(h)))
    return DecodePlan(h)


def make_plan_tiled(tile, seq_lens, num_q_heads, num_kv_heads, num_ctas):
    """The planner with an explicit tile size; host arithmetic only."""
    lens, p = _lens_arg(seq_lens)
    h = C.c_void_p()
    check(_lib.lib().pd_make_plan_tiled(tile, p, len(lens), num_q_heads, num_kv_heads, num_ctas, C.byref(h)))
    return DecodePlan(h)


class DevicePlan:
    """decode::DevicePlan (src/decode/decode.hpp:44-62)."""

    def __init__(self):
        h = C.c_void_p()
        check(_lib.lib().pd_device_plan_create(C.byref(h)))
        self._h = h

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                _lib.lib().pd_device_plan_destroy(self._h)
            except Exception:      # interpreter shutdown: the module is already gone
                pass
            self._h = None

    def upload(self, plan, group, head_dim, stream=0):
        check(_lib.lib().pd_device_plan_upload(self._h, plan._h, group, head_dim, stream))

    def bind(self, params):
        check(_lib.lib().pd_device_plan_bind(self._h, C.byref(params)))

    def reset(self, stream=0):
        """After a KernelTimeout: clear the arrival counters of the in-kernel merge, which the CTA that gave
        up has left short (not in the reference, whose kernels have no bounded waits)."""
        check(_lib.lib().pd_device_plan_reset(self._h, stream))

    def build(self, dtype, d_seq_lens, batch, num_q_heads, num_kv_heads, head_dim=128, num_ctas=0, d_slot_ids=None,
              stream=0):
        """Cut the step's plan on the device from device-resident lengths (no counterpart in the
        reference): same arrays as make_plan + upload, no host copy, no wait, capturable in a CUDA graph
        once the buffers have grown to the largest batch."""
        check(_lib.lib().pd_device_plan_build(self._h, int(dtype), _ptr(d_seq_lens), _ptr(d_slot_ids), batch, num_q_heads,
                                              num_kv_heads, head_dim, num_ctas, stream))

    def info(self, stream=0):
        """(CTAs with work, segments, most pieces of any (row, kv head), 1 + first row with a bad length) of a
        plan built on the device; waits for the stream."""
        out = (C.c_int * 4)()
        check(_lib.lib().pd_device_plan_info(self._h, out, stream))
        return tuple(out)

    def fetch(self, stream=0):
        """The device-built plan as a host DecodePlan; waits for the stream."""
        h = C.c_void_p()
        check(_lib.lib().pd_device_plan_fetch(self._h, C.byref(h), stream))
        return DecodePlan(h)


def paged_decode(dtype, params, stream=0, num_pages=0, d_k_scales=None, d_v_scales=None):
    """decode::paged_decode (src/decode/decode.hpp:66).  d_k_scales / d_v_scales (not in the reference):
    device arrays of one dequantisation scale per kv head, replacing params.k_scale / v_scale."""
    if d_k_scales is None and d_v_scales is None:
        check(_lib.lib().pd_paged_decode_bounded(int(dtype), C.byref(params), num_pages, stream))
    else:
        check(_lib.lib().pd_paged_decode_scaled(int(dtype), C.byref(params), num_pages, _ptr(d_k_scales), _ptr(d_v_scales),
                                                stream))


def paged_decode_static(dtype, params, plan, stream=0, num_pages=0, d_status=None):
    """Decode + merge with the library's built-in split-row workspace instead of params.partial_out /
    partial_lse: no device allocation happens in this call (there is no counterpart in the reference).
    For callers whose process has no HBM left to allocate from, or whose step loop forbids
    cudaMalloc/cudaFree.  `plan` is the DecodePlan the params were bound from: its segment count sizes the
    workspace (an integer count is accepted too; the kernels check it against the plan they walk and report
    status code 6 instead of storing outside the workspace).  Raises InvalidArgument when the plan needs
    more than the built-in 8 MiB."""
    num_segments = plan.num_segments if hasattr(plan, "num_segments") else int(plan)
    check(_lib.lib().pd_paged_decode_static(int(dtype), C.byref(params), num_segments, num_pages, _ptr(d_status), stream))


LAUNCH_SCHEDULES = ("caller's plan", "head-fused rows", "caller's plan in adaptive shares")


def describe_launch(dtype, params):
    """What a decode of these params would launch: dict with the schedule, grid, tile and kernel shape."""
    out = (C.c_int * 8)()
    check(_lib.lib().pd_describe_launch(int(dtype), C.byref(params), out))
    return _launch_dict(out)


def _launch_dict(out):
    return {"schedule": LAUNCH_SCHEDULES[out[0]], "grid": out[1], "tile_tokens": out[2], "kv_heads_per_tile": out[3],
            "consumer_warps": out[4], "stages": out[5], "ctas_per_sm": out[6],
            "merge": ("none", "merge kernel", "inside the decode kernel", "per row: in-kernel up to 4 pieces, else merge kernel")[out[7]]}


def kernel_status(stream=0):
    """Raises KernelTimeout if a bounded device-side wait of an earlier decode expired."""
    st = C.c_uint()
    check(_lib.lib().pd_kernel_status(stream, C.byref(st)))
    return st.value


def stream_read(d_buf, nbytes, blocks, stream=0):
    """Read-only streaming pass (the reference benchmark's "copy" probe)."""
    check(_lib.lib().pd_stream_read(_ptr(d_buf), nbytes, blocks, stream))


def append_tokens(dtype, d_k, d_v, k_cache, v_cache, d_block_table_row, start_pos, n, num_kv_heads, head_dim,
                  page_size, k_scale=1.0, v_scale=1.0, stream=0, d_k_scales=None, d_v_scales=None):
    """append_kernel<KV> (src/decode/paged_kv_cache.cu:25-39) on caller-owned buffers.  d_k_scales /
    d_v_scales (not in the reference): device arrays of one quantisation scale per kv head."""
    check(_lib.lib().pd_append_tokens_scaled(int(dtype), _ptr(d_k), _ptr(d_v), _ptr(k_cache), _ptr(v_cache),
                                             _ptr(d_block_table_row), start_pos, n, num_kv_heads, head_dim, page_size,
                                             k_scale, v_scale, _ptr(d_k_scales), _ptr(d_v_scales), stream))


class PagedKVCache:
    """decode::PagedKVCache (src/decode/paged_kv_cache.hpp:17-93)."""

    class Config:
        def __init__(self, num_pages=0, page_size=0, num_kv_heads=0, head_dim=0, max_slots=0, max_pages_per_slot=0,
                     dtype=KVDtype.FP16, k_scale=1.0, v_scale=1.0):
            self.num_pages, self.page_size, self.num_kv_heads, self.head_dim = num_pages, page_size, num_kv_heads, head_dim
            self.max_slots, self.max_pages_per_slot = max_slots, max_pages_per_slot
            self.dtype, self.k_scale, self.v_scale = dtype, k_scale, v_scale

        def _c(self):
            return pd_cache_config(self.num_pages, self.page_size, self.num_kv_heads, self.head_dim, self.max_slots,
                                   self.max_pages_per_slot, int(self.dtype), self.k_scale, self.v_scale)

    def __init__(self, cfg):
        self._h = None
        self._cfg = cfg
        h = C.c_void_p()
        c = cfg._c()
        check(_lib.lib().pd_cache_create(C.byref(c), C.byref(h)))
        self._h = h

    def close(self):
        if self._h:
            _lib.lib().pd_cache_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:          # interpreter shutdown: the module is already gone
            pass

    @staticmethod
    def bytes_per_page(cfg):
        c = cfg._c()
        return _lib.lib().pd_cache_bytes_per_page(C.byref(c))

    @staticmethod
    def pages_for_budget(cfg, budget_bytes):
        c = cfg._c()
        return _lib.lib().pd_cache_pages_for_budget(C.byref(c), budget_bytes)

    def admit(self):
        return _lib.lib().pd_cache_admit(self._h)

    def append(self, slot, d_k, d_v, n, stream=0):
        """True when appended, False (nothing changed) when the pool is out of pages."""
        rc = _lib.lib().pd_cache_append(self._h, slot, _ptr(d_k), _ptr(d_v), n, stream)
        if rc == _lib.PD_OUT_OF_PAGES:
            return False
        check(rc)
        return True

    def append_batch(self, slots, d_ks, d_vs, ns, stream=0):
        """One decode step's appends for many slots in one call (stream-ordered, no host wait).
        True when appended, False (nothing changed) when the pool cannot hold all of them."""
        count = len(slots)
        s = np.ascontiguousarray(slots, dtype=np.int32)
        n = np.ascontiguousarray(ns, dtype=np.int32)
        ks = (C.c_void_p * count)(*[_ptr(x) for x in d_ks])
        vs = (C.c_void_p * count)(*[_ptr(x) for x in d_vs])
        rc = _lib.lib().pd_cache_append_batch(self._h, count, s.ctypes.data_as(C.POINTER(C.c_int)), ks, vs,
                                              n.ctypes.data_as(C.POINTER(C.c_int)), stream)
        if rc == _lib.PD_OUT_OF_PAGES:
            return False
        check(rc)
        return True

    def release(self, slot):
        check(_lib.lib().pd_cache_release(self._h, slot))

    def shuffle_free_pages(self, seed):
        _lib.lib().pd_cache_shuffle_free_pages(self._h, seed)

    def set_head_scales(self, k_scales, v_scales):
        """One fp8 scale per kv head instead of one per tensor (not in the reference); None, None restores
        the per-tensor scales.  Only while the cache is empty."""
        arrays = []
        for scales in (k_scales, v_scales):
            a = None if scales is None else np.ascontiguousarray(scales, dtype=np.float32)
            if a is not None and a.shape != (self._cfg.num_kv_heads,):
                raise _lib.InvalidArgument("set_head_scales: one scale per kv head is needed")
            arrays.append(a)
        check(_lib.lib().pd_cache_set_head_scales(self._h, *[None if a is None else a.ctypes.data for a in arrays]))

    def plan(self, slots, num_q_heads, num_ctas=0, stream=0):
        s = np.ascontiguousarray(slots, dtype=np.int32)
        check(_lib.lib().pd_cache_plan(self._h, s.ctypes.data_as(C.POINTER(C.c_int)), len(s), num_q_heads, num_ctas, stream))

    def plan_device(self, batch, num_q_heads, num_ctas=0, d_slot_ids=None, stream=0):
        """plan() cut on the device from the cache's device-side lengths (slots 0..batch-1, or the device
        array d_slot_ids); nothing is copied from the host and the call does not wait."""
        check(_lib.lib().pd_cache_plan_device(self._h, _ptr(d_slot_ids), batch, num_q_heads, num_ctas, stream))

    def run(self, d_q, d_out, stream=0):
        check(_lib.lib().pd_cache_run(self._h, _ptr(d_q), _ptr(d_out), stream))

    def decode(self, d_q, d_out, batch, num_q_heads, num_ctas=0, stream=0):
        check(_lib.lib().pd_cache_decode(self._h, _ptr(d_q), _ptr(d_out), batch, num_q_heads, num_ctas, stream))

    def describe_launch(self):
        """What the next run() of the current plan launches (see describe_launch)."""
        out = (C.c_int * 8)()
        check(_lib.lib().pd_cache_describe_launch(self._h, out))
        return _launch_dict(out)

    def last_plan(self):
        h = _lib.lib().pd_cache_last_plan(self._h)
        return DecodePlan(C.c_void_p(h), owned=False) if h else None

    def params(self):
        p = pd_params()
        check(_lib.lib().pd_cache_params(self._h, C.byref(p)))
        return p

    def seq_len(self, slot):
        return _lib.lib().pd_cache_seq_len(self._h, slot)

    def occupied(self, slot):
        return bool(_lib.lib().pd_cache_occupied(self._h, slot))

    def free_pages(self):
        return _lib.lib().pd_cache_free_pages(self._h)

    def max_seq_len(self):
        return _lib.lib().pd_cache_max_seq_len(self._h)

    def total_bytes(self):
        return _lib.lib().pd_cache_total_bytes(self._h)

    def config(self):
        return self._cfg

    def block_table(self, slot):
        cap = self._cfg.max_pages_per_slot
        out = np.zeros(cap, np.int32)
        n = _lib.lib().pd_cache_block_table(self._h, slot, out.ctypes.data_as(C.POINTER(C.c_int)), cap)
        return out[:n].copy()

    def free_list(self):
        cap = self._cfg.num_pages
        out = np.zeros(cap, np.int32)
        n = _lib.lib().pd_cache_free_list(self._h, out.ctypes.data_as(C.POINTER(C.c_int)), cap)
        return out[:n].copy()


__all__ = ["KVDtype", "DecodeParams", "DecodePlan", "DevicePlan", "PagedKVCache", "InvalidArgument", "LengthError",
           "kv_dtype_bytes", "kv_dtype_name", "tile_tokens", "wave_ctas", "default_ctas", "make_plan",
           "make_plan_tiled", "make_plan_weighted", "plan_from_arrays", "paged_decode", "paged_decode_static", "append_tokens", "stream_read", "kernel_status", "describe_launch", "set_head_fused", "head_fused",
           "set_adaptive_cut", "adaptive_cut", "adaptive_cut_reset", "adaptive_cut_refresh", "adaptive_cut_tables"]
