"""`Decoder`: the reference's PyTorch binding (bindings/torch_decode.cu:14-81) over the C ABI.

Same constructor, `plan` / `run` split, argument order and checks; raw tensors, no PagedKVCache:

    dec = Decoder(num_q_heads, num_kv_heads, head_dim, page_size, fp8)
    dec.plan(seq_lens_cpu_int32, num_ctas=0)
    out = dec.run(q, k_cache, v_cache, block_table, seq_lens_dev, k_scale, v_scale)

q: [batch, hq, dim] fp16; k/v cache: [pages, hkv, page_size, dim] fp16 or float8_e4m3fn (or uint8 bytes);
block_table: [batch, max_pages] int32; seq_lens_dev: [batch] int32 on the device.
"""
import math

from . import decode as _d


class Decoder:
    def __init__(self, num_q_heads, num_kv_heads, head_dim, page_size, fp8):
        self.hq, self.hkv, self.dim, self.page = num_q_heads, num_kv_heads, head_dim, page_size
        self.dtype = _d.KVDtype.FP8_E4M3 if fp8 else _d.KVDtype.FP16
        self._plan = None
        self._device_plan = _d.DevicePlan()
        self._batch = 0

    def plan(self, seq_lens, num_ctas=0):
        """seq_lens: host int32 tensor [batch]; num_ctas = 0 uses the default grid."""
        import torch
        if seq_lens.device.type != "cpu" or seq_lens.dtype != torch.int32:
            raise TypeError("plan: seq_lens must be a CPU int32 tensor")
        lens = seq_lens.contiguous().numpy()
        self._plan = _d.make_plan(self.dtype, lens, self.hq, self.hkv, self.dim, num_ctas)
        self._device_plan.upload(self._plan, self.hq // self.hkv, self.dim, torch.cuda.current_stream().cuda_stream)
        self._batch = len(lens)

    def run(self, q, k_cache, v_cache, block_table, seq_lens_dev, k_scale=1.0, v_scale=1.0):
        import torch
        if not (q.is_cuda and q.dtype == torch.float16 and q.is_contiguous()):
            raise TypeError("run: q must be a contiguous CUDA fp16 tensor")
        if not (k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.is_contiguous()):
            raise TypeError("run: caches and block table must be contiguous")
        if self._plan is None or q.size(0) != self._batch:
            raise ValueError("q batch does not match the plan")
        out = torch.empty_like(q)
        p = _d.DecodeParams()
        p.q, p.out = q.data_ptr(), out.data_ptr()
        p.k_cache, p.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
        p.block_table, p.seq_lens, p.slot_ids = block_table.data_ptr(), seq_lens_dev.data_ptr(), None
        p.block_table_stride = block_table.size(1)
        p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.page_size = self._batch, self.hq, self.hkv, self.dim, self.page
        p.sm_scale = 1.0 / math.sqrt(float(self.dim))
        p.k_scale, p.v_scale = float(k_scale), float(v_scale)
        self._device_plan.bind(p)
        _d.paged_decode(self.dtype, p, torch.cuda.current_stream().cuda_stream, k_cache.size(0))
        return out

    @property
    def num_ctas(self):
        return self._plan.num_ctas if self._plan else 0

    @property
    def num_segments(self):
        return self._plan.num_segments if self._plan else 0
