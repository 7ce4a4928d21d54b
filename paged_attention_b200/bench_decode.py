"""CSV benchmark CLI for the paged decode kernel, with the modes, flags and CSV schema of the
reference's bench_decode (bench/bench_decode.cu:1-19, 213-330) so rows diff directly against its
published results/h100_*.csv:

    python -m paged_attention_b200.bench_decode sweep     [--dtype fp16|fp8]      batch x seq_len sweep
    python -m paged_attention_b200.bench_decode ctas      --batch B --len L        persistent-grid size sweep
    python -m paged_attention_b200.bench_decode pagesize  --batch B --len L        page-size sweep
    python -m paged_attention_b200.bench_decode capacity  [--budget-gib G]        sequences that fit a KV budget
    python -m paged_attention_b200.bench_decode copy                               attainable read bandwidth
    python -m paged_attention_b200.bench_decode single    --batch B --len L [...] one config (the ncu target)
    python -m paged_attention_b200.bench_decode ragged    [--seqs 256]             log-uniform lengths x page sizes

Common flags: --hq 32 --hkv 8 --dim 128 --page 16 --iters 50 --dtype fp16|fp8 --ctas N (0 = default grid)
              --contiguous-pages (skip the free-list shuffle) --peak-gbps X (default: theoretical DRAM peak)

Timing protocol (bench/bench_decode.cu:121-139): warm-ups, then every iteration first streams a buffer
4x the L2 size (read-only) and then times decode (+merge) with CUDA events; the median is reported.
Like the reference, the timed iterations run one plan; unlike it, each of the 24 warm-up iterations
plans the step again, as a serving loop does every step: that is where the engine's adaptive cut takes
in the per-CTA rates of the launches before it (--plan-once: plan a single time, as the reference does).  Bandwidth counts K+V of every token, q, out and the block-table reads.
Inputs are N(0,1) fp16 (seeded), quantised at append time for fp8.
"""
import argparse
import math
import statistics
import sys

import numpy as np


def parse_args(argv):
    ap = argparse.ArgumentParser(prog="bench_decode")
    ap.add_argument("mode", nargs="?", default="sweep",
                    choices=["sweep", "ctas", "pagesize", "capacity", "copy", "single", "ragged"])
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--dtype", default=None, choices=["fp16", "fp8"])
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--contiguous-pages", action="store_true")
    ap.add_argument("--plan-once", action="store_true")
    ap.add_argument("--peak-gbps", type=float, default=0.0)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--len", type=int, default=4096)
    ap.add_argument("--budget-gib", type=float, default=1.0)
    ap.add_argument("--max-len", type=int, default=8192)
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


class Bench:
    def __init__(self, args):
        import torch
        import paged_attention_b200 as pa
        self.torch, self.pa, self.a = torch, pa, args
        prop = torch.cuda.get_device_properties(0)
        self.name, self.sms, self.l2 = prop.name, prop.multi_processor_count, prop.L2_cache_size
        self.peak = args.peak_gbps
        if not self.peak:
            try:      # theoretical 2 * memclk * buswidth, as the reference computes it
                import pynvml
                pynvml.nvmlInit()
                h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
                mem_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_MEM)
                self.peak = 2.0 * mem_mhz * 1e6 * (pynvml.nvmlDeviceGetMemoryBusWidth(h) / 8) / 1e9
            except Exception:
                self.peak = 8000.0
        self.stream = torch.cuda.current_stream().cuda_stream
        self.flush_buf = torch.zeros(max(4 * self.l2, 256 << 20), dtype=torch.uint8, device="cuda")
        print(f"# {self.name}, {self.sms} SMs, L2 {self.l2 >> 20} MiB, theoretical DRAM peak {self.peak:.0f} GB/s",
              file=sys.stderr)

    def flush(self):
        self.pa.stream_read(self.flush_buf, self.flush_buf.numel(), self.sms * 8, self.stream)

    def time_cold(self, fn, iters, before=None):
        torch = self.torch
        for _ in range(24 if before else 5):
            if before:
                before()
            self.flush()
            fn()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for s, e in ev:
            self.flush()
            s.record()
            fn()
            e.record()
        torch.cuda.synchronize()
        return statistics.median(s.elapsed_time(e) for s, e in ev)

    def setup(self, dtype, lens, page, shuffle=True):
        """A cache sized exactly to fit, filled with N(0,1) tokens, plus q / out."""
        torch, pa, a = self.torch, self.pa, self.a
        pages = [(n + page - 1) // page for n in lens]
        scale = 5.0 / 448.0 if dtype == 1 else 1.0
        cfg = pa.PagedKVCache.Config(num_pages=sum(pages), page_size=page, num_kv_heads=a.hkv, head_dim=a.dim,
                                     max_slots=len(lens), max_pages_per_slot=max(pages), dtype=pa.KVDtype(dtype),
                                     k_scale=scale, v_scale=scale)
        cache = pa.PagedKVCache(cfg)
        if shuffle:
            cache.shuffle_free_pages(42)
        gen = torch.Generator(device="cuda").manual_seed(a.seed)
        src_len = max(lens)
        k = torch.randn(src_len, a.hkv, a.dim, device="cuda", dtype=torch.float16, generator=gen)
        v = torch.randn(src_len, a.hkv, a.dim, device="cuda", dtype=torch.float16, generator=gen)
        for n in lens:      # one source for every slot, like the reference's setup (bench/bench_decode.cu:171-174)
            if not cache.append(cache.admit(), k, v, n, self.stream):
                raise SystemExit("setup: out of pages")
        q = torch.randn(len(lens), a.hq, a.dim, device="cuda", dtype=torch.float16, generator=gen)
        return cache, q, torch.zeros_like(q)

    def bytes(self, dtype, lens, page):
        a = self.a
        kv = 2.0 * sum(lens) * a.hkv * a.dim * (2 if dtype == 0 else 1)
        qo = 2.0 * len(lens) * a.hq * a.dim * 2
        bt = 4.0 * sum((n + page - 1) // page for n in lens)
        return kv + qo + bt

    @staticmethod
    def header():
        print("gpu,dtype,batch,seq_len,hq,hkv,dim,page,ctas,segments,time_us,gbps,pct_peak", flush=True)

    def run_one(self, dtype, lens, page, ctas, cache=None, q=None, out=None, seq_label=None):
        a = self.a
        own = cache is None
        if own:
            cache, q, out = self.setup(dtype, lens, page, not a.contiguous_pages)
        slots = list(range(len(lens)))
        cache.plan(slots, a.hq, ctas, self.stream)
        replan = None if a.plan_once else (lambda: cache.plan(slots, a.hq, ctas, self.stream))
        ms = self.time_cold(lambda: cache.run(q, out, self.stream), a.iters, replan)
        self.pa.kernel_status(self.stream)
        plan = cache.last_plan()
        gbps = self.bytes(dtype, lens, page) / (ms * 1e-3) / 1e9
        print(f"{self.name},{self.pa.kv_dtype_name(dtype)},{len(lens)},{seq_label or lens[0]},{a.hq},{a.hkv},{a.dim},"
              f"{page},{plan.num_ctas},{plan.num_segments},{ms * 1e3:.2f},{gbps:.1f},{100.0 * gbps / self.peak:.1f}",
              flush=True)
        if own:
            cache.close()


def main(argv=None):
    a = parse_args(sys.argv[1:] if argv is None else argv)
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench_decode: no CUDA device")
    b = Bench(a)
    pa = b.pa
    dtypes = [0, 1] if a.dtype is None else [0 if a.dtype == "fp16" else 1]
    dt = dtypes[0]

    if a.mode == "copy":
        n = 4 << 30
        buf = torch.zeros(n, dtype=torch.uint8, device="cuda")
        print("gpu,kernel,bytes,time_us,gbps,pct_peak")
        for blocks in (b.sms * 4, b.sms * 8, b.sms * 16, b.sms * 32):
            ms = b.time_cold(lambda: pa.stream_read(buf, n, blocks, b.stream), a.iters)
            gbps = n / (ms * 1e-3) / 1e9
            print(f"{b.name},read_{blocks}x512,{n},{ms * 1e3:.2f},{gbps:.1f},{100.0 * gbps / b.peak:.1f}", flush=True)
        return
    if a.mode == "sweep":
        b.header()
        shapes = [(1, 4096), (1, 16384), (1, 65536), (1, 131072), (8, 4096), (8, 16384), (8, 32768), (32, 1024),
                  (32, 4096), (32, 8192), (64, 1024), (64, 4096), (128, 1024), (128, 2048)]
        for d in dtypes:
            for batch, length in shapes:
                b.run_one(d, [length] * batch, a.page, a.ctas)
        return
    if a.mode == "single":
        b.header()
        b.run_one(dt, [a.len] * a.batch, a.page, a.ctas)
        return
    if a.mode == "ctas":
        b.header()
        lens = [a.len] * a.batch
        cache, q, out = b.setup(dt, lens, a.page, not a.contiguous_pages)
        wave = pa.wave_ctas(pa.KVDtype(dt), a.dim, a.hq // a.hkv)
        print(f"# one wave = {wave} CTAs", file=sys.stderr)
        for n in (b.sms // 2, b.sms, 2 * b.sms, 3 * b.sms, 4 * b.sms, 6 * b.sms, 8 * b.sms, wave):
            if n <= wave:
                b.run_one(dt, lens, a.page, n, cache, q, out)
        cache.close()
        return
    if a.mode == "pagesize":
        b.header()
        for ps in (1, 4, 8, 16, 32, 64, 128, 256, 1024, a.len):
            if ps <= a.len:
                b.run_one(dt, [a.len] * a.batch, ps, a.ctas)
        return
    if a.mode == "ragged":
        # sequences with lengths log-uniform in [64, 32768] (seeded), pages scattered, page-size sweep
        b.header()
        rng = np.random.default_rng(a.seed)
        lens = np.round(np.exp(rng.uniform(math.log(64), math.log(32768), a.seqs))).astype(int).tolist()
        for ps in (4, 8, 16, 32, 64):
            b.run_one(dt, lens, ps, a.ctas, seq_label=f"loguniform[64;32768]sum{sum(lens)}")
        return
    if a.mode == "capacity":
        # Sequences that fit one layer's KV budget: contiguous reserves max_len tokens per sequence
        # up front; the paged numbers come from running the allocator until it refuses.
        budget = int(a.budget_gib * (1 << 30))
        print("dtype,layout,max_len,actual_len,sequences,bytes_per_seq")
        src = torch.zeros(8192 * a.hkv * a.dim, dtype=torch.float16, device="cuda")
        for actual in (256, 512, 1024, 2048, 4096, 8192):
            per_seq = 2 * a.max_len * a.hkv * a.dim * 2
            print(f"fp16,contiguous,{a.max_len},{actual},{budget // per_seq},{per_seq}")
            for d in (0, 1):
                cfg = pa.PagedKVCache.Config(page_size=a.page, num_kv_heads=a.hkv, head_dim=a.dim, dtype=pa.KVDtype(d),
                                             k_scale=2.0 / 448.0, v_scale=2.0 / 448.0)
                cfg.num_pages = pa.PagedKVCache.pages_for_budget(cfg, budget)
                cfg.max_pages_per_slot = (a.max_len + a.page - 1) // a.page
                cfg.max_slots = cfg.num_pages
                cache = pa.PagedKVCache(cfg)
                n = 0
                while True:
                    slot = cache.admit()
                    if slot < 0 or not cache.append(slot, src, src, actual, b.stream):
                        break
                    n += 1
                print(f"{pa.kv_dtype_name(d)},paged,{a.max_len},{actual},{n},{cache.total_bytes() // n if n else 0}", flush=True)
                cache.close()
        return


if __name__ == "__main__":
    main()
