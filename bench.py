#!/usr/bin/env python
"""Benchmark of the paged split-KV decode layer (one step = one decode layer over one batch).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c5|small|...]

Prints ONE JSON line.  Metric: achieved HBM GB/s over the algorithmic bytes of the
layer (K+V of every token once, q and out, block-table entries), with the layer
time in `ms_per_step`.  Inputs are synthetic, seeded, N(0,1), of the shape the
workload names; pages are scattered through a pool sized exactly to fit.

N > 1 (launched by torch.distributed.run, one rank per GPU): by default the batch
is sharded, every rank holds its own full-size layer shard (weak scaling) and the
outputs are gathered inside the timed step - by default by the decode kernel itself
(peer stores into every rank's buffer, `--gather peer`), or by ncclAllGather
(`--gather nccl`); `--shard heads` splits the KV heads of one fixed problem instead
(strong scaling, workload c5).  After the timed region every rank checks its gathered
buffer bit for bit against an NCCL all-gather of the ranks' local outputs and two
sampled rows against the CPU oracle (`gather_check`), and the 70B-shaped layer with
its KV heads sharded over the same ranks is measured in the same process group
(`c5_heads`, strong scaling against the unsharded layer on one GPU).

`--impl reference` times the reference's own CPU attention (compiled from its
sources into oracle/_ref, else the oracle port) on a bounded sample of the same
workload, on the host cores of this box.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (dtype, batch, seq_len, hq, hkv, page, description)
    "c2": (0, 64, 8192, 32, 8, 16, "Llama-3-8B layer, batch 64 x 8192, fp16 KV, 16-token pages scattered"),
    "c3": (1, 128, 4096, 32, 8, 16, "Llama-3-8B layer, batch 128 x 4096, fp8 e4m3 KV, 16-token pages scattered"),
    "c5": (1, 256, 16384, 64, 8, 16, "Llama-3-70B-shaped layer, batch 256 x 16384, fp8 e4m3 KV, kv heads sharded"),
    "c2-onepage": (0, 64, 8192, 32, 8, 8192, "c2 with one contiguous 8192-token page per sequence"),
    "small": (0, 8, 8192, 32, 8, 16, "profiling case: batch 8 x 8192 fp16 (268 MB of KV, larger than L2)"),
    "small-fp8": (1, 16, 8192, 32, 8, 16, "profiling case: batch 16 x 8192 fp8 (268 MB of KV)"),
    "small-wide": (0, 64, 1024, 32, 8, 16, "profiling case of the head-fused schedule: batch 64 x 1024 fp16 (268 MB of KV)"),
    "small-wide-fp8": (1, 64, 2048, 32, 8, 16, "profiling case of the head-fused e4m3 schedule: batch 64 x 2048 fp8 (268 MB of KV)"),
    "single": (0, 1, 16384, 32, 8, 16, "profiling case of the merge kernel: one sequence of 16384 tokens spread over the grid"),
}
DTYPE_NAMES = {0: "f16", 1: "f8e4m3"}
ARITHMETIC = {0: "mma.m16n8k16 f16 x f16 -> f32 accumulate, softmax in f32; KV stored as fp16",
              1: "e4m3 bytes widened to f16 in registers (exact), then mma.m16n8k16 f16 x f16 -> f32 accumulate, softmax in f32; "
                 "KV stored as fp8 e4m3"}


def algorithmic_bytes(dtype, lens, hq, hkv, page, d=128):
    """bytes = 2*sum(len)*Hkv*d*elem + 2*B*Hq*d*2 + 4*sum(ceil(len/page)) (bench/bench_decode.cu:186-191 of the reference)."""
    elem = 2 if dtype == 0 else 1
    return (2 * sum(lens) * hkv * d * elem + 2 * len(lens) * hq * d * 2
            + 4 * sum((n + page - 1) // page for n in lens))


class ClockSampler:
    """Reads SM clocks and clock-event (throttle) reasons through NVML every few milliseconds
    while the GPU is under load.  Read-only: no setting of the GPU is touched."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index, period=0.004):
        self.sm, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.period = period
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception as e:   # NVML missing: report that instead of a number
            self.error = str(e)

    def _run(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        if not self.thread:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "error", "?")]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.sm), "power_w_max": max(self.power) if self.power else None,
                "reasons": sorted(self.reasons)}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ---------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's cpu_attention over a bounded sample
# ---------------------------------------------------------------------------------------------

def checker():
    """The CPU oracle's ctypes wrapper (tests/oracle_lib.py): checker and CPU baseline only, never on the
    measured path."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    return oracle_lib


def cpu_sample_inputs(dtype, rows, L, hq, hkv, page, seed=7):
    """Host-side paged cache for `rows` sequences of length L, N(0,1) fp16 values, scattered pages."""
    ol = checker()
    rng = np.random.default_rng(seed)
    pages = (L + page - 1) // page
    perm = rng.permutation(rows * pages).astype(np.int32).reshape(rows, pages)
    scale = 5.0 / 448.0 if dtype == 1 else 1.0
    np_dt = np.uint16 if dtype == 0 else np.uint8
    kc = np.zeros(rows * pages * hkv * page * 128, np_dt)
    vc = np.zeros_like(kc)
    for r in range(rows):
        k = rng.standard_normal((L, hkv, 128), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((L, hkv, 128), dtype=np.float32).astype(np.float16)
        ol.append(dtype, k.view(np.uint16), v.view(np.uint16), kc, vc, perm[r], 0, hkv, 128, page, scale, scale)
    q = rng.standard_normal((rows, hq, 128), dtype=np.float32).astype(np.float16)
    return q, kc, vc, perm, scale


def run_cpu_attention(dtype, q, kc, vc, bt, lens, hq, hkv, page, scale, threads):
    """Returns (seconds of attention calls, kind, out) using oracle/_ref when present, else the oracle port."""
    ol = checker()
    rows = q.shape[0]
    out = np.zeros((rows, hq, 128), np.float32)
    lens_a = np.ascontiguousarray(lens, np.int32)
    bt = np.ascontiguousarray(bt, np.int32)
    R = ol.ref()
    i32p, u16p, f32p = C.POINTER(C.c_int), C.POINTER(C.c_uint16), C.POINTER(C.c_float)
    if R is not None:
        rws = np.arange(rows, dtype=np.int32)
        secs = C.c_double()
        R.ref_paged_cpu_decode(dtype, q.view(np.uint16).ctypes.data_as(u16p), kc.ctypes.data, vc.ctypes.data,
                               bt.ctypes.data_as(i32p), bt.shape[1], lens_a.ctypes.data_as(i32p),
                               rws.ctypes.data_as(i32p), rows, hq, hkv, 128, page, C.c_float(scale), C.c_float(scale),
                               out.ctypes.data_as(f32p), threads, C.byref(secs))
        return secs.value, "reference", out
    t0 = time.perf_counter()
    out = ol.paged_decode(0, dtype, q.view(np.uint16), kc, vc, bt, lens_a, hq, hkv, 128, page, k_scale=scale,
                          v_scale=scale, threads=threads)
    return time.perf_counter() - t0, "port", out


def cpu_leg(dtype, L, hq, hkv, page, batch, target_seconds=10.0):
    """Times the CPU attention on a bounded sample: calibrates on one row, then sizes the sample.  Also one
    sequence x all query heads on a single thread, which is how the reference itself runs cpu_attention."""
    cores = os.cpu_count() or 1
    q, kc, vc, bt, scale = cpu_sample_inputs(dtype, 1, L, hq, hkv, page)
    t1, kind, _ = run_cpu_attention(dtype, q, kc, vc, bt, [L], hq, hkv, page, scale, cores)
    t_single, _, _ = run_cpu_attention(dtype, q, kc, vc, bt, [L], hq, hkv, page, scale, 1)
    one_row_bytes = algorithmic_bytes(dtype, [L], hq, hkv, page)
    rows = int(max(1, min(batch, target_seconds / max(t1, 1e-6))))
    reps = 1
    if rows > 1:
        q, kc, vc, bt, scale = cpu_sample_inputs(dtype, rows, L, hq, hkv, page)
        secs, kind, _ = run_cpu_attention(dtype, q, kc, vc, bt, [L] * rows, hq, hkv, page, scale, cores)
        # a fast host finishes the whole batch early: repeat it until the CPU has worked for a few seconds
        reps = int(max(1, min(50, target_seconds / max(secs, 1e-6))))
        if reps > 1:
            secs = sum(run_cpu_attention(dtype, q, kc, vc, bt, [L] * rows, hq, hkv, page, scale, cores)[0]
                       for _ in range(reps)) / reps
    else:
        secs = t1
    nbytes = algorithmic_bytes(dtype, [L] * rows, hq, hkv, page)
    what = "cpu_attention from the reference sources" if kind == "reference" else "oracle port of cpu_attention"
    return {"value": nbytes / secs / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{rows} of {batch} sequences x {hq} q heads at length {L} "
                      f"({what}, OpenMP over (row, q head), gather excluded, {secs:.2f} s per pass, mean of {reps} passes)",
            "single_thread": {"value": one_row_bytes / t_single / 1e9, "unit": "GB/s", "cores": 1,
                              "sample": f"1 of {batch} sequences x {hq} q heads at length {L} on one thread, as the reference "
                                        f"runs it ({t_single:.3f} s; the whole layer would take {t_single * batch:.1f} s)"}}


def reference_arm(args, wl):
    dtype, B, L, hq, hkv, page, desc = wl
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    # calibrate the sample so that warmup + steps finish within a few minutes
    q, kc, vc, bt, scale = cpu_sample_inputs(dtype, 1, L, hq, hkv, page)
    t1, kind, _ = run_cpu_attention(dtype, q, kc, vc, bt, [L], hq, hkv, page, scale, cores)
    budget = 120.0 / max(1, args.steps + args.warmup)
    rows = int(max(1, min(B, budget / max(t1, 1e-6))))
    q, kc, vc, bt, scale = cpu_sample_inputs(dtype, rows, L, hq, hkv, page)
    for _ in range(args.warmup):
        run_cpu_attention(dtype, q, kc, vc, bt, [L] * rows, hq, hkv, page, scale, cores)
    secs = [run_cpu_attention(dtype, q, kc, vc, bt, [L] * rows, hq, hkv, page, scale, cores)[0] for _ in range(args.steps)]
    nbytes = algorithmic_bytes(dtype, [L] * rows, hq, hkv, page)
    per = sum(secs) / len(secs)
    value = nbytes / per / 1e9
    sample = (f"each step = {rows} of {B} sequences x {hq} q heads at length {L}; "
              f"{'cpu_attention compiled from the reference sources (oracle/_ref)' if kind == 'reference' else 'oracle port of cpu_attention'}, "
              f"{cores} OpenMP threads, gather excluded")
    print(json.dumps({
        "impl": "reference", "metric": "paged_decode_achieved_hbm_bandwidth", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

class _Dev:
    """Zero-copy torch view of raw device memory."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


class Layer:
    """One decode layer resident on this GPU: a cache filled with seeded N(0,1) tokens in scattered pages, the
    query rows, an output buffer, and the plan, driven through the plan API as a serving engine does (plan
    once per step, run per layer)."""

    def __init__(self, torch, pa, dtype, B, L, hq, hkv, page, seed, stream, contiguous=False, ctas=0, shared_source=False):
        self.torch, self.pa = torch, pa
        self.dtype, self.B, self.L, self.hq, self.hkv, self.page, self.stream = dtype, B, L, hq, hkv, page, stream
        self.group = hq // hkv
        self.lens = [L] * B
        pages = (L + page - 1) // page
        self.scale = 5.0 / 448.0 if dtype == 1 else 1.0
        self.cfg = pa.PagedKVCache.Config(num_pages=pages * B, page_size=page, num_kv_heads=hkv, head_dim=128, max_slots=B,
                                          max_pages_per_slot=pages, dtype=pa.KVDtype(dtype), k_scale=self.scale,
                                          v_scale=self.scale)
        self.cache = pa.PagedKVCache(self.cfg)
        if not contiguous:
            self.cache.shuffle_free_pages(42)
        gen = torch.Generator(device="cuda").manual_seed(seed)
        k = v = None
        for b in range(B):
            if k is None or not shared_source:      # shared_source: every slot gets the same tokens (as the reference's bench does)
                k = torch.randn(L, hkv, 128, device="cuda", dtype=torch.float16, generator=gen)
                v = torch.randn(L, hkv, 128, device="cuda", dtype=torch.float16, generator=gen)
            slot = self.cache.admit()
            if not self.cache.append(slot, k, v, L, stream):
                raise SystemExit("bench.py: pool out of pages")
        del k, v
        self.q_host = torch.randn(B, hq, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(seed + 99)).pin_memory()
        self.out_host = torch.empty_like(self.q_host).pin_memory()
        self.q = self.q_host.cuda()
        self.out = torch.zeros_like(self.q)
        self.plan = pa.make_plan(pa.KVDtype(dtype), self.lens, hq, hkv, 128, ctas)
        self.dplan = pa.DevicePlan()
        self.params = self.cache.params()
        self.params.q, self.params.out = self.q.data_ptr(), self.out.data_ptr()
        self.params.batch, self.params.num_q_heads = B, hq
        self.replan()
        self.bytes = algorithmic_bytes(dtype, self.lens, hq, hkv, page)

    def replan(self):
        self.dplan.upload(self.plan, self.group, 128, self.stream)
        self.dplan.bind(self.params)

    def decode(self):
        self.pa.paged_decode(self.pa.KVDtype(self.dtype), self.params, self.stream, self.cfg.num_pages)

    def launch(self):
        return self.pa.describe_launch(self.pa.KVDtype(self.dtype), self.params)

    def oracle_rows(self, rows):
        """Checker: the oracle's output for a few rows, from the cache bytes as stored on the device."""
        ol = checker()
        torch, cfg = self.torch, self.cfg
        elem = 2 if self.dtype == 0 else 1
        page_elems = self.hkv * self.page * 128
        t_dt, n_dt = (torch.float16, np.uint16) if self.dtype == 0 else (torch.uint8, np.uint8)
        nbytes = cfg.num_pages * page_elems * elem
        kpool = torch.as_tensor(_Dev(self.params.k_cache, nbytes), device="cuda").view(t_dt).view(cfg.num_pages, page_elems)
        vpool = torch.as_tensor(_Dev(self.params.v_cache, nbytes), device="cuda").view(t_dt).view(cfg.num_pages, page_elems)
        pages = (self.L + self.page - 1) // self.page
        out = {}
        for row in rows:
            table = torch.from_numpy(self.cache.block_table(row).astype(np.int64)).cuda()
            kc = kpool[table].cpu().numpy().view(n_dt).reshape(-1)
            vc = vpool[table].cpu().numpy().view(n_dt).reshape(-1)
            q = self.q[row:row + 1].cpu().numpy()
            out[row] = ol.paged_decode(1, self.dtype, q.view(np.uint16), kc, vc, np.arange(pages, dtype=np.int32)[None],
                                       [self.L], self.hq, self.hkv, 128, self.page, k_scale=self.scale, v_scale=self.scale)[0]
        return out

    def close(self):
        self.cache.close()


class Gather:
    """Output gather of one sharded layer: peer stores by the decode kernel, or ncclAllGather."""

    def __init__(self, torch, pa, dist, layer, shard, mode, world, rank):
        self.torch, self.pa, self.dist, self.layer, self.shard, self.world, self.rank = torch, pa, dist, layer, shard, world, rank
        self.rows_total = layer.B if shard == "heads" else layer.B * world
        self.heads_total = layer.hq * world if shard == "heads" else layer.hq
        self.full_bytes = self.rows_total * self.heads_total * 128 * 2
        self.head_off = rank * layer.hq if shard == "heads" else 0
        self.row_off = 0 if shard == "heads" else rank * layer.B
        self.note = None
        self.gg = None
        self.mode = mode
        if mode == "peer":
            # Peer stores need CUDA IPC mappings between all GPUs of the node.  If any rank cannot set them
            # up, every rank falls back to ncclAllGather (and the JSON line says so).
            from paged_attention_b200.sharding import GatherGroup
            ok = torch.ones(1, device="cuda")
            try:
                self.gg = GatherGroup(self.full_bytes)
            except Exception as e:
                ok.zero_()
                self.note = "peer setup failed (%s); fell back to ncclAllGather" % str(e)[:120]
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                if self.gg is not None:
                    self.gg.close()
                    self.gg = None
                self.mode = "nccl"
                self.note = self.note or "a peer could not set up IPC mappings; fell back to ncclAllGather"
        if self.mode == "nccl":
            self.gathered = torch.empty((world * layer.B, layer.hq, 128), dtype=torch.float16, device="cuda")
        else:
            self.views = [torch.as_tensor(_Dev(self.gg.buffer_ptr(i), self.full_bytes), device="cuda") for i in range(4)]
            self.share = self.full_bytes // world      # each rank returns its 1/world of the gathered result to the host
            self.full_host = torch.empty(self.share, dtype=torch.uint8).pin_memory()

    def decode(self, sync=False):
        """One layer with its rows stored into every rank's buffer.  sync: the kernel launched behind the decode
        also waits for the peers' rows (the step is complete when it has run); else `wait` does, later."""
        ly = self.layer
        if self.mode == "peer":
            self.gg.decode(self.pa.KVDtype(ly.dtype), ly.params, self.heads_total, self.head_off, self.row_off, ly.stream,
                           ly.cfg.num_pages, sync=sync)
        else:
            ly.decode()
            self.dist.all_gather_into_tensor(self.gathered, ly.out)

    def wait(self, back=0):
        """Wait (bounded, on the stream) until every rank's rows of the step `back` steps ago have landed."""
        if self.mode == "peer":
            self.gg.wait_epoch(self.gg.epoch - back, self.layer.stream)

    def last_view(self):
        """The gathered result of the last step as a [rows][heads][128] fp16 tensor, in the full layout."""
        torch = self.torch
        if self.mode == "peer":
            return self.views[self.gg.epoch % 4].view(torch.float16).view(self.rows_total, self.heads_total, 128)
        g = self.gathered
        if self.shard == "heads":
            return g.view(self.world, self.layer.B, self.layer.hq, 128).permute(1, 0, 2, 3).reshape(self.rows_total, self.heads_total, 128)
        return g

    def check(self):
        """After the timed region: this rank's gathered buffer against an NCCL all-gather of the ranks' local
        outputs of the same plan (bit for bit), and two of this rank's rows against the CPU oracle."""
        torch, dist, ly = self.torch, self.dist, self.layer
        self.decode(sync=True)
        torch.cuda.synchronize()
        got = self.last_view().clone()
        ly.out.zero_()
        ly.decode()                                   # local output of the same device plan
        parts = torch.empty((self.world * ly.B, ly.hq, 128), dtype=torch.float16, device="cuda")
        dist.all_gather_into_tensor(parts, ly.out)
        if self.shard == "heads":
            want = parts.view(self.world, ly.B, ly.hq, 128).permute(1, 0, 2, 3).reshape(self.rows_total, self.heads_total, 128)
        else:
            want = parts
        equal = bool(torch.equal(got, want))
        rows = (0, ly.B - 1)
        oracle = ly.oracle_rows(rows)
        worst = 0.0
        for row, w in oracle.items():
            mine = got[row + self.row_off, self.head_off:self.head_off + ly.hq].float().cpu().numpy()
            worst = max(worst, float(np.abs(mine - w).max()))
        flags = torch.tensor([1.0 if equal else 0.0, -worst], device="cuda")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        all_equal, all_worst = bool(flags[0].item() == 1.0), float(-flags[1].item())
        return {"ok": all_equal and all_worst <= 2e-3, "bit_exact_vs_nccl_all_gather": all_equal,
                "max_abs_vs_oracle": all_worst, "tolerance": 2e-3,
                "checked": "every rank: its whole gathered buffer vs ncclAllGather of the local outputs; rows %s of its shard vs the CPU oracle"
                           % (list(rows),)}

    def close(self):
        if self.gg is not None:
            self.dist.barrier()
            self.gg.close()


def our_arm(args, wl):
    import torch
    import paged_attention_b200 as pa

    dtype, B, L, hq, hkv, page, desc = wl
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pa.set_adaptive_cut(args.adaptive_cut == "on")
    if args.workload in ("small-wide", "small-wide-fp8"):
        pa.set_head_fused(2)      # the profiling case of the head-fused kernel is too short for it to be chosen by itself
    stream = torch.cuda.current_stream().cuda_stream

    flush_buf = torch.zeros(512 << 20, dtype=torch.uint8, device="cuda")

    def flush():   # read-only pass over 4x L2: the next kernel starts cold and L2 holds no dirty lines
        pa.stream_read(flush_buf, flush_buf.numel(), 148 * 8, stream)

    rendezvous = torch.zeros(1, device="cuda")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, before=None, after_last=None):
        """Per step: flush (outside the events), ranks rendezvous, events around fn().  after_last runs inside
        the last step's events.  Returns the per-step milliseconds of this rank."""
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for i, (s, e) in enumerate(ev):
            if before:
                before()
            flush()
            if world > 1:      # device-side rendezvous: all ranks enter the step together, so one rank's
                dist.all_reduce(rendezvous)   # slower flush is not charged to the others' step
            s.record()
            fn()
            if after_last and i == steps - 1:
                after_last()
            e.record()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in ev]

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def measure(layer, gather, steps, warmup, settle_to=24):
        """The step protocol for one layer (+ gather).  Returns a dict of per-step milliseconds (max over ranks)."""
        if gather is None:
            step = layer.decode
        else:
            # a step is complete when every rank's rows are in this rank's buffer: decode, then ONE dependent
            # kernel that announces this rank's rows and waits for the others'
            def step():
                gather.decode(sync=True)
        # W warm-up steps as asked (at least 3), preceded by as many settling steps as it takes to make
        # `settle_to` untimed steps in all: the adaptive cut folds in one reading per plan and needs about 20
        # to settle, as it would have in any serving loop.  All of them are reported as warm-up.
        untimed = max(max(warmup, 3), settle_to if pa.adaptive_cut() else 0)
        for _ in range(untimed):
            layer.replan()
            flush()
            step()
        barrier()
        t0 = time.perf_counter()
        ms = timed(step, steps, before=layer.replan if args.replan_every_step else None)
        barrier()
        wall = time.perf_counter() - t0
        res = {"untimed": untimed, "wall": wall, "ms_list": ms}
        res["ms_kernel"] = timed(layer.decode, steps)          # the decode (+ merge) alone, local output
        per = max_over_ranks([sum(ms) / steps, sum(res["ms_kernel"]) / steps, statistics.median(ms)])
        res["per_step"], res["per_kernel"], res["median"] = per
        return res

    # ---- the headline workload ------------------------------------------------------------------------------
    shard = args.shard or ("heads" if args.workload == "c5" else "batch")
    if shard == "heads":
        if hkv % world or hq % world:
            raise SystemExit("--shard heads needs the head counts to divide by the number of GPUs")
        l_hq, l_hkv, scaling = hq // world, hkv // world, "strong"
    else:
        l_hq, l_hkv, scaling = hq, hkv, "weak"          # every rank holds a full-size shard of the global batch
    layer = Layer(torch, pa, dtype, B, L, l_hq, l_hkv, page, 1234 + rank, stream, args.contiguous_pages, args.ctas,
                  shared_source=args.workload == "c5")
    gather = Gather(torch, pa, dist, layer, shard, args.gather, world, rank) if world > 1 else None
    needs_merge = layer.params.needs_merge

    sampler = ClockSampler(local_rank) if rank == 0 else None
    m = measure(layer, gather, args.steps, args.warmup)

    # end to end through host buffers: pinned q -> device, the step, result -> pinned host
    def step_e2e():
        layer.q.copy_(layer.q_host, non_blocking=True)
        if gather is None:
            layer.decode()
            layer.out_host.copy_(layer.out, non_blocking=True)
        else:
            gather.decode(sync=True)
            if gather.mode == "peer":     # the gathered result comes back to the host once, one share per rank
                buf = gather.views[gather.gg.epoch % 4]
                gather.full_host.copy_(buf[rank * gather.share:(rank + 1) * gather.share], non_blocking=True)
            else:
                layer.out_host.copy_(gather.gathered[rank * layer.B:(rank + 1) * layer.B], non_blocking=True)

    def step_e2e_direct():
        # The same call with q and out pointing straight at the pinned host buffers: the kernel's own
        # copy engine pulls each segment's query rows over PCIe and the epilogue stores go to host
        # memory, so the transfers are inside the kernel (1 GPU only).
        layer.params.q, layer.params.out = layer.q_host.data_ptr(), layer.out_host.data_ptr()
        layer.decode()
        layer.params.q, layer.params.out = layer.q.data_ptr(), layer.out.data_ptr()

    ms_e2e = timed(step_e2e, args.steps)
    ms_direct, direct_ok = None, None
    if world == 1:
        ms_direct = timed(step_e2e_direct, args.steps)
        torch.cuda.synchronize()           # the host buffer must hold the same result as the device path
        layer.decode()
        torch.cuda.synchronize()
        direct_ok = bool(torch.equal(layer.out_host, layer.out.cpu()))
    per_e2e = max_over_ranks([sum(ms_e2e) / args.steps])[0]
    barrier()
    clocks = sampler.stop() if sampler else None
    pa.kernel_status(stream)

    # two layers back to back (no flush between them): in order = (decode + announce-and-wait) twice; overlapped =
    # decode, announce, decode, announce, then the two waits: the first layer's wait overlaps the second decode
    back_to_back = None
    if gather is not None and gather.mode == "peer":
        def two_in_order():
            gather.decode(sync=True); gather.decode(sync=True)

        def two_overlapped():
            gather.decode(); gather.decode(); gather.wait(back=1); gather.wait()
        a = max_over_ranks([sum(timed(two_in_order, args.steps)) / args.steps])[0]
        b = max_over_ranks([sum(timed(two_overlapped, args.steps)) / args.steps])[0]
        back_to_back = {"two_layers_in_order_ms": a, "two_layers_overlapped_ms": b,
                        "note": "events around two consecutive layers; overlapped launches the second decode before waiting for the first layer's rows"}

    gather_check = gather.check() if gather is not None else None
    launch = layer.launch()
    per_step, per_kernel = m["per_step"], m["per_kernel"]
    local_bytes = layer.bytes
    job_bytes = local_bytes * world
    value = job_bytes / (per_step * 1e-3) / 1e9
    e2e_value = job_bytes / (per_e2e * 1e-3) / 1e9
    peak, peak_src = measured_peak()
    merged_in_kernel = launch["merge"] != "merge kernel" and not launch["merge"].startswith("per row")
    achieved = local_bytes / (per_kernel * 1e-3) / 1e9
    one_row_check = None
    if world == 1:
        layer.decode()
        torch.cuda.synchronize()
        want = layer.oracle_rows((0, B - 1))
        one_row_check = max(float(np.abs(layer.out[r].float().cpu().numpy() - w).max()) for r, w in want.items())

    # ---- the reference's own GPU kernel on the same cache bytes (1 GPU; checker library, outside the timed region)
    reference_gpu = None
    if world == 1 and not args.no_reference_gpu:
        reference_gpu = time_reference_kernel(torch, layer, flush, args.steps)

    # ---- the 70B-shaped layer with its kv heads sharded over the same ranks (strong scaling) ----------------------
    c5 = None
    if args.workload != "c5" and not args.no_c5 and 8 % world == 0:
        if gather is not None:
            gather.close()
            gather = None
        layer.close()
        c5 = c5_heads(torch, pa, dist, world, rank, stream, measure, max_over_ranks, args)

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_leg(dtype, L, hq, hkv, page, B)
        gather_mode = gather_mode_of(world, args, launch, gather_check)
        line = {
            "metric": "paged_decode_achieved_hbm_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": m["untimed"], "warmup_requested": args.warmup, "ms_per_step": per_step,
            "ms_per_step_median": m["median"],
            "us_per_layer": per_step * 1e3, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": DTYPE_NAMES[dtype],
            "data": "synthetic",
            "config": {"workload": desc, "name": args.workload, "arithmetic": ARITHMETIC[dtype],
                       "batch_per_gpu": B, "seq_len": L, "q_heads_per_gpu": l_hq,
                       "kv_heads_per_gpu": l_hkv, "page_size": page, "sharding": "none" if world == 1 else shard,
                       "gather": gather_mode,
                       "pages": "contiguous" if args.contiguous_pages else "scattered (shuffle seed 42)",
                       "plan_of_the_caller": {"ctas": layer.plan.num_ctas, "segments": layer.plan.num_segments, "tile": layer.plan.tile},
                       "launch": launch,
                       "plan": "uploaded before every untimed step, timed steps reuse the last one; adaptive cut %s"
                               % ("on" if pa.adaptive_cut() else "off"),
                       "l2": "KV per step (%.0f MB) exceeds L2 and a read-only flush of 512 MB runs before every step, outside the events"
                             % (local_bytes / 1e6),
                       "timing": "CUDA events around decode+merge%s per step, summed over steps (mean; median beside it), max over ranks"
                                 % (" + output gather (the step ends when all ranks' rows are in this rank's buffer); ranks "
                                    "rendezvous (1-element all-reduce) after the flush, before the start event" if world > 1 else "")},
            "algorithmic_bytes_per_step": job_bytes,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src, "kernel": "paged_decode_kernel",
                         "kernel_ms": per_kernel,
                         "kernel_ms_source": ("the decode launch timed alone with local output (split rows merged inside it)"
                                              if merged_in_kernel else "decode + merge kernel timed alone with local output"),
                         "frac_of_8TBps_nominal": achieved / 8000.0},
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": per_e2e,
                    "h2d_bytes_per_step": layer.q_host.numel() * 2,
                    "d2h_bytes_per_step": layer.out_host.numel() * 2,
                    "note": "pinned q -> device, decode+merge%s, result -> pinned host, per step; the KV cache is resident state"
                            % (" + gather + wait, one 1/N share of the gathered result" if world > 1 else "")},
            "e2e_host_pointers": None if ms_direct is None else {
                "value": job_bytes / (sum(ms_direct) / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                "ms_per_step": sum(ms_direct) / args.steps, "matches_device_path": direct_ok,
                "note": "same C-ABI call with q/out = pinned host pointers: query rows and outputs cross PCIe inside the kernel, no separate copies"},
            "gpu_launches": args.steps * launches_per_step(world, args, launch),
            "gpu_launches_note": "per step: paged_decode_kernel%s%s + stream_read_kernel (L2 flush)"
                                 % ("" if merged_in_kernel else " + merge_segments_kernel",
                                    " + gather_signal_kernel" if world > 1 and args.gather == "peer" else ""),
            "clocks": clocks, "wall_s_timed_region": m["wall"],
        }
        if world > 1:
            line["gather_check"] = gather_check
            line["back_to_back"] = back_to_back
        if one_row_check is not None:
            line["oracle_check"] = {"max_abs_rows_0_and_last": one_row_check, "tolerance": 2e-3, "ok": one_row_check <= 2e-3}
        if reference_gpu:
            line["reference_gpu"] = reference_gpu
        if c5:
            line["c5_heads"] = c5
        if cpu:
            line["cpu_baseline"] = cpu
        traffic_path = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(traffic_path):
            with open(traffic_path) as f:
                t = json.load(f).get(args.workload)
            if t:
                line["roofline"]["traffic"] = t["dram_bytes_per_launch"]
                line["roofline"]["traffic_source"] = t["source"]
        print(json.dumps(line))
    if gather is not None:
        gather.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if gather_check is not None and not gather_check["ok"]:
        raise SystemExit("bench.py: the gathered output differs (gather_check)")


def gather_mode_of(world, args, launch, gather_check):
    if world == 1:
        return "single GPU"
    if args.gather == "peer":
        return "decode kernel stores into every peer's buffer (16-byte NVLink peer stores) + one dependent kernel that raises this rank's flag on the peers and waits for theirs"
    return "ncclAllGather after the decode"


def launches_per_step(world, args, launch):
    n = 2                                         # decode + L2 flush
    if launch["merge"] == "merge kernel" or launch["merge"].startswith("per row"):
        n += 1
    if world > 1 and args.gather == "peer":
        n += 1
    return n


def time_reference_kernel(torch, layer, flush, steps):
    """The reference's paged_decode_kernel (mma.sync + cp.async), compiled for sm_100a from its own sources into
    oracle/_ref, on the engine's cache bytes and block table: same flush + event protocol, outside the
    headline's timed region (bench/bench_decode.cu:121-139,198-209 of the reference)."""
    ol = checker()
    R = ol.ref()
    if R is None:
        return {"unavailable": "oracle/_ref/libpd_ref.so is not built"}
    p = layer.params
    dec = R.ref_decoder_create()
    lens = np.ascontiguousarray(layer.lens, np.int32)
    ref_out = torch.zeros_like(layer.q)
    if R.ref_decoder_plan(dec, layer.dtype, lens.ctypes.data_as(C.POINTER(C.c_int)), layer.B, layer.hq, layer.hkv, 128, 0) != 0:
        return {"unavailable": R.ref_last_error().decode()}
    pages = (layer.L + layer.page - 1) // layer.page

    def run():
        rc = R.ref_decoder_run(dec, layer.dtype, layer.q.data_ptr(), ref_out.data_ptr(), p.k_cache, p.v_cache, p.block_table,
                               pages, p.seq_lens, layer.B, layer.hq, layer.hkv, 128, layer.page, layer.scale, layer.scale, None)
        if rc != 0:
            raise SystemExit("reference kernel: " + R.ref_last_error().decode())
    for _ in range(5):
        flush()
        run()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in ev:
        flush()
        s.record()
        run()
        e.record()
    torch.cuda.synchronize()
    ms = [s.elapsed_time(e) for s, e in ev]
    layer.decode()
    torch.cuda.synchronize()
    ctas, segs = C.c_int(), C.c_int()
    R.ref_decoder_info(dec, C.byref(ctas), C.byref(segs))
    R.ref_decoder_destroy(dec)
    mean = sum(ms) / len(ms)
    return {"kernel": "the reference's paged_decode_kernel + merge_segments_kernel (mma.sync m16n8k16 + cp.async), its own sources "
                      "compiled for sm_100a into oracle/_ref, on the engine's cache bytes and block table",
            "us_per_layer": mean * 1e3, "us_per_layer_median": statistics.median(ms) * 1e3,
            "value": layer.bytes / (mean * 1e-3) / 1e9, "unit": "GB/s", "ctas": ctas.value, "segments": segs.value,
            "max_abs_diff_vs_engine": float((ref_out.float() - layer.out.float()).abs().max().item())}


def c5_heads(torch, pa, dist, world, rank, stream, measure, max_over_ranks, args):
    """BASELINE config 5: Hq 64 / Hkv 8, batch 256 x 16384, e4m3, 16-token pages, kv heads sharded over the ranks
    (one fixed problem: strong scaling), outputs gathered by the decode kernel's peer stores."""
    dtype, B, L, hq, hkv, page, desc = WORKLOADS["c5"]
    if args.c5_batch:
        B = args.c5_batch
    l_hq, l_hkv = hq // world, hkv // world
    layer = Layer(torch, pa, dtype, B, L, l_hq, l_hkv, page, 4321 + rank, stream, shared_source=True)
    gather = Gather(torch, pa, dist, layer, "heads", args.gather, world, rank) if world > 1 else None
    m = measure(layer, gather, args.steps, args.warmup)
    check = gather.check() if gather is not None else None
    launch = layer.launch()
    full_bytes = algorithmic_bytes(dtype, [L] * B, hq, hkv, page)
    local_bytes = layer.bytes
    if gather is not None:
        gather.close()
    layer.close()
    del layer
    torch.cuda.empty_cache()
    single = None
    if world > 1:
        # the unsharded layer on one GPU (rank 0), for the strong-scaling ratio; the others wait
        if rank == 0:
            full = Layer(torch, pa, dtype, B, L, hq, hkv, page, 4321, stream, shared_source=True)
            single = measure_single(torch, pa, full, stream, args)
            full.close()
        dist.barrier()
    else:
        single = m["per_step"]
    out = {"workload": desc if not args.c5_batch else desc + " [batch reduced to %d]" % B, "n_gpus": world,
           "us_per_layer": m["per_step"] * 1e3,
           "us_decode_kernel_alone": m["per_kernel"] * 1e3,
           "value": full_bytes / (m["per_step"] * 1e-3) / 1e9, "unit": "GB/s (whole layer, all GPUs)",
           "per_gpu_gbs": local_bytes / (m["per_step"] * 1e-3) / 1e9, "scaling": "strong",
           "kv_heads_per_gpu": l_hkv, "q_heads_per_gpu": l_hq, "launch": launch, "gather_check": check}
    if rank == 0 and single is not None:
        out["us_per_layer_one_gpu"] = single * 1e3
        out["speedup_vs_one_gpu"] = single / m["per_step"]
        out["strong_scaling_efficiency"] = single / m["per_step"] / world
    return out


def measure_single(torch, pa, layer, stream, args):
    """Rank 0 alone: the same protocol without the rendezvous (no collective may be called by one rank)."""
    flush_buf = torch.zeros(512 << 20, dtype=torch.uint8, device="cuda")
    untimed = max(max(args.warmup, 3), 24 if pa.adaptive_cut() else 0)
    for _ in range(untimed):
        layer.replan()
        pa.stream_read(flush_buf, flush_buf.numel(), 148 * 8, stream)
        layer.decode()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for s, e in ev:
        pa.stream_read(flush_buf, flush_buf.numel(), 148 * 8, stream)
        s.record()
        layer.decode()
        e.record()
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in ev) / len(ev)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--replan-every-step", action="store_true",
                    help="upload the plan again before every timed step too (outside the events), not only during warm-up")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--shard", default=None, choices=["batch", "heads"])
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--contiguous-pages", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true")
    ap.add_argument("--adaptive-cut", default="on", choices=["on", "off"],
                    help="off: equal shares as in the reference (and no settling steps); profiling runs use it to keep the launch count small")
    ap.add_argument("--no-c5", action="store_true", help="skip the kv-head-sharded 70B-shaped layer after the headline")
    ap.add_argument("--c5-batch", type=int, default=0, help="batch of that layer (default: the workload's 256)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        reference_arm(args, wl)
    else:
        our_arm(args, wl)


if __name__ == "__main__":
    main()
