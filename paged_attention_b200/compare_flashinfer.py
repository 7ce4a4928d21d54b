"""Optional comparison with FlashInfer's paged decode on the same tensors (the reference's published claim
is "within a few percent of FlashInfer").  To be comparable with the reference's own harness the inputs
and the fp32 check restate scripts/compare_flashinfer.py:80-126 of the reference: `make_inputs` builds the
same HND pools, per-tensor scales amax/448 and permuted page table (:80-97), `fp32_reference` is the same
per-row einsum softmax (:113-126), and FlashInfer is driven through the same wrapper call.  The timing loop,
the CSV and the command line are this package's.  FlashInfer is never a dependency of the engine: if it is
not importable (or cannot build its kernels here) the script says so and exits 0.

    python -m paged_attention_b200.compare_flashinfer [--iters 30] [--shapes 32x8192,64x8192,128x4096]

Prints CSV: dtype,batch,seq_len,ours_us,flashinfer_us,flashinfer_tc_us,ratio_fi_over_ours,max_abs_vs_fi,max_abs_vs_fp32
Timing: cold L2 (read-only flush before each run), CUDA events, median.
"""
import argparse
import math
import statistics
import sys

HQ, HKV, DIM, PAGE = 32, 8, 128, 16


def make_inputs(torch, batch, seq_len, fp8, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages_per_seq = math.ceil(seq_len / PAGE)
    num_pages = batch * pages_per_seq
    k = torch.randn(num_pages, HKV, PAGE, DIM, device="cuda", dtype=torch.float16, generator=g)
    v = torch.randn(num_pages, HKV, PAGE, DIM, device="cuda", dtype=torch.float16, generator=g)
    k_scale = v_scale = 1.0
    if fp8:
        k_scale, v_scale = k.abs().max().item() / 448.0, v.abs().max().item() / 448.0
        k, v = (k / k_scale).to(torch.float8_e4m3fn), (v / v_scale).to(torch.float8_e4m3fn)
    table = torch.randperm(num_pages, device="cuda", generator=g).to(torch.int32).view(batch, pages_per_seq).contiguous()
    q = torch.randn(batch, HQ, DIM, device="cuda", dtype=torch.float16, generator=g)
    return q, k, v, k_scale, v_scale, table


def fp32_reference(torch, q, k, v, k_scale, v_scale, table, seq_len):
    outs = []
    group = HQ // HKV
    for b in range(table.shape[0]):
        pages = table[b].long()
        kb = (k[pages].float() * k_scale).permute(1, 0, 2, 3).reshape(HKV, -1, DIM)[:, :seq_len]
        vb = (v[pages].float() * v_scale).permute(1, 0, 2, 3).reshape(HKV, -1, DIM)[:, :seq_len]
        s = torch.einsum("hgd,htd->hgt", q[b].float().view(HKV, group, DIM), kb) / math.sqrt(DIM)
        outs.append(torch.einsum("hgt,htd->hgd", s.softmax(-1), vb).reshape(HQ, DIM))
    return torch.stack(outs)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--shapes", default="32x8192,64x8192,128x4096,8x32768")
    a = ap.parse_args(argv)
    import torch
    import paged_attention_b200 as pa
    from paged_attention_b200.torch_decode import Decoder
    try:
        import flashinfer
    except Exception as e:   # not installed: nothing to compare with
        print(f"# flashinfer unavailable: {e}")
        return 0
    flush_buf = torch.zeros(512 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def time_cold(fn, before=None):
        for _ in range(24):          # the same warm-up for both sides (the engine's adaptive cut settles within it)
            if before:
                before()
            pa.stream_read(flush_buf, flush_buf.numel(), 148 * 8, stream)
            fn()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.iters)]
        for s, e in ev:
            pa.stream_read(flush_buf, flush_buf.numel(), 148 * 8, stream)
            s.record()
            fn()
            e.record()
        torch.cuda.synchronize()
        return statistics.median(s.elapsed_time(e) for s, e in ev) * 1e3

    print("dtype,batch,seq_len,ours_us,flashinfer_us,flashinfer_tc_us,ratio_fi_over_ours,max_abs_vs_fi,max_abs_vs_fp32")
    for shape in a.shapes.split(","):
        batch, seq_len = (int(x) for x in shape.split("x"))
        for fp8 in (False, True):
            q, k, v, ks, vs, table = make_inputs(torch, batch, seq_len, fp8)
            lens = torch.full((batch,), seq_len, dtype=torch.int32)
            dec = Decoder(HQ, HKV, DIM, PAGE, fp8)
            dec.plan(lens)
            lens_dev = lens.cuda()
            ours = lambda: dec.run(q, k, v, table, lens_dev, ks, vs)
            t_ours = time_cold(ours, lambda: dec.plan(lens))
            out = ours()
            fi_times, fi_out = [], None
            for use_tc in (False, True):
                try:
                    ws = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
                    w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "HND", use_tensor_cores=use_tc)
                    pages_per_seq = table.shape[1]
                    indptr = torch.arange(0, batch + 1, dtype=torch.int32, device="cuda") * pages_per_seq
                    last = torch.full((batch,), seq_len - (pages_per_seq - 1) * PAGE, dtype=torch.int32, device="cuda")
                    w.plan(indptr, table.reshape(-1).contiguous(), last, HQ, HKV, DIM, PAGE, pos_encoding_mode="NONE",
                           q_data_type=torch.float16, kv_data_type=k.dtype)
                    run = lambda: w.run(q, (k, v), k_scale=ks, v_scale=vs)
                    fi_times.append(time_cold(run))
                    fi_out = run()
                except Exception as e:
                    print(f"# flashinfer (tensor cores {use_tc}) failed for {shape} fp8={fp8}: {str(e)[:200]}", file=sys.stderr)
                    fi_times.append(float("nan"))
            ref = fp32_reference(torch, q, k, v, ks, vs, table, seq_len)
            d_fi = (out.float() - fi_out.float()).abs().max().item() if fi_out is not None else float("nan")
            d_ref = (out.float() - ref).abs().max().item()
            best_fi = min((t for t in fi_times if t == t), default=float("nan"))
            print(f"{'fp8_e4m3' if fp8 else 'fp16'},{batch},{seq_len},{t_ours:.1f},{fi_times[0]:.1f},{fi_times[1]:.1f},"
                  f"{best_fi / t_ours:.3f},{d_fi:.2e},{d_ref:.2e}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
