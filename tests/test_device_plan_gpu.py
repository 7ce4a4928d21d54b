"""The device-side planner (pd_device_plan_build): the plan of decode::make_plan
(src/decode/decode.cu:65-108 of the reference) cut by a kernel from lengths that live on the GPU.

Checked here: its arrays equal the host planner's bit for bit over random batches, grids and kv-head
counts (also through slot ids and for batches wider than the planner's thread block); decoding with it
gives the same bits as decoding with the uploaded host plan; rows with a bad length get no work and are
reported; the cache's plan_device; and a CUDA graph of plan + decode replayed while the lengths grow.
"""
import numpy as np
import pytest

from common import TOL, Case, build_cache, seeded_kv

pytestmark = pytest.mark.gpu

FP16, FP8 = 0, 1


def _same_plan(dev, host):
    assert dev.num_ctas == host.num_ctas
    assert dev.tile == host.tile
    assert dev.num_segments == host.num_segments
    assert (dev.segments == host.segments).all()
    assert (dev.cta_seg_begin == host.cta_seg_begin).all()
    assert (dev.item_seg_begin == host.item_seg_begin).all()


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_device_plan_equals_host_plan(dtype, torch_cuda, pa):
    torch = torch_cuda
    rng = np.random.default_rng(123 + dtype)
    dp = pa.DevicePlan()
    cases = [([1], 8, 0), ([64], 8, 5), ([65], 1, 3), ([100000], 8, 0), ([8192] * 64, 8, 0), ([1] * 300, 4, 0),
             ([4096] * 128, 8, 296), ([17, 16, 15, 1, 4100], 8, 7), ([5000, 100], 8, 1000), ([512] * 37, 2, 1)]
    for _ in range(25):
        batch = int(rng.integers(1, 200))
        lens = np.round(np.exp(rng.uniform(0, np.log(40000), batch))).astype(int).tolist()
        cases.append((lens, int(rng.choice([1, 2, 4, 8])), int(rng.choice([0, 1, 13, 148, 296, 443, 2000]))))
    cases.append((rng.integers(1, 3000, 2500).tolist(), 8, 0))      # more rows than the planner has threads
    cases.append((rng.integers(1, 300, 5000).tolist(), 4, 64))
    for lens, hkv, ctas in cases:
        hq = hkv * 4
        d_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
        dp.build(dtype, d_lens, len(lens), hq, hkv, 128, ctas)
        host = pa.make_plan(pa.KVDtype(dtype), lens, hq, hkv, 128, ctas)
        _same_plan(dp.fetch(), host)
        used, nseg, widest, bad = dp.info()
        assert (used, nseg, bad) == (host.num_ctas, host.num_segments, 0)
        assert widest == int(np.diff(host.item_seg_begin).max())


def test_device_plan_follows_slot_ids(torch_cuda, pa):
    torch = torch_cuda
    lens = [900, 40, 2500, 333, 1, 7000]
    slots = [5, 2, 0, 3]
    dp = pa.DevicePlan()
    dp.build(FP16, torch.tensor(lens, dtype=torch.int32, device="cuda"), len(slots), 32, 8, 128, 0,
             d_slot_ids=torch.tensor(slots, dtype=torch.int32, device="cuda"))
    _same_plan(dp.fetch(), pa.make_plan(pa.KVDtype.FP16, [lens[s] for s in slots], 32, 8, 128, 0))


def _decode_with(torch, pa, dtype, cache, cfg, q, lens, dplan):
    p = cache.params()
    out = torch.full_like(q, float("nan"))
    p.q, p.out = q.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads = len(lens), q.shape[1]
    dplan.bind(p)
    pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    return out


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("lens,ctas", [([3000, 700, 4099, 90], 0), ([20000], 0), ([20000, 100, 64], 300),
                                       ([1, 2, 3], 0), ([513] * 9, 5)])
def test_decode_with_device_plan_gives_the_host_plan_bits(dtype, lens, ctas, torch_cuda, pa):
    torch = torch_cuda
    case = Case(dtype, 32, 8, 16, lens, shuffle=5, seed=31)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    q = torch.randn(len(lens), 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(2)).cuda()
    before = pa.head_fused()
    pa.set_head_fused(0)          # the (row, kv head) schedule on both sides; the head-fused one has its own test
    try:
        host_plan = pa.make_plan(pa.KVDtype(dtype), lens, 32, 8, 128, ctas)
        hp = pa.DevicePlan()
        hp.upload(host_plan, 4, 128)
        want = _decode_with(torch, pa, dtype, cache, cfg, q, lens, hp)
        dp = pa.DevicePlan()
        dp.build(dtype, torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), 32, 8, 128, ctas)
        got = _decode_with(torch, pa, dtype, cache, cfg, q, lens, dp)
        assert torch.isfinite(got).all()
        assert torch.equal(got, want)
        # a second step with the same device plan object (counters re-armed, buffers reused)
        dp.build(dtype, torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), 32, 8, 128, ctas)
        assert torch.equal(_decode_with(torch, pa, dtype, cache, cfg, q, lens, dp), want)
    finally:
        pa.set_head_fused(before)
    cache.close()


def test_bad_length_is_reported_and_gets_no_work(torch_cuda, pa):
    torch = torch_cuda
    lens = [500, 0, 64, -3, 9]
    dp = pa.DevicePlan()
    dp.build(FP16, torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), 8, 8, 128, 10)
    used, nseg, widest, bad = dp.info()
    assert bad in (2, 4)             # 1 + a row whose length is not positive
    plan = dp.fetch()
    rows = set(plan.segments[:, 0].tolist())
    assert rows == {0, 2, 4}
    with pytest.raises(pa.InvalidArgument):
        pa.make_plan(pa.KVDtype.FP16, lens, 8, 8, 128, 10)   # the host planner refuses the same batch


def test_cache_plan_device_matches_cache_plan(torch_cuda, pa):
    torch = torch_cuda
    lens = [1500, 33, 4096, 700, 12]
    case = Case(FP8, 32, 8, 16, lens, shuffle=8, seed=3)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    q = torch.randn(len(lens), 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(4)).cuda()
    want, got, got_sub = torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(q)
    cache.plan(list(range(len(lens))), 32)
    cache.run(q, want)
    cache.plan_device(len(lens), 32)
    assert cache.last_plan() is None
    cache.run(q, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # a subset of the slots, through a device array of slot ids
    slots = [3, 0, 2]
    d_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    cache.plan_device(len(slots), 32, d_slot_ids=d_slots)
    cache.run(q[:3].contiguous(), got_sub[:3])
    cache.plan(slots, 32)
    sub_want = torch.zeros_like(q[:3])
    cache.run(q[:3].contiguous(), sub_want)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    assert torch.equal(got_sub[:3], sub_want)
    cache.close()


def test_plan_and_decode_replay_in_a_cuda_graph(torch_cuda, pa):
    """Capture {device plan, decode} once; replay it while the sequences grow.  The captured calls make
    no allocation, no host copy and no wait, or the capture itself would fail."""
    torch = torch_cuda
    lens0 = [700, 31, 2048, 15]
    steps = 5
    final = [n + steps for n in lens0]
    case = Case(FP16, 32, 8, 16, final, shuffle=6, seed=17)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)      # holds every token the steps will reveal
    q = torch.randn(len(lens0), 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(9)).cuda()
    out = torch.zeros_like(q)
    d_lens = torch.tensor(lens0, dtype=torch.int32, device="cuda")    # the lengths the graph reads
    p = cache.params()
    p.seq_lens = d_lens.data_ptr()
    p.q, p.out = q.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads = len(lens0), 32
    dp = pa.DevicePlan()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        # once outside the capture: buffers grow to their final size, kernels get configured
        dp.build(FP16, d_lens, len(lens0), 32, 8, 128, 0, stream=side.cuda_stream)
        dp.bind(p)
        pa.paged_decode(pa.KVDtype.FP16, p, side.cuda_stream, cfg.num_pages)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            s = torch.cuda.current_stream().cuda_stream
            dp.build(FP16, d_lens, len(lens0), 32, 8, 128, 0, stream=s)
            dp.bind(p)
            pa.paged_decode(pa.KVDtype.FP16, p, s, cfg.num_pages)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    before = pa.head_fused()
    pa.set_head_fused(0)
    try:
        for step in range(steps + 1):
            cur = [n + step for n in lens0]
            d_lens.copy_(torch.tensor(cur, dtype=torch.int32))
            out.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert pa.kernel_status() == 0
            hp = pa.DevicePlan()
            hp.upload(pa.make_plan(pa.KVDtype.FP16, cur, 32, 8, 128, 0), 4, 128)
            want = torch.zeros_like(q)
            p2 = cache.params()
            p2.seq_lens = d_lens.data_ptr()
            p2.q, p2.out = q.data_ptr(), want.data_ptr()
            p2.batch, p2.num_q_heads = len(lens0), 32
            hp.bind(p2)
            pa.paged_decode(pa.KVDtype.FP16, p2, 0, cfg.num_pages)
            torch.cuda.synchronize()
            assert torch.equal(out, want), f"step {step}"
    finally:
        pa.set_head_fused(before)
    cache.close()


@pytest.mark.parametrize("lens,ctas", [([700] * 60 + [3000, 64, 1], 0), ([20000, 5000] + [300] * 58, 0), ([513] * 9, 5)])
def test_device_plan_runs_the_head_fused_schedule_too(lens, ctas, torch_cuda, pa):
    """fp16, 8 kv heads, a wide batch: the device planner also cuts the step by rows for the head-fused
    kernel.  Its result has the bits of the host-planned head-fused step: same cut, and rows cut in more
    than 4 pieces are merged by the same separate kernel in both."""
    torch = torch_cuda
    case = Case(FP16, 32, 8, 16, lens, shuffle=2, seed=41)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    q = torch.randn(len(lens), 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(6)).cuda()
    before = pa.head_fused()
    pa.set_head_fused(2)
    try:
        hp = pa.DevicePlan()
        hp.upload(pa.make_plan(pa.KVDtype.FP16, lens, 32, 8, 128, ctas), 4, 128)
        want = _decode_with(torch, pa, FP16, cache, cfg, q, lens, hp)
        dp = pa.DevicePlan()
        dp.build(FP16, torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), 32, 8, 128, ctas)
        got = _decode_with(torch, pa, FP16, cache, cfg, q, lens, dp)
        pa.set_head_fused(0)
        plain = _decode_with(torch, pa, FP16, cache, cfg, q, lens, dp)
    finally:
        pa.set_head_fused(before)
    assert torch.equal(got, want)
    assert not torch.equal(got, plain), "mode 0 runs the (row, kv head) schedule of the same device plan"
    assert (got.float() - plain.float()).abs().max().item() <= TOL
    cache.close()
