"""The adaptive cut: device plans whose CTA shares follow the streaming rates the CTAs showed in earlier
launches (the reference always cuts in equal shares, src/decode/decode.cu:86-100).

Checked: with the switch on, a serving-style loop (plan, then a few layers, again and again) keeps giving
outputs within the path's tolerance of the oracle and of the equal-share result while the shares move; the
caller-visible plan never changes; the learned weights stay a bounded distribution with mean 1; reset
returns to equal shares, which reproduce the bits of a run with the switch off.
"""
import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, block_table_matrix, build_cache, oracle_cache, seeded_kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,B,L", [(0, 64, 4096), (0, 24, 8192), (1, 96, 4096)])
def test_adaptive_cut_keeps_parity_while_shares_move(dtype, B, L, torch_cuda, pa):
    torch = torch_cuda
    hq, hkv = 32, 8
    case = Case(dtype, hq, hkv, 16, [L] * B, shuffle=7, seed=4)
    # one source sequence shared by all slots keeps the host work small; parity is checked on a few rows
    K, V = seeded_kv([L], hkv, 128, case.seed)
    scale = case.scale
    pages = (L + 15) // 16
    cfg = pa.PagedKVCache.Config(num_pages=B * pages, page_size=16, num_kv_heads=hkv, head_dim=128, max_slots=B,
                                 max_pages_per_slot=pages, dtype=pa.KVDtype(dtype), k_scale=scale, v_scale=scale)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(7)
    dK = torch.from_numpy(K[0].view(np.int16)).cuda().view(torch.float16)
    dV = torch.from_numpy(V[0].view(np.int16)).cuda().view(torch.float16)
    for b in range(B):
        assert cache.admit() == b and cache.append(b, dK, dV, L)
    q = torch.randn(B, hq, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(3)).cuda()

    def steps(n, layers=3):
        outs = []
        for _ in range(n):
            cache.plan(list(range(B)), hq)
            for _ in range(layers):
                out = torch.zeros_like(q)
                cache.run(q, out)
                outs.append(out)
        torch.cuda.synchronize()
        assert pa.kernel_status() == 0
        return outs

    pa.adaptive_cut_reset()
    cache.plan(list(range(B)), hq)
    seg_before = cache.last_plan().segments.copy()
    fixed = steps(1)[-1]                                   # the autouse fixture has switched the adaptive cut off
    pa.set_adaptive_cut(True)
    moving = steps(8)
    assert (cache.last_plan().segments == seg_before).all(), "the caller-visible plan keeps the reference's equal cut"
    worst = max((o.float() - fixed.float()).abs().max().item() for o in moving)
    assert worst <= 2.5e-4, worst                          # different split points: rounding only

    # the oracle on the first two rows (all rows share one source sequence, their pages differ)
    rows = 2
    np_dt = np.uint16 if dtype == 0 else np.uint8
    elems = cfg.num_pages * hkv * 16 * 128
    kc, vc = np.zeros(elems, np_dt), np.zeros(elems, np_dt)
    bt = np.zeros((rows, pages), np.int32)
    for b in range(rows):
        bt[b] = cache.block_table(b)
        ol.append(dtype, K[0].view(np.uint16), V[0].view(np.uint16), kc, vc, bt[b], 0, hkv, 128, 16, scale, scale)
    want = ol.paged_decode(1, dtype, q[:rows].cpu().numpy().view(np.uint16), kc, vc, bt, [L] * rows, hq, hkv, 128, 16,
                           k_scale=scale, v_scale=scale, threads=0)
    assert float(np.abs(moving[-1][:rows].float().cpu().numpy() - want).max()) <= TOL

    tables = [t for t in pa.adaptive_cut_tables() if t[1] > 0]
    assert tables, "launches were recorded"
    for weights, launches in tables:
        assert abs(float(weights.mean()) - 1.0) < 1e-3
        assert 0.69 <= float(weights.min()) and float(weights.max()) <= 1.31

    # forgetting the rates brings back equal shares and with them the bits of the fixed cut
    pa.adaptive_cut_reset()
    again = steps(1, layers=1)[-1]
    assert torch.equal(again, fixed)
    cache.close()


@pytest.mark.parametrize("dtype,B,L,hq", [(1, 96, 4096, 32), (0, 64, 4096, 32)])
def test_device_planner_follows_the_adaptive_shares(dtype, B, L, hq, torch_cuda, pa):
    """Plans cut on the device read the same weights: once the host has seen usable rates, the fetched
    device plan is the cut of make_plan_weighted for those weights, bit for bit, and outputs stay within
    rounding distance of the equal-share result."""
    torch = torch_cuda
    hkv = 8
    pages = (L + 15) // 16
    scale = 4.0 / 448.0 if dtype == 1 else 1.0
    cfg = pa.PagedKVCache.Config(num_pages=B * pages, page_size=16, num_kv_heads=hkv, head_dim=128, max_slots=B,
                                 max_pages_per_slot=pages, dtype=pa.KVDtype(dtype), k_scale=scale, v_scale=scale)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(3)
    K, V = seeded_kv([L], hkv, 128, 6)
    dK = torch.from_numpy(K[0].view(np.int16)).cuda().view(torch.float16)
    dV = torch.from_numpy(V[0].view(np.int16)).cuda().view(torch.float16)
    for b in range(B):
        assert cache.admit() == b and cache.append(b, dK, dV, L)
    q = torch.randn(B, hq, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(5)).cuda()
    before = pa.head_fused()
    pa.set_head_fused(0)                                   # one schedule, so that fetch() shows the plan that ran
    try:
        pa.adaptive_cut_reset()
        out = torch.zeros_like(q)
        cache.plan_device(B, hq)
        cache.run(q, out)
        torch.cuda.synchronize()
        fixed = out.clone()                                # adaptive cut off (fixture): equal shares
        pa.set_adaptive_cut(True)
        for _ in range(10):
            cache.plan_device(B, hq)
            for _ in range(3):
                cache.run(q, out)
        torch.cuda.synchronize()
        assert pa.kernel_status() == 0
        assert (out.float() - fixed.float()).abs().max().item() <= 2.5e-4
        # the plan of one more step against the host's weighted planner with the weights of this moment
        dp = pa.DevicePlan()
        d_lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        dp.build(dtype, d_lens, B, hq, hkv, 128, 0)
        plan = dp.fetch()
        tables = [w for w, launches in pa.adaptive_cut_tables() if launches > 0 and len(w) == plan.num_ctas]
        moved = [w for w in tables if float(np.abs(w - 1.0).max()) > 0]
        if moved:                                          # rates were usable (they are on any real GPU)
            # tables are kept per (kernel, grid): another kernel's table may have the same grid
            wants = [pa.make_plan_weighted(plan.tile, [L] * B, hq, hkv, w) for w in moved]
            assert any(w.num_segments == plan.num_segments and (plan.segments == w.segments).all() and
                       (plan.cta_seg_begin == w.cta_seg_begin).all() and
                       (plan.item_seg_begin == w.item_seg_begin).all() for w in wants)
        pa.adaptive_cut_reset()
        dp.build(dtype, d_lens, B, hq, hkv, 128, 0)
        equal = pa.make_plan(pa.KVDtype(dtype), [L] * B, hq, hkv, 128, 0)
        again = dp.fetch()
        assert (again.segments == equal.segments).all() and again.num_ctas == equal.num_ctas
    finally:
        pa.set_head_fused(before)
    cache.close()


def test_captured_step_follows_refreshed_shares(torch_cuda, pa):
    """{device plan, decode} captured once in a CUDA graph with the adaptive cut on; between replays the
    host folds new readings in with adaptive_cut_refresh, and the replayed plan follows them."""
    torch = torch_cuda
    B, L, hq, hkv = 64, 4096, 32, 8
    pages = (L + 15) // 16
    cfg = pa.PagedKVCache.Config(num_pages=B * pages, page_size=16, num_kv_heads=hkv, head_dim=128, max_slots=B,
                                 max_pages_per_slot=pages, dtype=pa.KVDtype.FP16)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(9)
    K, V = seeded_kv([L], hkv, 128, 12)
    dK = torch.from_numpy(K[0].view(np.int16)).cuda().view(torch.float16)
    dV = torch.from_numpy(V[0].view(np.int16)).cuda().view(torch.float16)
    for b in range(B):
        assert cache.admit() == b and cache.append(b, dK, dV, L)
    q = torch.randn(B, hq, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(8)).cuda()
    out = torch.zeros_like(q)
    d_lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
    p = cache.params()
    p.seq_lens, p.q, p.out, p.batch, p.num_q_heads = d_lens.data_ptr(), q.data_ptr(), out.data_ptr(), B, hq
    before = pa.head_fused()
    pa.set_head_fused(0)
    try:
        pa.adaptive_cut_reset()
        dp = pa.DevicePlan()
        dp.build(0, d_lens, B, hq, hkv, 128, 0)
        dp.bind(p)
        pa.paged_decode(pa.KVDtype.FP16, p, 0, cfg.num_pages)       # equal shares (fixture: adaptive cut off)
        torch.cuda.synchronize()
        fixed = out.clone()
        pa.set_adaptive_cut(True)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            dp.build(0, d_lens, B, hq, hkv, 128, 0, stream=side.cuda_stream)   # tables and buffers exist before the capture
            dp.bind(p)
            pa.paged_decode(pa.KVDtype.FP16, p, side.cuda_stream, cfg.num_pages)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                s = torch.cuda.current_stream().cuda_stream
                dp.build(0, d_lens, B, hq, hkv, 128, 0, stream=s)
                dp.bind(p)
                pa.paged_decode(pa.KVDtype.FP16, p, s, cfg.num_pages)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(12):
            pa.adaptive_cut_refresh()
            graph.replay()
        torch.cuda.synchronize()
        assert pa.kernel_status() == 0
        assert (out.float() - fixed.float()).abs().max().item() <= 2.5e-4
        plan = dp.fetch()
        moved = [w for w, n in pa.adaptive_cut_tables() if n > 0 and len(w) == plan.num_ctas and float(np.abs(w - 1).max()) > 0]
        if moved:
            # tables are kept per (kernel, grid): another kernel's table may have the same grid
            wants = [pa.make_plan_weighted(plan.tile, [L] * B, hq, hkv, w) for w in moved]
            assert any(w.num_segments == plan.num_segments and (plan.segments == w.segments).all() and
                       (plan.cta_seg_begin == w.cta_seg_begin).all() for w in wants)
    finally:
        pa.set_head_fused(before)
    cache.close()
