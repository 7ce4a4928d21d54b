"""pd_paged_decode_static: decode + merge that allocates nothing.

Who needs it: a serving process that has handed all free HBM to its KV pool (a workspace
cudaMalloc during a step would fail), or a step loop that bans cudaMalloc/cudaFree because they
stall the device.  The entry point swaps the allocated split-row workspace for an 8 MiB array
built into the library; everything else is the same launch.

Checked here, through the C ABI: its output equals the ordinary entry point's on the same plan
(bit for bit) and the CPU oracle's (within the path's tolerance), on two calls in a row (the shared
workspace still holds the first call's partials during the second), then on a different problem
(stale contents of the workspace do not leak in); the free device memory reported by the driver is
the same before and after the calls; a plan that needs more than the built-in workspace is refused
before anything is launched, and a segment count smaller than the bound plan's is caught on the
device (status code 6) instead of letting partial rows land outside the workspace.

Collected last on purpose: a failure here cannot hide the result of any other test.
"""
import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, block_table_matrix, build_cache, oracle_cache, seeded_kv

pytestmark = pytest.mark.gpu


def _problem(torch, pa, dtype, lens, num_ctas, seed, want_oracle=False):
    case = Case(dtype, 32, 8, 16, lens, shuffle=seed, seed=seed)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    B = len(lens)
    q = torch.randn(B, 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(seed)).cuda()
    plan = pa.make_plan(pa.KVDtype(dtype), lens, 32, 8, 128, num_ctas)
    assert plan.num_segments > B * 8, "the case must split rows so that the workspace is used"
    dplan = pa.DevicePlan()
    dplan.upload(plan, 4, 128)
    p = cache.params()
    p.q = q.data_ptr()
    p.batch, p.num_q_heads = B, 32
    dplan.bind(p)
    oracle = None
    if want_oracle:
        kc, vc = oracle_cache(case, cfg, K, V, model)
        bt = block_table_matrix(model, B, cfg.max_pages_per_slot)
        oracle = ol.paged_decode(1, dtype, q.cpu().numpy().view(np.uint16), kc, vc, bt, lens, 32, 8, 128, 16,
                                 k_scale=case.scale, v_scale=case.scale, threads=0)
    return cache, cfg, dplan, plan, p, q, oracle


@pytest.mark.parametrize("dtype", [0, 1])
def test_static_workspace_decode_matches_allocating_decode(dtype, torch_cuda, pa):
    torch = torch_cuda
    # The entry point always runs the (row, kv head) schedule, so compare it with the existing entry
    # point on that same schedule (bit for bit), and with the default head-fused schedule within TOL.
    fused_before = pa.head_fused()
    cache, cfg, dplan, plan, p, q, oracle = _problem(torch, pa, dtype, [3000, 700, 4099, 90], 200, 21, want_oracle=True)
    default_out = torch.zeros_like(q)
    p.out = default_out.data_ptr()
    pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)
    torch.cuda.synchronize()
    pa.set_head_fused(False)
    try:
        _check_static_against_existing(torch, pa, dtype, cache, cfg, dplan, plan, p, q, default_out, oracle)
    finally:
        pa.set_head_fused(fused_before)
    cache.close()


def _check_static_against_existing(torch, pa, dtype, cache, cfg, dplan, plan, p, q, default_out, oracle):
    want = torch.zeros_like(q)
    p.out = want.data_ptr()
    pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)          # the existing entry point
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    assert float(np.abs(want.float().cpu().numpy() - oracle).max()) <= TOL

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = torch.full_like(q, float("nan"))
    p.out = got.data_ptr()
    # Once before measuring: the first launch of a kernel in a process makes the driver load its code,
    # which is not an allocation of this library's but shows in the free-memory figure all the same.
    pa.paged_decode_static(pa.KVDtype(dtype), p, plan, 0, cfg.num_pages, status)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for call in range(2):                                             # two calls in a row
        got.fill_(float("nan"))
        pa.paged_decode_static(pa.KVDtype(dtype), p, plan, 0, cfg.num_pages, status)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
        assert int(status.item()) == 0
        assert torch.isfinite(got).all()
        assert float(np.abs(got.float().cpu().numpy() - oracle).max()) <= TOL, f"call {call}: differs from the oracle"
        assert torch.equal(got, want), f"call {call}: same kernels, same plan, so the same bits"
        assert (got.float() - default_out.float()).abs().max().item() <= TOL

    # a different, smaller problem right after: whatever the workspace still holds must not matter
    cache2, cfg2, dplan2, plan2, p2, q2, oracle2 = _problem(torch, pa, dtype, [513, 64, 2000], 77, 5, want_oracle=True)
    want2, got2 = torch.zeros_like(q2), torch.zeros_like(q2)
    p2.out = want2.data_ptr()
    pa.paged_decode(pa.KVDtype(dtype), p2, 0, cfg2.num_pages)
    p2.out = got2.data_ptr()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    pa.paged_decode_static(pa.KVDtype(dtype), p2, plan2, 0, cfg2.num_pages, None)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(got2, want2)
    assert float(np.abs(got2.float().cpu().numpy() - oracle2).max()) <= TOL
    cache2.close()


def test_static_workspace_refuses_oversized_plans(torch_cuda, pa):
    torch = torch_cuda
    cache, cfg, dplan, plan, p, q, _ = _problem(torch, pa, 0, [3000, 700], 64, 3)
    out = torch.zeros_like(q)
    p.out = out.data_ptr()
    limit = (8 << 20) // (4 * 4 * 129)            # segments that fit 8 MiB at group 4, head_dim 128
    pa.paged_decode_static(pa.KVDtype.FP16, p, plan, 0, cfg.num_pages)   # fits
    with pytest.raises(pa.InvalidArgument, match="built-in workspace"):
        pa.paged_decode_static(pa.KVDtype.FP16, p, limit + 1, 0, cfg.num_pages)
    with pytest.raises(pa.InvalidArgument):
        pa.paged_decode_static(pa.KVDtype.FP16, p, -1, 0, cfg.num_pages)
    torch.cuda.synchronize()
    cache.close()


def test_static_workspace_catches_a_stale_segment_count(torch_cuda, pa):
    """A count smaller than the bound plan's (left over from an earlier, smaller plan): the partial rows of
    the segments beyond it would overlap the LSE region or leave the array.  The kernels compare the count
    with the plan they walk; the CTAs concerned store nothing and the status word says why."""
    torch = torch_cuda
    fused_before = pa.head_fused()
    pa.set_head_fused(False)
    try:
        cache, cfg, dplan, plan, p, q, _ = _problem(torch, pa, 0, [3000, 700, 4099, 90], 200, 9)
        want = torch.zeros_like(q)
        p.out = want.data_ptr()
        pa.paged_decode(pa.KVDtype.FP16, p, 0, cfg.num_pages)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.zeros_like(q)
        p.out = out.data_ptr()
        pa.paged_decode_static(pa.KVDtype.FP16, p, plan.num_segments - 7, 0, cfg.num_pages, status)
        torch.cuda.synchronize()
        assert (int(status.item()) >> 24) == 6, hex(int(status.item()))
        status.zero_()
        pa.paged_decode_static(pa.KVDtype.FP16, p, plan, 0, cfg.num_pages, status)   # the right count: all is well again
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and torch.equal(out, want)
        cache.close()
    finally:
        pa.set_head_fused(fused_before)
