"""pd_paged_decode_static: decode + merge that allocates nothing.

Who needs it: a serving process that has handed all free HBM to its KV pool (a workspace
cudaMalloc during a step would fail), or a step loop that bans cudaMalloc/cudaFree because they
stall the device.  The entry point swaps the allocated split-row workspace for an 8 MiB array
built into the library; everything else is the same launch.

Checked here, through the C ABI: its output equals the ordinary entry point's on the same plan,
on two calls in a row (the shared workspace still holds the first call's partials during the
second), then on a different problem (stale contents of the workspace do not leak in), and a
plan that needs more than the built-in workspace is refused before anything is launched.

Collected last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest

from common import TOL, Case, build_cache, seeded_kv

pytestmark = pytest.mark.gpu


def _problem(torch, pa, dtype, lens, num_ctas, seed):
    case = Case(dtype, 32, 8, 16, lens, shuffle=seed, seed=seed)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, _, cfg = build_cache(case, K, V, torch, pa)
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
    return cache, cfg, dplan, plan, p, q


@pytest.mark.parametrize("dtype", [0, 1])
def test_static_workspace_decode_matches_allocating_decode(dtype, torch_cuda, pa):
    torch = torch_cuda
    # The new entry point always runs the (row, kv head) schedule, so compare it with the existing entry
    # point on that same schedule (bit for bit), and with the default head-fused schedule within TOL.
    fused_before = pa.head_fused()
    cache, cfg, dplan, plan, p, q = _problem(torch, pa, dtype, [3000, 700, 4099, 90], 200, 21)
    default_out = torch.zeros_like(q)
    p.out = default_out.data_ptr()
    pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)
    torch.cuda.synchronize()
    pa.set_head_fused(False)
    try:
        _check_static_against_existing(torch, pa, dtype, cache, cfg, dplan, plan, p, q, default_out)
    finally:
        pa.set_head_fused(fused_before)
    cache.close()


def _check_static_against_existing(torch, pa, dtype, cache, cfg, dplan, plan, p, q, default_out):
    want = torch.zeros_like(q)
    p.out = want.data_ptr()
    pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)          # the existing entry point
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in range(2):                                             # two calls in a row
        got = torch.full_like(q, float("nan"))
        p.out = got.data_ptr()
        pa.paged_decode_static(pa.KVDtype(dtype), p, plan.num_segments, 0, cfg.num_pages, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.isfinite(got).all()
        assert (got.float() - want.float()).abs().max().item() <= TOL, f"call {call}"
        assert torch.equal(got, want), f"call {call}: same kernels, same plan, so the same bits"
        assert (got.float() - default_out.float()).abs().max().item() <= TOL

    # a different, smaller problem right after: whatever the workspace still holds must not matter
    cache2, cfg2, dplan2, plan2, p2, q2 = _problem(torch, pa, dtype, [513, 64, 2000], 77, 5)
    want2, got2 = torch.zeros_like(q2), torch.zeros_like(q2)
    p2.out = want2.data_ptr()
    pa.paged_decode(pa.KVDtype(dtype), p2, 0, cfg2.num_pages)
    p2.out = got2.data_ptr()
    pa.paged_decode_static(pa.KVDtype(dtype), p2, plan2.num_segments, 0, cfg2.num_pages, None)
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    cache2.close()


def test_static_workspace_refuses_oversized_plans(torch_cuda, pa):
    torch = torch_cuda
    cache, cfg, dplan, plan, p, q = _problem(torch, pa, 0, [3000, 700], 64, 3)
    out = torch.zeros_like(q)
    p.out = out.data_ptr()
    limit = (8 << 20) // (4 * 4 * 129)            # segments that fit 8 MiB at group 4, head_dim 128
    pa.paged_decode_static(pa.KVDtype.FP16, p, plan.num_segments, 0, cfg.num_pages)   # fits
    with pytest.raises(pa.InvalidArgument, match="built-in workspace"):
        pa.paged_decode_static(pa.KVDtype.FP16, p, limit + 1, 0, cfg.num_pages)
    with pytest.raises(pa.InvalidArgument):
        pa.paged_decode_static(pa.KVDtype.FP16, p, -1, 0, cfg.num_pages)
    torch.cuda.synchronize()
    cache.close()
