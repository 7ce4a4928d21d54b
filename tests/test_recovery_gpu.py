"""Recovery after a bounded wait has expired (no counterpart in the reference, whose kernels wait forever).

A CTA that gives up on a wait skips its arrivals: the arrival counters of the in-kernel merge are then left
with partial counts, and a later launch of the same plan would merge rows early or never.  No wait is made to expire here and nothing faults: the state such a
launch leaves is written from the host with plain memsets, then pd_device_plan_reset is called and the next
decode is compared with the oracle.  (The gathered-output path keeps no such state: its flags carry step
numbers and the decode kernel counts nothing.)
"""
import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, block_table_matrix, build_cache, device_view, oracle_cache, seeded_kv

pytestmark = pytest.mark.gpu


def _problem(torch, pa, dtype, lens, num_ctas, seed):
    case = Case(dtype, 32, 8, 16, lens, shuffle=seed, seed=seed)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    B = len(lens)
    q = torch.randn(B, 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(seed)).cuda()
    kc, vc = oracle_cache(case, cfg, K, V, model)
    bt = block_table_matrix(model, B, cfg.max_pages_per_slot)
    want = ol.paged_decode(1, dtype, q.cpu().numpy().view(np.uint16), kc, vc, bt, lens, 32, 8, 128, 16,
                           k_scale=case.scale, v_scale=case.scale, threads=0)
    return cache, cfg, q, want


@pytest.mark.parametrize("dtype", [0, 1])
def test_plan_reset_clears_poisoned_arrival_counters(dtype, torch_cuda, pa):
    torch = torch_cuda
    fused_before = pa.head_fused()
    pa.set_head_fused(0)            # one schedule region: the caller's plan, whose workspace pd_params shows
    try:
        lens = [3000, 700, 4099, 90]
        cache, cfg, q, want = _problem(torch, pa, dtype, lens, 24, 31)
        plan = pa.make_plan(pa.KVDtype(dtype), lens, 32, 8, 128, 24)
        assert plan.num_segments > len(lens) * 8
        dplan = pa.DevicePlan()
        dplan.upload(plan, 4, 128)
        p = cache.params()
        out = torch.zeros_like(q)
        p.q, p.out, p.batch, p.num_q_heads = q.data_ptr(), out.data_ptr(), len(lens), 32
        dplan.bind(p)
        assert p.needs_merge == 2, "rows cut in few pieces: merged inside the decode kernel"
        pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)
        torch.cuda.synchronize()
        assert float(np.abs(out.float().cpu().numpy() - want).max()) <= TOL

        # what a CTA that bailed out leaves behind: counters that no longer start at zero
        items = len(lens) * 8
        counters = device_view(p.partial_lse + 4 * plan.num_segments * 4, 4 * items, torch).view(torch.int32)
        counters.fill_(1)
        out.zero_()
        pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)     # merges fire early or not at all
        torch.cuda.synchronize()
        assert pa.kernel_status() == 0                              # and nothing reports it: hence the reset
        dplan.reset()
        out.zero_()
        pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)
        torch.cuda.synchronize()
        assert int(counters.abs().sum().item()) == 0, "merging warps re-arm their counters"
        assert float(np.abs(out.float().cpu().numpy() - want).max()) <= TOL
        cache.close()
    finally:
        pa.set_head_fused(fused_before)
