"""Work moving between the CTAs of a head-fused launch while it runs (pd_set_tail_steal).

Which pieces move depends on how fast each SM happens to stream, so the tests use mode 2, in which the row cut
is skewed on purpose (shares alternate 0.6 / 1.4): the CTAs with small shares run out early and take work from
their neighbours in every launch.  Outputs are compared with the oracle (tolerance of the path), the count of
moved pieces must grow, and repeated launches of one plan must keep agreeing (the words, counters and slots
the kernel leaves behind are what the next launch starts from)."""
import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, block_table_matrix, build_cache, oracle_cache, run_case, seeded_kv

pytestmark = pytest.mark.gpu
FP16, FP8 = 0, 1


@pytest.fixture
def skewed(pa):
    fused = pa.head_fused()
    pa.set_head_fused(1)
    pa.set_tail_steal(2)
    yield
    pa.set_tail_steal(0)
    pa.set_head_fused(fused)


def _lens(seed, batch, lo, hi):
    return np.random.default_rng(seed).integers(lo, hi + 1, batch).tolist()


CASES = [
    # dtype, hq, hkv, page size, lengths, forced CTAs
    (FP16, 32, 8, 16, _lens(1, 160, 1200, 1800), 0),
    (FP8, 32, 8, 16, _lens(2, 160, 1500, 2500), 0),
    (FP16, 64, 8, 16, _lens(3, 150, 900, 1100), 0),      # group 8
    (FP8, 64, 8, 16, _lens(4, 150, 1800, 2200), 0),
    (FP8, 8, 8, 32, _lens(5, 200, 700, 900), 0),         # group 1
    (FP16, 16, 8, 8, _lens(6, 170, 600, 1000), 0),       # two boxes per tile
    (FP16, 32, 8, 1, _lens(7, 152, 250, 350), 0),        # one box per token
    (FP16, 32, 8, 16, [640] * 296, 0),                   # short rows: many stay whole inside one CTA until a piece is taken
    (FP16, 32, 8, 48, _lens(8, 100, 1500, 1700), 60),    # odd page size, fewer CTAs than SMs
    (FP8, 32, 8, 16, _lens(9, 333, 100, 1300), 0),
]


@pytest.mark.parametrize("index,spec", list(enumerate(CASES)))
def test_skewed_cut_against_the_oracle(index, spec, torch_cuda, pa, skewed):
    dtype, hq, hkv, ps, lens, ctas = spec
    before = pa.tail_steal_count()
    case = Case(dtype, hq, hkv, ps, lens, num_ctas=ctas, seed=100 + index, shuffle=7 + index)
    err, out, want, info = run_case(case, torch_cuda, pa, check_bytes=False)
    assert err <= TOL, (spec[:4], err)
    assert pa.tail_steal_count() > before, "a cut this uneven leaves the early CTAs something to take"


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_repeated_launches_of_one_plan(dtype, torch_cuda, pa, skewed):
    torch = torch_cuda
    hq, hkv, ps = 32, 8, 16
    lens = _lens(11, 160, 1000, 2000)
    case = Case(dtype, hq, hkv, ps, lens, seed=55, shuffle=3)
    K, V = seeded_kv(lens, hkv, 128, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    q = np.random.default_rng(56).standard_normal((len(lens), hq, 128), dtype=np.float32).astype(np.float16)
    dq = torch.from_numpy(q.view(np.int16)).cuda().view(torch.float16)
    kc, vc = oracle_cache(case, cfg, K, V, model)
    bt = block_table_matrix(model, len(lens), cfg.max_pages_per_slot)
    want = ol.paged_decode(1, dtype, q.view(np.uint16), kc, vc, bt, lens, hq, hkv, 128, ps, k_scale=case.scale,
                           v_scale=case.scale, threads=0)
    cache.plan(list(range(len(lens))), hq)
    assert cache.describe_launch()["schedule"].endswith("work moving between CTAs")
    before = pa.tail_steal_count()
    outs = []
    for _ in range(6):
        out = torch.full_like(dq, float("nan"))
        cache.run(dq, out)
        outs.append(out)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    assert pa.tail_steal_count() >= before + 6
    for out in outs:
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert float(np.abs(got - want).max()) <= TOL
        assert float((out.float() - outs[0].float()).abs().max()) <= 2.5e-4
    # a new plan of the same cache (other rows first) starts from what the last launch left behind
    slots = list(range(len(lens)))[::-1]
    cache.plan(slots, hq)
    out = torch.full_like(dq, float("nan"))
    cache.run(dq, out)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    want_r = ol.paged_decode(1, dtype, q.view(np.uint16), kc, vc, bt[slots], [lens[s] for s in slots], hq, hkv, 128, ps,
                             k_scale=case.scale, v_scale=case.scale, threads=0)
    assert float(np.abs(out.float().cpu().numpy() - want_r).max()) <= TOL
    cache.close()


def test_switch_off_runs_the_plain_head_fused_kernel(torch_cuda, pa):
    """Mode 0 (what every bit-comparing suite runs with): no workspace for moved pieces, the plain kernel."""
    torch = torch_cuda
    lens = [1500] * 160
    case = Case(FP16, 32, 8, 16, lens, seed=5)
    K, V = seeded_kv(lens, 8, 128, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    cache.plan(list(range(len(lens))), 32)
    assert cache.describe_launch()["schedule"] == "head-fused rows"
    before = pa.tail_steal_count()
    dq = torch.randn(len(lens), 32, 128, device="cuda", dtype=torch.float16)
    a, b = torch.zeros_like(dq), torch.zeros_like(dq)
    cache.run(dq, a)
    cache.run(dq, b)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and pa.tail_steal_count() == before
    cache.close()
