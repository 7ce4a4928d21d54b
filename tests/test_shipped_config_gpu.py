"""The configuration that ships: adaptive cut ON (device plans cut in shares that follow the per-CTA rates
of earlier launches) on top of the default schedule choice, at the real sizes of the benchmark workloads.

The other suites switch the adaptive cut off because they compare bits between entry points; here it stays
on, a dozen plan + run steps let the shares move first, and the outputs are compared with the ORACLE (the
double-precision restatement of the reference's test oracle, tests/test_paged_decode.cu:111-145 of the
reference) on sampled rows, whose cache pages are gathered from the device pool as stored:

  C2  batch 64 x 8192, fp16, 16-token pages                      (the headline workload)
  C3  batch 128 x 4096, e4m3 with the per-tensor scale amax/448  (scripts/compare_flashinfer.py:87-91 of the
      reference), also against the reference's own FP8 kernel on the same bytes where oracle/_ref is built
  C4  256 sequences, lengths log-uniform in [64, 32768], fp16, page sizes 4..64
  C5  the 70B-shaped layer (64 query / 8 kv heads, group 8), e4m3, 16384 tokens per row

plus the same through indirect slots and through a plan cut on the device, and cuts with unequal shares of
random shapes (the weighted planner's plans run as the caller's own plan).
"""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, block_table_matrix, build_cache, device_view, oracle_cache, seeded_kv

pytestmark = pytest.mark.gpu
FP16, FP8 = 0, 1


@pytest.fixture
def adaptive_on(pa):
    """Runs after the autouse fixture that switches the adaptive cut off."""
    pa.adaptive_cut_reset()
    pa.set_adaptive_cut(True)
    yield
    pa.set_adaptive_cut(False)
    pa.adaptive_cut_reset()


def _fill(torch, pa, dtype, lens, hkv, ps, seed, scale=None):
    """A cache whose slots hold prefixes of one seeded source sequence (host work stays small; rows still
    differ through their pages and their queries).  Returns (cache, cfg, scale)."""
    top = max(lens)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(top, hkv, 128, device="cuda", dtype=torch.float16, generator=gen)
    v = torch.randn(top, hkv, 128, device="cuda", dtype=torch.float16, generator=gen)
    if scale is None:
        scale = 1.0
        if dtype == FP8:      # one per-tensor scale = amax / 448
            scale = float(max(k.abs().max().item(), v.abs().max().item())) / 448.0
    pages = [(n + ps - 1) // ps for n in lens]
    cfg = pa.PagedKVCache.Config(num_pages=sum(pages), page_size=ps, num_kv_heads=hkv, head_dim=128, max_slots=len(lens),
                                 max_pages_per_slot=max(pages), dtype=pa.KVDtype(dtype), k_scale=scale, v_scale=scale)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(42)
    for b, n in enumerate(lens):
        assert cache.admit() == b and cache.append(b, k, v, n)
    assert cache.free_pages() == 0
    return cache, cfg, scale


def _oracle_rows(torch, cache, cfg, dtype, dq, rows, lens, hq, scale, slots=None):
    """Oracle outputs of the sampled batch rows, from the cache bytes as stored on the device."""
    hkv, ps = cfg.num_kv_heads, cfg.page_size
    elem = 2 if dtype == FP16 else 1
    page_elems = hkv * ps * 128
    p = cache.params()
    t_dt, n_dt = (torch.float16, np.uint16) if dtype == FP16 else (torch.uint8, np.uint8)
    kpool = device_view(p.k_cache, cfg.num_pages * page_elems * elem, torch).view(t_dt).view(cfg.num_pages, page_elems)
    vpool = device_view(p.v_cache, cfg.num_pages * page_elems * elem, torch).view(t_dt).view(cfg.num_pages, page_elems)
    out = {}
    for row in rows:
        slot = row if slots is None else slots[row]
        n = lens[slot]
        pages = (n + ps - 1) // ps
        table = torch.from_numpy(cache.block_table(slot).astype(np.int64)).cuda()
        kc = kpool[table].cpu().numpy().view(n_dt).reshape(-1)
        vc = vpool[table].cpu().numpy().view(n_dt).reshape(-1)
        q = dq[row:row + 1].cpu().numpy()
        out[row] = ol.paged_decode(1, dtype, q.view(np.uint16), kc, vc, np.arange(pages, dtype=np.int32)[None], [n], hq, hkv,
                                   128, ps, k_scale=scale, v_scale=scale)[0]
    return out


def _settle(torch, pa, cache, slots, hq, dq, steps=12, layers=3):
    """A serving-style loop: plan, a few layers, again; the adaptive cut folds in one reading per plan."""
    out = torch.zeros_like(dq)
    for _ in range(steps):
        cache.plan(slots, hq)
        for _ in range(layers):
            cache.run(dq, out)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    return out


def _check(torch, out, want):
    for row, w in want.items():
        err = float(np.abs(out[row].float().cpu().numpy() - w).max())
        assert err <= TOL, (row, err)


def test_c2_headline_with_moving_shares(torch_cuda, pa, adaptive_on):
    torch = torch_cuda
    B, L, hq, hkv = 64, 8192, 32, 8
    cache, cfg, scale = _fill(torch, pa, FP16, [L] * B, hkv, 16, 1)
    dq = torch.randn(B, hq, 128, device="cuda", dtype=torch.float16, generator=torch.Generator(device="cuda").manual_seed(2))
    out = _settle(torch, pa, cache, list(range(B)), hq, dq)
    moved = [w for w, n in pa.adaptive_cut_tables() if n > 0 and float(np.abs(w - 1).max()) > 0]
    assert moved, "a 300 us layer gives usable per-CTA rates: the shares have left the equal cut"
    info = cache.describe_launch()
    assert info["schedule"] == "head-fused rows" and info["kv_heads_per_tile"] == 8 and info["tile_tokens"] == 16
    _check(torch, out, _oracle_rows(torch, cache, cfg, FP16, dq, (0, 29, 63), [L] * B, hq, scale))
    # the same step through indirect slots (rows read the slots in reverse) and a plan cut on the device
    slots = list(range(B))[::-1]
    out2 = _settle(torch, pa, cache, slots, hq, dq, steps=2, layers=1)
    _check(torch, out2, _oracle_rows(torch, cache, cfg, FP16, dq, (0, 5), [L] * B, hq, scale, slots=slots))
    out3 = torch.zeros_like(dq)
    for _ in range(3):
        cache.plan_device(B, hq)
        cache.run(dq, out3)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    _check(torch, out3, _oracle_rows(torch, cache, cfg, FP16, dq, (1, 62), [L] * B, hq, scale))
    cache.close()


def test_c3_fp8_with_moving_shares(torch_cuda, pa, adaptive_on):
    torch = torch_cuda
    B, L, hq, hkv = 128, 4096, 32, 8
    cache, cfg, scale = _fill(torch, pa, FP8, [L] * B, hkv, 16, 3)
    dq = torch.randn(B, hq, 128, device="cuda", dtype=torch.float16, generator=torch.Generator(device="cuda").manual_seed(4))
    out = _settle(torch, pa, cache, list(range(B)), hq, dq)
    _check(torch, out, _oracle_rows(torch, cache, cfg, FP8, dq, (0, 77, 127), [L] * B, hq, scale))
    if ol.have_ref():
        # the reference's own FP8 kernel on the engine's cache: same quantised bytes, same table
        R = ol.ref()
        ref = torch.zeros_like(dq)
        p = cache.params()
        dec = R.ref_decoder_create()
        lens = np.full(B, L, np.int32)
        assert R.ref_decoder_plan(dec, FP8, lens.ctypes.data_as(C.POINTER(C.c_int)), B, hq, hkv, 128, 0) == 0
        assert R.ref_decoder_run(dec, FP8, dq.data_ptr(), ref.data_ptr(), p.k_cache, p.v_cache, p.block_table, L // 16,
                                 p.seq_lens, B, hq, hkv, 128, 16, scale, scale, None) == 0
        torch.cuda.synchronize()
        assert (out.float() - ref.float()).abs().max().item() <= TOL
        R.ref_decoder_destroy(dec)
    cache.close()


@pytest.mark.parametrize("ps", [4, 8, 16, 32, 64])
def test_c4_ragged_batch_with_moving_shares(ps, torch_cuda, pa, adaptive_on):
    torch = torch_cuda
    hq, hkv = 32, 8
    rng = np.random.default_rng(2024)
    lens = np.round(np.exp(rng.uniform(np.log(64), np.log(32768), 256))).astype(int).tolist()
    cache, cfg, scale = _fill(torch, pa, FP16, lens, hkv, ps, 5)
    B = len(lens)
    dq = torch.randn(B, hq, 128, device="cuda", dtype=torch.float16, generator=torch.Generator(device="cuda").manual_seed(6))
    out = _settle(torch, pa, cache, list(range(B)), hq, dq, steps=8, layers=2)
    longest, shortest = int(np.argmax(lens)), int(np.argmin(lens))
    _check(torch, out, _oracle_rows(torch, cache, cfg, FP16, dq, (0, longest, shortest, 255), lens, hq, scale))
    cache.close()


def test_c5_shape_group_of_eight_fp8(torch_cuda, pa, adaptive_on):
    torch = torch_cuda
    B, L, hq, hkv = 32, 16384, 64, 8          # the 70B-shaped layer's rows; 32 of its 256 rows keep the pool at 1 GiB
    cache, cfg, scale = _fill(torch, pa, FP8, [L] * B, hkv, 16, 7)
    dq = torch.randn(B, hq, 128, device="cuda", dtype=torch.float16, generator=torch.Generator(device="cuda").manual_seed(8))
    out = _settle(torch, pa, cache, list(range(B)), hq, dq)
    _check(torch, out, _oracle_rows(torch, cache, cfg, FP8, dq, (0, 13, 31), [L] * B, hq, scale))
    # one kv head per GPU, as on eight GPUs: the shard's pool has a single head and group stays 8
    shard, scfg, sscale = _fill(torch, pa, FP8, [L] * B, 1, 16, 9)
    sq = dq[:, :8].contiguous()
    sout = _settle(torch, pa, shard, list(range(B)), 8, sq, steps=4, layers=2)
    _check(torch, sout, _oracle_rows(torch, shard, scfg, FP8, sq, (0, 31), [L] * B, 8, sscale))
    shard.close()
    cache.close()


def _weighted_cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        hkv = int(rng.choice([1, 2, 4, 8, 8]))
        group = int(rng.choice([1, 2, 4, 8]))
        ps = int(rng.choice([1, 3, 8, 16, 16, 32, 100]))
        batch = int(rng.integers(1, 24))
        lens = rng.integers(1, int(rng.choice([300, 5000])) + 1, batch).tolist()
        ctas = int(rng.choice([2, 7, 40, 148, 296, 500]))
        out.append((int(rng.integers(0, 2)), hkv * group, hkv, ps, lens, ctas, int(rng.integers(0, 1 << 16))))
    return out


@pytest.mark.parametrize("index,spec", list(enumerate(_weighted_cases(77, 24))))
def test_unequal_shares_of_random_shapes(index, spec, torch_cuda, pa):
    """Cuts with unequal shares (what the adaptive cut produces) on shapes too short for it to engage by itself:
    the weighted planner's plan, with random shares between 0.7 and 1.3 and a few CTAs left nearly empty, is
    uploaded as the caller's own plan and run against the oracle."""
    torch = torch_cuda
    dtype, hq, hkv, ps, lens, ctas, seed = spec
    case = Case(dtype, hq, hkv, ps, lens, seed=seed, shuffle=seed % 89)
    K, V = seeded_kv(case.seq_lens, hkv, 128, seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    kc, vc = oracle_cache(case, cfg, K, V, model)
    B = len(lens)
    rng = np.random.default_rng(seed)
    weights = rng.uniform(0.7, 1.3, ctas).astype(np.float32)
    weights[rng.integers(0, ctas, max(1, ctas // 16))] = 1e-3
    tile = pa.tile_tokens(pa.KVDtype(dtype), 128, hq // hkv)
    plan = pa.make_plan_weighted(tile, lens, hq, hkv, weights)
    q = rng.standard_normal((B, hq, 128), dtype=np.float32).astype(np.float16)
    dq = torch.from_numpy(q).cuda()
    out = torch.zeros_like(dq)
    dp = pa.DevicePlan()
    dp.upload(plan, hq // hkv, 128)
    p = cache.params()
    p.q, p.out, p.batch, p.num_q_heads = dq.data_ptr(), out.data_ptr(), B, hq
    dp.bind(p)
    pa.paged_decode(pa.KVDtype(dtype), p, 0, cfg.num_pages)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    bt = block_table_matrix(model, B, cfg.max_pages_per_slot)
    want = ol.paged_decode(1, dtype, q.view(np.uint16), kc, vc, bt, lens, hq, hkv, 128, ps, k_scale=case.scale,
                           v_scale=case.scale)
    assert float(np.abs(out.float().cpu().numpy() - want).max()) <= TOL
    cache.close()


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_many_launches_leave_nothing_behind(dtype, torch_cuda, pa, adaptive_on):
    """600 launches of a ragged batch whose rows are cut in up to four pieces, a new plan every seventh launch,
    outputs pre-filled with NaN: a row that was not merged, or merged before all its pieces had landed, shows."""
    torch = torch_cuda
    rng = np.random.default_rng(77)
    lens = rng.integers(300, 5000, 96).tolist()
    hq, hkv = 32, 8
    cache, cfg, scale = _fill(torch, pa, dtype, lens, hkv, 16, 4)
    B = len(lens)
    dq = torch.randn(B, hq, 128, device="cuda", dtype=torch.float16, generator=torch.Generator(device="cuda").manual_seed(6))
    out = torch.zeros_like(dq)
    slots = list(range(B))
    first = None
    for i in range(600):
        if i % 7 == 0:
            cache.plan(slots, hq)
        out.fill_(float("nan"))
        cache.run(dq, out)
        if i % 40 == 39:
            torch.cuda.synchronize()
            assert torch.isfinite(out).all()
            if first is None:
                first = out.clone()
            assert float((out.float() - first.float()).abs().max()) <= 2.5e-4
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    _check(torch, out, _oracle_rows(torch, cache, cfg, dtype, dq, (0, 50, B - 1), lens, hq, scale))
    cache.close()
