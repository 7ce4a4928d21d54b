"""GPU parity tests of the decode path, through the C ABI.

The first block restates the reference's own hot-path suite (tests/test_paged_decode.cu:158-221)
case by case; the checker is the CPU oracle over the cache bytes as stored.  The allocator
decisions, block tables and cache bytes are compared bit-exactly inside run_case; outputs to
TOL = 2e-3 max-abs (the reference's own test allows 4e-3).  Where oracle/_ref is present the
reference's CUDA kernels run next to the engine on the same bytes.
"""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, block_table_matrix, build_cache, cache_bytes, device_view, oracle_cache, raw_decode, run_case, seeded_kv
from golden_inputs import config1_inputs

pytestmark = pytest.mark.gpu
FP16, FP8 = 0, 1
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


# ---- the reference's hot-path suite ----------------------------------------------------------

@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_single_token_sequence(dtype, torch_cuda, pa):
    err, *_ = run_case(Case(dtype, 32, 8, 16, [1]), torch_cuda, pa)
    assert err < TOL


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 4), (16, 4), (32, 8), (8, 1)])
def test_gqa_groups(dtype, hq, hkv, torch_cuda, pa):
    err, *_ = run_case(Case(dtype, hq, hkv, 16, [777]), torch_cuda, pa)
    assert err < TOL


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_mixed_length_batch(dtype, torch_cuda, pa):
    err, *_ = run_case(Case(dtype, 32, 8, 16, [1, 15, 16, 17, 129, 1000, 4099]), torch_cuda, pa)
    assert err < TOL


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("ps", [1, 8, 16, 32, 128])
def test_page_sizes(dtype, ps, torch_cuda, pa):
    err, *_ = run_case(Case(dtype, 16, 4, ps, [300, 2500]), torch_cuda, pa)
    assert err < TOL


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("ps", [2, 4, 5, 24, 64, 100, 4096])
def test_more_page_sizes(dtype, ps, torch_cuda, pa):
    # sizes that do not divide the tile (5, 24, 100) use boxes of gcd(page, tile) tokens
    err, *_ = run_case(Case(dtype, 16, 4, ps, [300, 2500]), torch_cuda, pa)
    assert err < TOL


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("ctas", [1, 2, 7, 64, 1000])
def test_forced_cta_counts(dtype, ctas, torch_cuda, pa):
    # few CTAs: long multi-sequence streams; many: sequences cut into many segments and merged
    err, _, _, info = run_case(Case(dtype, 32, 8, 16, [5000, 90, 1, 700], num_ctas=ctas), torch_cuda, pa)
    assert err < TOL
    assert info["num_ctas"] <= ctas


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_scattered_pages(dtype, torch_cuda, pa):
    # round-robin appends of 5 tokens interleave every sequence's pages in memory
    err, *_ = run_case(Case(dtype, 32, 8, 16, [400, 333, 612], chunk=5), torch_cuda, pa)
    assert err < TOL


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_long_sequence(dtype, torch_cuda, pa):
    err, *_ = run_case(Case(dtype, 32, 8, 16, [32768]), torch_cuda, pa)
    assert err < TOL


def test_fp8_quantization_error_is_small(torch_cuda, pa):
    # against the unquantised values FP8 adds bounded error (reference bound: 5e-2 at T = 2048)
    case = Case(FP8, 32, 8, 16, [2048])
    err, out, want_q, _ = run_case(case, torch_cuda, pa)
    assert err < TOL
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    q = np.random.default_rng(case.seed + 1).standard_normal((1, 32, 128), dtype=np.float32).astype(np.float16)
    kc = np.zeros(128 * 8 * 16 * 128, np.uint16)
    vc = np.zeros_like(kc)
    bt = np.arange(128, dtype=np.int32)[None]
    ol.append(0, K[0].view(np.uint16), V[0].view(np.uint16), kc, vc, bt[0], 0, 8, 128, 16)
    want = ol.paged_decode(1, 0, q.view(np.uint16), kc, vc, bt, [2048], 32, 8, 128, 16)
    assert np.abs(out - want).max() < 5e-2


def test_out_of_pages_rejects_append(torch_cuda, pa):
    torch = torch_cuda
    cfg = pa.PagedKVCache.Config(num_pages=2, page_size=16, num_kv_heads=1, head_dim=128, max_slots=2, max_pages_per_slot=4)
    cache = pa.PagedKVCache(cfg)
    d = torch.zeros(64 * 64, dtype=torch.float16, device="cuda")
    s = cache.admit()
    assert cache.append(s, d, d, 32)
    assert cache.free_pages() == 0
    assert not cache.append(s, d, d, 1)
    assert cache.seq_len(s) == 32
    cache.release(s)
    assert cache.free_pages() == 2
    cache.close()


# ---- error behaviour of the cache (same exceptions as the reference) -----------------------------

def test_cache_argument_errors(torch_cuda, pa):
    torch = torch_cuda
    cfg = pa.PagedKVCache.Config(num_pages=8, page_size=16, num_kv_heads=2, head_dim=128, max_slots=2, max_pages_per_slot=2)
    cache = pa.PagedKVCache(cfg)
    d = torch.zeros(64 * 2 * 128, dtype=torch.float16, device="cuda")
    with pytest.raises(pa.InvalidArgument, match="not admitted"):
        cache.append(0, d, d, 1)
    with pytest.raises(pa.InvalidArgument, match="not admitted"):
        cache.release(1)
    a, b = cache.admit(), cache.admit()
    assert (a, b) == (0, 1) and cache.admit() == -1
    assert cache.append(a, d, d, 0)                      # n <= 0 is a no-op that succeeds
    with pytest.raises(pa.LengthError, match="max_pages_per_slot"):
        cache.append(a, d, d, 33)
    assert cache.append(a, d, d, 32) and cache.seq_len(a) == 32 and cache.max_seq_len() == 32
    with pytest.raises(pa.InvalidArgument, match="not admitted"):
        cache.plan([0, 5], 4)
    with pytest.raises(pa.InvalidArgument, match="at least one token"):
        cache.plan([0, 1], 4)                            # slot 1 is admitted but empty
    with pytest.raises(pa.InvalidArgument, match="multiple"):
        cache.plan([0], 3)
    with pytest.raises(pa.InvalidArgument, match="group"):
        cache.plan([0], 32)                              # group 16 is not supported
    cache.release(b)
    assert cache.admit() == 1                            # first free slot is reused
    assert cache.total_bytes() == 8 * 2 * 2 * 16 * 128 * 2
    cache.close()


def test_page_recycling_follows_the_allocator_model(torch_cuda, pa):
    torch = torch_cuda
    cfg = pa.PagedKVCache.Config(num_pages=6, page_size=16, num_kv_heads=1, head_dim=128, max_slots=2, max_pages_per_slot=6)
    cache, model = pa.PagedKVCache(cfg), ol.PoolModel(6, 16, 2, 6)
    d = torch.zeros(96 * 128, dtype=torch.float16, device="cuda")
    for pool in (cache, model):
        pool.admit()
    assert cache.append(0, d, d, 48) and model.append(0, 48)
    cache.release(0), model.release(0)
    assert cache.free_list().tolist() == model.free_list().tolist() == [5, 4, 3, 0, 1, 2]
    cache.admit(), model.admit()
    assert cache.append(0, d, d, 15) and model.append(0, 15)
    assert cache.append(0, d, d, 2) and model.append(0, 2)     # crosses a page boundary
    assert cache.block_table(0).tolist() == model.table(0).tolist() == [2, 1]
    cache.shuffle_free_pages(42), model.shuffle(42)
    assert cache.free_list().tolist() == model.free_list().tolist()
    cache.close()


# ---- the benchmark spec's config 1 against the reference's CPU outputs ---------------------------------

def test_config1_against_reference_cpu_outputs(torch_cuda, pa):
    torch = torch_cuda
    g = np.load(os.path.join(GOLD, "config1.npz"))
    c1 = config1_inputs()
    assert c1["sha256"] == str(g["inputs_sha256"])
    hq, hkv, d, ps = c1["hq"], c1["hkv"], c1["d"], c1["ps"]
    k_cache = torch.zeros(512, hkv, ps, d, dtype=torch.float16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    bt = c1["block_table"]
    d_bt = torch.from_numpy(bt).cuda()
    for b in range(4):
        k = torch.from_numpy(c1["K"][b].astype(np.float16)).cuda()
        v = torch.from_numpy(c1["V"][b].astype(np.float16)).cuda()
        pa.append_tokens(pa.KVDtype.FP16, k, v, k_cache, v_cache, d_bt[b], 0, int(c1["seq_lens"][b]), hkv, d, ps)
    dq = torch.from_numpy(c1["q"].astype(np.float16)).cuda()
    out, plan = raw_decode(torch, pa, FP16, dq, k_cache, v_cache, bt, c1["seq_lens"], hq, hkv, ps, num_pages=512)
    out = out.float().cpu().numpy()
    assert out.shape == (4, 32, 128)
    assert np.abs(out - g["out_fp16_inputs"]).max() < TOL      # reference cpu_attention on the stored fp16 values
    assert np.abs(out - g["out_fp32_inputs"]).max() < TOL      # and on the original fp32 inputs


# ---- more of the domain ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_slot_ids_and_block_table_stride(dtype, torch_cuda, pa):
    # batch rows read cache slots out of order; the table is wider than any sequence needs
    torch = torch_cuda
    case = Case(dtype, 16, 4, 16, [130, 700, 64, 1], shuffle=3)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    kc, vc = oracle_cache(case, cfg, K, V, model)
    slots = [2, 0, 3]
    q = np.random.default_rng(5).standard_normal((3, 16, 128), dtype=np.float32).astype(np.float16)
    dq = torch.from_numpy(q).cuda()
    dout = torch.zeros_like(dq)
    cache.plan(slots, 16, 9)
    cache.run(dq, dout)
    torch.cuda.synchronize()
    bt = block_table_matrix(model, 4, cfg.max_pages_per_slot)
    want = ol.paged_decode(1, dtype, q.view(np.uint16), kc, vc, bt, case.seq_lens, 16, 4, 128, 16, k_scale=case.scale,
                           v_scale=case.scale, slot_ids=slots)
    assert np.abs(dout.float().cpu().numpy() - want).max() < TOL
    # run() again with the same plan (one plan per step, one run per layer) is bit-identical
    dout2 = torch.zeros_like(dq)
    cache.run(dq, dout2)
    torch.cuda.synchronize()
    assert torch.equal(dout, dout2)
    cache.close()


@pytest.mark.parametrize("ps", [4, 8, 16, 32, 64])
def test_ragged_batch_page_size_sweep(ps, torch_cuda, pa):
    # 48 sequences, lengths log-uniform in [64, 8192] (seeded): cross-sequence work ranges + split merge
    rng = np.random.default_rng(99)
    lens = np.round(np.exp(rng.uniform(np.log(64), np.log(8192), 48))).astype(int).tolist()
    err, _, _, info = run_case(Case(FP16, 32, 8, ps, lens, shuffle=11), torch_cuda, pa, check_bytes=(ps == 16))
    assert err < TOL
    assert info["segments"] > 48 * 8     # some rows were split


def test_fp8_cache_against_fp16_cache(torch_cuda, pa):
    # K/V ~ N(0,1) quantised at append time with per-tensor scale amax/448; the FP8 result differs from
    # the FP16-cache result by quantisation only (the reference reports relative L2 of 3.8e-2)
    torch = torch_cuda
    lens = [4096] * 4
    K, V = seeded_kv(lens, 8, 128, 77)
    k_scale = float(max(np.abs(k.astype(np.float32)).max() for k in K)) / 448.0
    c16 = Case(FP16, 32, 8, 16, lens, seed=77, shuffle=5)
    c8 = Case(FP8, 32, 8, 16, lens, seed=77, shuffle=5, scale=k_scale)
    e16, o16, _, _ = run_case(c16, torch, pa)
    e8, o8, _, _ = run_case(c8, torch, pa)
    assert e16 < TOL and e8 < TOL
    rel = np.linalg.norm(o8 - o16) / np.linalg.norm(o16)
    assert 1e-3 < rel < 6e-2


def test_garbage_past_the_end_of_a_page_is_ignored(torch_cuda, pa):
    # a caller-owned pool that was never cleared: NaN bytes beyond the last token of a sequence
    # (and in unused pages) must not reach the output
    torch = torch_cuda
    hq, hkv, ps, n = 8, 2, 16, 37
    for dtype, tdt in ((FP16, torch.float16), (FP8, torch.uint8)):
        fill = float("nan") if dtype == FP16 else 0x7f
        k_cache = torch.full((8, hkv, ps, 128), fill, dtype=tdt, device="cuda")
        v_cache = torch.full((8, hkv, ps, 128), fill, dtype=tdt, device="cuda")
        bt = np.array([[5, 2, 7, 0]], np.int32)
        K, V = seeded_kv([n], hkv, 128, 3)
        scale = 4.0 / 448.0 if dtype == FP8 else 1.0
        pa.append_tokens(pa.KVDtype(dtype), torch.from_numpy(K[0]).cuda(), torch.from_numpy(V[0]).cuda(), k_cache, v_cache,
                         torch.from_numpy(bt[0]).cuda(), 0, n, hkv, 128, ps, scale, scale)
        q = np.random.default_rng(4).standard_normal((1, hq, 128), dtype=np.float32).astype(np.float16)
        out, _ = raw_decode(torch, pa, dtype, torch.from_numpy(q).cuda(), k_cache, v_cache, bt, [n], hq, hkv, ps, scale, scale)
        out = out.float().cpu().numpy()
        assert np.isfinite(out).all()
        kc = k_cache.cpu().numpy().view(np.uint16 if dtype == FP16 else np.uint8).reshape(-1)
        vc = v_cache.cpu().numpy().view(np.uint16 if dtype == FP16 else np.uint8).reshape(-1)
        want = ol.paged_decode(1, dtype, q.view(np.uint16), kc, vc, bt, [n], hq, hkv, 128, ps, k_scale=scale, v_scale=scale)
        assert np.abs(out - want).max() < TOL


# ---- next to the reference's own CUDA kernels --------------------------------------------------------------------

@pytest.mark.skipif(not ol.have_ref(), reason="oracle/_ref not built")
@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_against_reference_cache_and_kernels(dtype, torch_cuda, pa):
    """The reference's PagedKVCache (append + decode) and the engine on the same seeded inputs: block
    tables and cache bytes bit-exact, outputs within TOL of each other."""
    torch = torch_cuda
    R = ol.ref()
    case = Case(dtype, 32, 8, 16, [1, 15, 16, 17, 129, 1000, 4099, 2048], shuffle=42, chunk=300)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    B = len(case.seq_lens)
    rc = R.ref_cache_create(cfg.num_pages, 16, 8, 128, B, cfg.max_pages_per_slot, dtype, case.scale, case.scale)
    assert rc
    R.ref_cache_shuffle(rc, 42)
    dK = [torch.from_numpy(k).cuda() for k in K]
    dV = [torch.from_numpy(v).cuda() for v in V]
    done = [0] * B
    for b in range(B):
        assert R.ref_cache_admit(rc) == b
    progress = True
    while progress:
        progress = False
        for b in range(B):
            n = min(300, case.seq_lens[b] - done[b])
            if n <= 0:
                continue
            assert R.ref_cache_append(rc, b, dK[b][done[b]:].data_ptr(), dV[b][done[b]:].data_ptr(), n) == 1
            done[b] += n
            progress = True
    for b in range(B):
        t = np.zeros(cfg.max_pages_per_slot, np.int32)
        n = R.ref_cache_table(rc, b, t.ctypes.data_as(C.POINTER(C.c_int)), len(t))
        assert t[:n].tolist() == cache.block_table(b).tolist()
    assert R.ref_cache_free_pages(rc) == cache.free_pages()
    ptrs = [C.c_void_p() for _ in range(4)]
    R.ref_cache_pointers(rc, *[C.byref(p) for p in ptrs])
    elems = cfg.num_pages * 8 * 16 * 128 * (2 if dtype == FP16 else 1)
    mine_k, mine_v = cache_bytes(cache, cfg, torch)
    # the reference never clears its pools: compare the bytes that were written
    kc, vc = oracle_cache(case, cfg, K, V, model)
    written = np.zeros(cfg.num_pages * 8 * 16 * 128, bool)
    for b, n in enumerate(case.seq_lens):
        table = model.table(b)
        for t in range(n):
            base = ((table[t // 16] * 8) * 16 + t % 16) * 128
            for h in range(8):
                written[base + h * 16 * 128: base + h * 16 * 128 + 128] = True
    np_dt = np.uint16 if dtype == FP16 else np.uint8
    ref_k = device_view(ptrs[0].value, elems, torch).cpu().numpy().view(np_dt)
    ref_v = device_view(ptrs[1].value, elems, torch).cpu().numpy().view(np_dt)
    assert (ref_k[written] == mine_k[written]).all() and (ref_v[written] == mine_v[written]).all()
    assert (kc[written] == mine_k[written]).all()
    q = np.random.default_rng(8).standard_normal((B, 32, 128), dtype=np.float32).astype(np.float16)
    dq = torch.from_numpy(q).cuda()
    o_ref, o_mine = torch.zeros_like(dq), torch.zeros_like(dq)
    assert R.ref_cache_decode(rc, dq.data_ptr(), o_ref.data_ptr(), B, 32, 0) == 0
    cache.decode(dq, o_mine, B, 32)
    torch.cuda.synchronize()
    assert (o_ref.float() - o_mine.float()).abs().max().item() < TOL
    R.ref_cache_destroy(rc)
    cache.close()


@pytest.mark.skipif(not ol.have_ref(), reason="oracle/_ref not built")
@pytest.mark.parametrize("dtype,B,L", [(FP16, 16, 8192), (FP8, 32, 4096)])
def test_reference_kernel_on_the_same_quantised_cache(dtype, B, L, torch_cuda, pa):
    """The reference's decode kernel reads the engine's own cache (same quantised bytes, same table)."""
    torch = torch_cuda
    R = ol.ref()
    pages = L // 16
    scale = 5.0 / 448.0 if dtype == FP8 else 1.0
    cfg = pa.PagedKVCache.Config(num_pages=pages * B, page_size=16, num_kv_heads=8, head_dim=128, max_slots=B,
                                 max_pages_per_slot=pages, dtype=pa.KVDtype(dtype), k_scale=scale, v_scale=scale)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(42)
    gen = torch.Generator(device="cuda").manual_seed(3)
    for b in range(B):
        k = torch.randn(L, 8, 128, device="cuda", dtype=torch.float16, generator=gen)
        v = torch.randn(L, 8, 128, device="cuda", dtype=torch.float16, generator=gen)
        assert cache.append(cache.admit(), k, v, L)
    dq = torch.randn(B, 32, 128, device="cuda", dtype=torch.float16, generator=gen)
    mine, ref = torch.zeros_like(dq), torch.zeros_like(dq)
    cache.decode(dq, mine, B, 32)
    p = cache.params()
    dec = R.ref_decoder_create()
    lens = np.full(B, L, np.int32)
    assert R.ref_decoder_plan(dec, dtype, lens.ctypes.data_as(C.POINTER(C.c_int)), B, 32, 8, 128, 0) == 0
    assert R.ref_decoder_run(dec, dtype, dq.data_ptr(), ref.data_ptr(), p.k_cache, p.v_cache, p.block_table, pages,
                             p.seq_lens, B, 32, 8, 128, 16, scale, scale, None) == 0
    torch.cuda.synchronize()
    assert (mine.float() - ref.float()).abs().max().item() < TOL
    R.ref_decoder_destroy(dec)
    cache.close()


# ---- full-size properties (the headline shape) ------------------------------------------------------------------------

def test_headline_shape_properties(torch_cuda, pa):
    """Batch 64 x 8192, fp16, 16-token scattered pages.  Size-independent checks: the result does not
    depend on how rows are split over CTAs, a repeated run is bit-identical, and sampled rows agree
    with the oracle."""
    torch = torch_cuda
    B, L, hq, hkv = 64, 8192, 32, 8
    pages = L // 16
    cfg = pa.PagedKVCache.Config(num_pages=pages * B, page_size=16, num_kv_heads=hkv, head_dim=128, max_slots=B,
                                 max_pages_per_slot=pages)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(42)
    gen = torch.Generator(device="cuda").manual_seed(1)
    for b in range(B):
        k = torch.randn(L, hkv, 128, device="cuda", dtype=torch.float16, generator=gen)
        v = torch.randn(L, hkv, 128, device="cuda", dtype=torch.float16, generator=gen)
        assert cache.append(cache.admit(), k, v, L)
    assert cache.free_pages() == 0
    dq = torch.randn(B, hq, 128, device="cuda", dtype=torch.float16, generator=gen)
    outs = []
    for ctas in (0, 148, 1000):
        o = torch.zeros_like(dq)
        cache.decode(dq, o, B, hq, ctas)
        torch.cuda.synchronize()
        assert pa.kernel_status() == 0
        outs.append(o)
    assert (outs[0].float() - outs[1].float()).abs().max().item() < 1e-3
    assert (outs[0].float() - outs[2].float()).abs().max().item() < 1e-3
    again = torch.zeros_like(dq)
    cache.decode(dq, again, B, hq, 1000)
    torch.cuda.synchronize()
    assert torch.equal(again, outs[2])
    # oracle on two sampled rows: gather their pages to the host
    p = cache.params()
    pool_bytes = cfg.num_pages * hkv * 16 * 128 * 2
    kpool = device_view(p.k_cache, pool_bytes, torch).view(torch.float16).view(cfg.num_pages, hkv * 16 * 128)
    vpool = device_view(p.v_cache, pool_bytes, torch).view(torch.float16).view(cfg.num_pages, hkv * 16 * 128)
    for row in (0, 41):
        table = torch.from_numpy(cache.block_table(row).astype(np.int64)).cuda()
        kc = kpool[table].cpu().numpy().view(np.uint16).reshape(-1)
        vc = vpool[table].cpu().numpy().view(np.uint16).reshape(-1)
        q = dq[row:row + 1].cpu().numpy()
        want = ol.paged_decode(1, FP16, q.view(np.uint16), kc, vc, np.arange(pages, dtype=np.int32)[None], [L], hq, hkv, 128, 16)
        assert np.abs(outs[0][row].float().cpu().numpy() - want[0]).max() < TOL
    cache.close()
