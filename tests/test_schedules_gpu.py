"""The two schedules of the decode kernel on layers with 8 kv heads (both cache dtypes).

Plans made by the planner run, by default, with tiles of 16 tokens x all 8 kv heads (one consumer warp
per kv head, work cut by rows) where that wins (rows cut in at most 4 pieces); otherwise, and with the
switch off, they run the (row, kv head) schedule that every other shape uses.  The tests force each.  Both must agree with the oracle within the path's tolerance and with each other,
also when rows are cut into many pieces (separate merge kernel), for ragged batches, odd page sizes,
indirect slots and appends between steps.
"""
import numpy as np
import pytest

from common import TOL, Case, raw_decode, run_case, seeded_kv

pytestmark = pytest.mark.gpu

FP16, FP8 = 0, 1


@pytest.fixture
def both_schedules(pa):
    before = pa.head_fused()

    def run(fn):
        outs = []
        try:
            for mode in (2, 0):          # always head-fused, never head-fused
                pa.set_head_fused(mode)
                assert pa.head_fused() == mode
                outs.append(fn())
        finally:
            pa.set_head_fused(before)
        return outs
    return run


@pytest.mark.parametrize("ps,lens,ctas", [
    (16, [1], 0),
    (16, [15, 16, 17, 1, 4100], 0),
    (16, [8192] * 3, 0),
    (16, [20000], 0),            # one row cut into hundreds of pieces: merged by the separate kernel
    (16, [777, 3000, 64], 7),
    (16, [5000, 100], 1000),
    (1, [300, 5], 0),
    (8, [1000, 2000, 31], 0),
    (32, [4097, 33], 0),
    (128, [4000, 129], 0),
    (24, [1000, 25], 0),
    (4096, [5000, 4096], 0),
])
@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_fused_and_row_head_schedules_agree(dtype, ps, lens, ctas, torch_cuda, pa, both_schedules):
    case = Case(dtype, 32, 8, ps, lens, num_ctas=ctas, shuffle=9, seed=77)
    (e1, o1, want, i1), (e2, o2, _, i2) = both_schedules(lambda: run_case(case, torch_cuda, pa))
    assert e1 <= TOL and e2 <= TOL, (e1, e2)
    assert float(np.abs(o1 - o2).max()) <= TOL
    assert i1 == i2, "the plan a caller sees does not depend on the schedule"


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("hq", [8, 16, 32, 64])
def test_group_sizes_on_eight_kv_heads(dtype, hq, torch_cuda, pa, both_schedules):
    case = Case(dtype, hq, 8, 16, [2049, 300, 16], shuffle=3, seed=5)
    (e1, o1, _, _), (e2, o2, _, _) = both_schedules(lambda: run_case(case, torch_cuda, pa))
    assert e1 <= TOL and e2 <= TOL, (e1, e2)
    assert float(np.abs(o1 - o2).max()) <= TOL


def test_slot_indirection_in_both_schedules(torch_cuda, pa, both_schedules):
    torch = torch_cuda
    hq, hkv, d, ps = 32, 8, 128, 16
    lens = [900, 40, 2500, 333, 1]
    slots = [4, 2, 0]
    rng = np.random.default_rng(11)
    pages = [(n + ps - 1) // ps for n in lens]
    num_pages = sum(pages) + 2
    perm = rng.permutation(num_pages).astype(np.int32)
    bt = np.zeros((len(lens), max(pages) + 3), np.int32)
    at = 0
    for b, n in enumerate(pages):
        bt[b, :n] = perm[at:at + n]
        at += n
    kc = torch.randn(num_pages, hkv, ps, d, dtype=torch.float16, generator=torch.Generator().manual_seed(1)).cuda()
    vc = torch.randn(num_pages, hkv, ps, d, dtype=torch.float16, generator=torch.Generator().manual_seed(2)).cuda()
    q = torch.randn(len(slots), hq, d, dtype=torch.float16, generator=torch.Generator().manual_seed(3)).cuda()

    def run():
        out, _ = raw_decode(torch, pa, FP16, q, kc, vc, bt, lens, hq, hkv, ps, slot_ids=slots, num_pages=num_pages)
        return out.float().cpu().numpy()
    fused, plain = both_schedules(run)
    import oracle_lib as ol
    want = ol.paged_decode(1, FP16, q.cpu().numpy().view(np.uint16), kc.cpu().numpy().view(np.uint16).reshape(-1),
                           vc.cpu().numpy().view(np.uint16).reshape(-1), bt[slots], [lens[s] for s in slots],
                           hq, hkv, d, ps, threads=0)
    assert float(np.abs(fused - want).max()) <= TOL
    assert float(np.abs(plain - want).max()) <= TOL


def test_steps_with_appends_between_them(torch_cuda, pa, both_schedules):
    """A serving loop: decode, append one token to every sequence, plan again, decode; in both schedules
    the outputs track the oracle on the growing cache."""
    torch = torch_cuda
    import oracle_lib as ol
    from common import block_table_matrix, build_cache, oracle_cache
    lens0 = [31, 1000, 16]            # two of them cross a page boundary while growing
    steps = 3

    def run():
        case = Case(FP16, 32, 8, 16, [n + steps for n in lens0], shuffle=4, seed=8, extra_pages=6)
        K, V = seeded_kv(case.seq_lens, 8, 128, case.seed)
        first = Case(FP16, 32, 8, 16, lens0, shuffle=4, seed=8, extra_pages=6 + len(lens0))
        cache, model, cfg = build_cache(first, [k[:n] for k, n in zip(K, lens0)], [v[:n] for v, n in zip(V, lens0)],
                                        torch, pa)
        q = torch.randn(len(lens0), 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(6)).cuda()
        errs = []
        for s in range(steps):
            for b, n in enumerate(lens0):
                tok_k = torch.from_numpy(K[b][n + s:n + s + 1].view(np.int16)).cuda().view(torch.float16)
                tok_v = torch.from_numpy(V[b][n + s:n + s + 1].view(np.int16)).cuda().view(torch.float16)
                assert cache.append(b, tok_k, tok_v, 1) and model.append(b, 1)
            cur = [n + s + 1 for n in lens0]
            out = torch.zeros_like(q)
            cache.decode(q, out, len(lens0), 32, 0)
            torch.cuda.synchronize()
            assert pa.kernel_status() == 0
            now = Case(FP16, 32, 8, 16, cur, seed=8)
            kc, vc = oracle_cache(now, cfg, [k[:n] for k, n in zip(K, cur)], [v[:n] for v, n in zip(V, cur)], model)
            bt = block_table_matrix(model, len(lens0), cfg.max_pages_per_slot)
            want = ol.paged_decode(1, FP16, q.cpu().numpy().view(np.uint16), kc, vc, bt, cur, 32, 8, 128, 16, threads=0)
            errs.append(float(np.abs(out.float().cpu().numpy() - want).max()))
        cache.close()
        return errs
    fused, plain = both_schedules(run)
    assert max(fused) <= TOL and max(plain) <= TOL, (fused, plain)


def test_plan_rebuilt_from_arrays_gets_both_schedules(torch_cuda, pa):
    """C++ callers hand the device plan a decode::DecodePlan they hold as plain arrays
    (DevicePlan::upload, src/decode/decode.cu:112-156); the layer is recovered from the arrays, so such
    plans run the head-fused schedule too."""
    torch = torch_cuda
    from common import build_cache
    lens = [2049, 300, 4100, 16, 777]
    case = Case(FP16, 32, 8, 16, lens, shuffle=1, seed=21)
    K, V = seeded_kv(case.seq_lens, 8, 128, case.seed)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    q = torch.randn(len(lens), 32, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(12)).cuda()
    made = pa.make_plan(pa.KVDtype.FP16, lens, 32, 8, 128, 0)
    rebuilt = pa.plan_from_arrays(made.num_ctas, made.tile, made.segments, made.cta_seg_begin, made.item_seg_begin)
    before = pa.head_fused()
    outs = {}
    try:
        for name, plan in (("made", made), ("rebuilt", rebuilt)):
            for mode in (2, 0):
                pa.set_head_fused(mode)          # before the upload: it decides which schedules the device plan carries
                dp = pa.DevicePlan()
                dp.upload(plan, 4, 128)
                p = cache.params()
                out = torch.zeros_like(q)
                p.q, p.out, p.batch, p.num_q_heads = q.data_ptr(), out.data_ptr(), len(lens), 32
                dp.bind(p)
                pa.paged_decode(pa.KVDtype.FP16, p, 0, cfg.num_pages)
                torch.cuda.synchronize()
                assert pa.kernel_status() == 0
                outs[name, mode] = out
    finally:
        pa.set_head_fused(before)
    assert torch.equal(outs["made", 2], outs["rebuilt", 2])
    assert torch.equal(outs["made", 0], outs["rebuilt", 0])
    assert not torch.equal(outs["rebuilt", 2], outs["rebuilt", 0]), "the two schedules round differently somewhere"
    assert (outs["rebuilt", 2].float() - outs["rebuilt", 0].float()).abs().max().item() <= TOL
    cache.close()


@pytest.mark.parametrize("dtype", [FP16, FP8])
@pytest.mark.parametrize("hq", [8, 16])
@pytest.mark.parametrize("ctas", [0, 37, 50, 99])
def test_small_groups_with_split_rows(dtype, hq, ctas, torch_cuda, pa, both_schedules):
    """Groups of 1 and 2 query heads per kv head with rows cut across CTAs: the second schedule's partial
    rows start wherever the first schedule's workspace ends, and the merges read them 16 bytes at a time,
    so every region of the workspace has to start on a 16-byte boundary for any segment count."""
    case = Case(dtype, hq, 8, 16, [3000] * 21 + [17], num_ctas=ctas, shuffle=4, seed=15)
    (e1, o1, _, i1), (e2, o2, _, _) = both_schedules(lambda: run_case(case, torch_cuda, pa))
    assert e1 <= TOL and e2 <= TOL, (e1, e2)
    assert float(np.abs(o1 - o2).max()) <= TOL
    assert i1["segments"] > 22 * 8, "rows are split"
