"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol the
header declares, and its host logic (planner, argument checks, sizes) agrees with the oracle
and the golden vectors.  No compute call is made here."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import oracle_lib as ol

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")


def declared_symbols():
    with open(os.path.join(ROOT, "include", "pd_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(pd_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pa):
    from paged_attention_b200 import _lib
    L = C.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 45
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/pd_b200.h but not exported"
    # and the Python binding covers the same set
    assert sorted(_lib.SIGNATURES) == names


def test_params_struct_layout(pa):
    from paged_attention_b200 import _lib
    # decode::DecodeParams is 7 pointers, 6 ints + 3 floats, 3 pointers, 2 ints, 2 pointers on LP64
    assert C.sizeof(_lib.pd_params) == 7 * 8 + 9 * 4 + 4 + 3 * 8 + 2 * 4 + 2 * 8
    assert _lib.pd_params.segments.offset == 96 and _lib.pd_params.partial_lse.offset == 136
    assert C.sizeof(_lib.pd_cache_config) == 36


def test_dtype_helpers(pa):
    assert pa.kv_dtype_bytes(pa.KVDtype.FP16) == 2 and pa.kv_dtype_bytes(pa.KVDtype.FP8_E4M3) == 1
    assert pa.kv_dtype_name(pa.KVDtype.FP16) == "fp16" and pa.kv_dtype_name(pa.KVDtype.FP8_E4M3) == "fp8_e4m3"


def test_tile_tokens_and_dispatch_errors(pa):
    for dt in (pa.KVDtype.FP16, pa.KVDtype.FP8_E4M3):
        for g in (1, 2, 4, 8):
            t = pa.tile_tokens(dt, 128, g)
            assert t > 0 and t % 16 == 0
    with pytest.raises(pa.InvalidArgument, match="head_dim"):
        pa.tile_tokens(pa.KVDtype.FP16, 64, 4)
    with pytest.raises(pa.InvalidArgument, match="group"):
        pa.tile_tokens(pa.KVDtype.FP16, 128, 3)
    with pytest.raises(pa.InvalidArgument, match="group"):
        pa.tile_tokens(pa.KVDtype.FP8_E4M3, 128, 16)


def test_planner_matches_oracle_and_golden(pa):
    with open(os.path.join(GOLD, "planner.json")) as f:
        g = json.load(f)
    for p in g["plans"]:
        plan = pa.make_plan_tiled(p["tile"], p["seq_lens"], p["hq"], p["hkv"], p["num_ctas_in"])
        assert plan.tile == p["tile"] and plan.num_ctas == p["num_ctas"] and plan.num_segments == p["num_segments"]
        assert plan.item_seg_begin.tolist() == p["item_seg_begin"]
        assert int(plan.segments.astype(np.int64).sum()) == p["segments_sum"]
        assert int(plan.cta_seg_begin.astype(np.int64).sum()) == p["cta_seg_begin_sum"]
        if p["segments"] is not None:
            assert plan.segments.tolist() == p["segments"]
    rng = np.random.default_rng(17)
    for _ in range(200):
        b = int(rng.integers(1, 10))
        hkv = int(rng.choice([1, 2, 4, 8]))
        tile = int(rng.choice([16, 64, 128]))
        lens = rng.integers(1, 7000, b)
        nc = int(rng.integers(1, 800))
        plan = pa.make_plan_tiled(tile, lens, hkv * 2, hkv, nc)
        c, seg, cta, item = ol.make_plan(tile, nc, lens, hkv * 2, hkv)
        assert plan.num_ctas == c
        assert (plan.segments == seg).all() and (plan.cta_seg_begin == cta).all() and (plan.item_seg_begin == item).all()


def test_planner_with_the_kernels_own_tile(pa):
    # make_plan with an explicit grid needs no GPU; the cut is the oracle's at the kernel's tile
    for dt in (pa.KVDtype.FP16, pa.KVDtype.FP8_E4M3):
        lens = [8192] * 64
        plan = pa.make_plan(dt, lens, 32, 8, 128, 296)
        tile = pa.tile_tokens(dt, 128, 4)
        c, seg, cta, item = ol.make_plan(tile, 296, lens, 32, 8)
        assert plan.tile == tile and plan.num_ctas == c and (plan.segments == seg).all()
        # every CTA gets the same number of work units to within one
        per = [sum((s[3] - s[2] + tile - 1) // tile for s in seg[cta[i]:cta[i + 1]]) for i in range(c)]
        assert max(per) - min(per) <= 1 or min(per) == per[-1]


def test_planner_argument_errors(pa):
    with pytest.raises(pa.InvalidArgument, match="at least one token"):
        pa.make_plan_tiled(64, [5, 0], 8, 8, 4)
    with pytest.raises(pa.InvalidArgument, match="multiple"):
        pa.make_plan_tiled(64, [5], 7, 4, 4)
    with pytest.raises(pa.InvalidArgument, match="multiple"):
        pa.make_plan(pa.KVDtype.FP16, [5], 7, 4, 128, 4)
    with pytest.raises(pa.InvalidArgument, match="head_dim"):
        pa.make_plan(pa.KVDtype.FP16, [5], 8, 4, 96, 4)
    plan = pa.make_plan_tiled(64, [], 8, 8, 4)      # an empty batch is an empty plan, not a crash
    assert plan.num_ctas == 0 and plan.num_segments == 0


def test_page_sizing(pa):
    # bytes_per_page / pages_for_budget (src/decode/paged_kv_cache.cu:43-49 of the reference) and the
    # capacity table it published: 1 GiB -> 16384 fp16 pages / 32768 fp8 pages
    cfg = pa.PagedKVCache.Config(page_size=16, num_kv_heads=8, head_dim=128, dtype=pa.KVDtype.FP16)
    assert pa.PagedKVCache.bytes_per_page(cfg) == 65536
    assert pa.PagedKVCache.pages_for_budget(cfg, 1 << 30) == 16384
    cfg.dtype = pa.KVDtype.FP8_E4M3
    assert pa.PagedKVCache.bytes_per_page(cfg) == 32768
    assert pa.PagedKVCache.pages_for_budget(cfg, 1 << 30) == 32768


def test_cache_config_errors_need_no_gpu(pa):
    for bad in (dict(num_pages=0), dict(page_size=0), dict(num_kv_heads=0), dict(max_slots=0), dict(max_pages_per_slot=0)):
        kw = dict(num_pages=4, page_size=16, num_kv_heads=2, head_dim=128, max_slots=2, max_pages_per_slot=2)
        kw.update(bad)
        with pytest.raises(pa.InvalidArgument, match="positive"):
            pa.PagedKVCache(pa.PagedKVCache.Config(**kw))
    with pytest.raises(pa.InvalidArgument, match="head_dim"):
        pa.PagedKVCache(pa.PagedKVCache.Config(num_pages=4, page_size=16, num_kv_heads=2, head_dim=64, max_slots=2,
                                               max_pages_per_slot=2))


def test_every_exported_entry_point_is_declared():
    """Nothing is exported that the header does not declare (an undeclared export is an untested one)."""
    import subprocess
    from paged_attention_b200 import _lib
    out = subprocess.check_output(["nm", "-D", "--defined-only", _lib.LIB_PATH], text=True)
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line and line.split()[-1].startswith("pd_")}
    assert exported == set(declared_symbols()), exported ^ set(declared_symbols())


def test_product_does_not_reach_for_the_oracle():
    # the shipped package must not import, load or name the checker
    pkg = os.path.join(ROOT, "paged_attention_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                with open(os.path.join(dirpath, f)) as fh:
                    text = fh.read()
                assert "oracle" not in text.lower() or f == "build.py", f"{f} mentions the oracle"


def _check_cover(plan, lens, hkv, tile):
    """Every (row, kv head) is covered from 0 to its length by consecutive segments, in item order, and the
    CTA table walks the segment array without gaps."""
    seg, item, cta = plan.segments, plan.item_seg_begin, plan.cta_seg_begin
    assert item[0] == 0 and item[-1] == len(seg) and cta[0] == 0 and cta[-1] == len(seg)
    assert (np.diff(cta) >= 0).all() and (np.diff(item) >= 1).all()
    for i in range(len(lens) * hkv):
        b, h = divmod(i, hkv)
        at = 0
        for s in seg[item[i]:item[i + 1]]:
            assert (s[0], s[1], s[2]) == (b, h, at) and s[2] % tile == 0 and s[3] > s[2]
            at = s[3]
        assert at == lens[b]


def test_weighted_planner_shares_follow_the_weights(pa):
    rng = np.random.default_rng(5)
    for _ in range(30):
        tile = int(rng.choice([16, 64]))
        hkv = int(rng.choice([1, 2, 8]))
        lens = rng.integers(1, 9000, int(rng.integers(1, 80))).tolist()
        grid = int(rng.choice([1, 7, 148, 296, 443]))
        w = rng.uniform(0.7, 1.3, grid).astype(np.float32)
        plan = pa.make_plan_weighted(tile, lens, hkv * 4, hkv, w)
        assert plan.num_ctas == grid and plan.tile == tile
        _check_cover(plan, lens, hkv, tile)
        # tiles per CTA against the ideal share: off by less than one tile at each end
        tiles = np.zeros(grid)
        seg, cta = plan.segments, plan.cta_seg_begin
        for c in range(grid):
            for s in seg[cta[c]:cta[c + 1]]:
                tiles[c] += -(-(s[3] - s[2]) // tile)
        total = sum(-(-n // tile) for n in lens) * hkv
        assert tiles.sum() == total
        assert np.abs(tiles - total * w.astype(np.float64) / w.astype(np.float64).sum()).max() <= 1.0 + 1e-6
    # a CTA with weight 0 gets nothing and the rest still cover everything
    plan = pa.make_plan_weighted(64, [5000, 300], 32, 8, [1, 0, 1, 0, 0, 2])
    _check_cover(plan, [5000, 300], 8, 64)
    cta = plan.cta_seg_begin
    assert cta[1] == cta[2] and cta[3] == cta[4] == cta[5]
    with pytest.raises(pa.InvalidArgument):
        pa.make_plan_weighted(64, [10], 32, 8, [1.0, -1.0])


def test_equal_cut_covers_like_the_weighted_one(pa):
    lens = [8192] * 5 + [17]
    plan = pa.make_plan_tiled(64, lens, 32, 8, 296)
    _check_cover(plan, lens, 8, 64)
