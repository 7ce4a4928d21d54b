"""Pins the CPU oracle (oracle/pd_oracle.cpp) to the reference.

Always: against the golden vectors under tests/golden/, which were produced by the
reference's own code (tests/golden/make_golden.py).  When oracle/_ref has been built
here: also live against the reference compiled from its sources.
"""
import json
import os

import numpy as np
import pytest

import oracle_lib as ol
from golden_inputs import config1_inputs

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def same(a, b):
    return (a == b) | (np.isnan(a) & np.isnan(b))


def test_fp8_quantiser_matches_golden_for_every_half_value():
    g = np.load(os.path.join(GOLD, "conversions.npz"))
    allh = np.arange(65536, dtype=np.uint16)
    for i, scale in enumerate(g["scales"]):
        got = ol.quantize_e4m3(allh, float(scale))
        assert (got == g[f"q_{i}"]).all(), f"scale {scale}"


def test_fp8_known_values():
    # spot values of the E4M3 encoding: round to nearest even, saturate to +-448, flush tiny to zero
    L = ol.oracle()
    for x, want in [(0.3, 0x2a), (447.9, 0x7e), (500.0, 0x7e), (-1000.0, 0xfe), (17.0, 0x58), (19.0, 0x5a), (1e-4, 0x00),
                    (448.0, 0x7e), (-0.0, 0x80), (2.0 ** -9, 0x01), (2.0 ** -10, 0x00), (1.5 * 2.0 ** -9, 0x02)]:
        assert L.orc_e4m3_from_float(x) == want, x
    assert L.orc_e4m3_from_float(float("nan")) == 0x7f


def test_storage_conversions_match_golden():
    g = np.load(os.path.join(GOLD, "conversions.npz"))
    L = ol.oracle()
    e2f = np.array([L.orc_e4m3_to_float(b) for b in range(256)], np.float32)
    assert same(e2f, g["e4m3_to_float"]).all()
    h2f = np.array([L.orc_half_to_float(h) for h in range(65536)], np.float32)
    assert same(h2f, g["half_to_float"]).all()
    f2h = np.array([L.orc_float_to_half(float(x)) for x in g["f2h_in"]], np.uint16)
    assert (f2h == g["f2h_out"]).all()


def test_cpu_attention_matches_golden():
    g = np.load(os.path.join(GOLD, "cpu_attention.npz"))
    i = 0
    while f"q{i}" in g:
        got = ol.cpu_attention(g[f"q{i}"], g[f"K{i}"], g[f"V{i}"])
        assert np.array_equal(got, g[f"out{i}"]), f"case {i}"   # same scalar fp32 arithmetic: bit-exact
        i += 1
    assert i >= 5


def test_cpu_attention_closed_forms():
    # the three closed-form cases of the reference's CPU-attention test (tests/test_cpu_attention.cpp:7-67)
    d, T = 8, 16
    out = ol.cpu_attention(np.full(d, 0.5), np.full((T, d), 0.25), np.zeros((T, d)))
    assert (out == 0).all()
    V = np.repeat(np.arange(T, dtype=np.float32)[:, None], d, 1)
    out = ol.cpu_attention(np.ones(d), np.ones((T, d)), V)
    assert np.allclose(out, (T - 1) / 2.0, atol=1e-5)
    q = np.array([10.0, 0, 0, 0], np.float32)
    K = np.array([[1, 0, 0, 0], [0, 1, 0, 0]], np.float32)
    V = np.array([[1, 2, 3, 4], [5, 6, 7, 8]], np.float32)
    out = ol.cpu_attention(q, K, V)
    s = np.array([10.0, 0.0]) / 2.0
    w = np.exp(s - s[0])
    w /= w.sum()
    assert np.allclose(out, w @ V, atol=1e-5)


def test_planner_known_answers_and_golden_plans():
    with open(os.path.join(GOLD, "planner.json")) as f:
        g = json.load(f)
    # (ctas, segments) pairs the reference published for its H100 runs: grid 264 (fp16) / 396 (fp8) or the
    # swept grid sizes, tile 64
    n = 0
    for k in g["known_answers"]:
        lens = [k["seq_len"]] * k["batch"]
        if k["source"].endswith("h100_sweep.csv"):
            grids = [264 if k["dtype"] == 0 else 396]
        else:
            grids = [66, 132, 264, 396]   # the ctas sweep asked for sms/2, sms, 2 sms, 3 sms on 132 SMs
        hits = [ol.make_plan(64, nc, lens, k["hq"], k["hkv"]) for nc in grids]
        assert any(c == k["ctas"] and len(seg) == k["segments"] for c, seg, _, _ in hits), k
        n += 1
    assert n >= 28
    for p in g["plans"]:
        c, seg, cta, item = ol.make_plan(p["tile"], p["num_ctas_in"], p["seq_lens"], p["hq"], p["hkv"])
        assert c == p["num_ctas"] and len(seg) == p["num_segments"]
        assert int(seg.astype(np.int64).sum()) == p["segments_sum"]
        assert int(cta.astype(np.int64).sum()) == p["cta_seg_begin_sum"]
        assert item.tolist() == p["item_seg_begin"]
        if p["segments"] is not None:
            assert seg.tolist() == p["segments"]
        if p["cta_seg_begin"] is not None:
            assert cta.tolist() == p["cta_seg_begin"]


def test_planner_rejects_what_the_reference_rejects():
    with pytest.raises(ValueError):
        ol.make_plan(64, 8, [10, 0], 8, 8)        # a sequence without tokens
    with pytest.raises(ValueError):
        ol.make_plan(64, 8, [10], 7, 4)           # q heads not a multiple of kv heads


def test_config1_oracle_matches_reference_outputs():
    g = np.load(os.path.join(GOLD, "config1.npz"))
    c1 = config1_inputs()
    assert c1["sha256"] == str(g["inputs_sha256"]), "seeded inputs changed; regenerate the golden vectors"
    hq, hkv, d, ps = c1["hq"], c1["hkv"], c1["d"], c1["ps"]
    # build the paged fp16 cache with the oracle append and decode it with the oracle's fp32 path
    kc = np.zeros(512 * hkv * ps * d, np.uint16)
    vc = np.zeros_like(kc)
    for b in range(4):
        ol.append(0, c1["K"][b].astype(np.float16).view(np.uint16), c1["V"][b].astype(np.float16).view(np.uint16),
                  kc, vc, c1["block_table"][b], 0, hkv, d, ps)
    out = ol.paged_decode(0, 0, c1["q"].astype(np.float16).view(np.uint16), kc, vc, c1["block_table"], c1["seq_lens"],
                          hq, hkv, d, ps)
    assert np.array_equal(out, g["out_fp16_inputs"])          # identical arithmetic on identical values
    assert np.abs(out - g["out_fp32_inputs"]).max() < 2e-3     # fp16 rounding of the inputs only
    out64 = ol.paged_decode(1, 0, c1["q"].astype(np.float16).view(np.uint16), kc, vc, c1["block_table"],
                            c1["seq_lens"], hq, hkv, d, ps)
    assert np.abs(out64 - out).max() < 1e-5


def test_allocator_model_semantics():
    # free-list order, slot reuse, page recycling, -1 when full: the pool behaviour the reference tests
    # (tests/test_paged_decode.cu:206-221, tests/test_paged_pool.cpp:25-77, tests/test_contiguous_pool.cpp:34-65)
    p = ol.PoolModel(2, 16, 2, 4)
    s = p.admit()
    assert s == 0
    assert p.append(s, 32)
    assert p.free_pages() == 0 and p.table(s).tolist() == [0, 1]
    assert not p.append(s, 1)
    assert p.seq_len(s) == 32
    p.release(s)
    assert p.free_pages() == 2
    with pytest.raises(ValueError):
        p.release(s)
    with pytest.raises(ValueError):
        p.append(5, 1)
    # appending across a page boundary takes exactly one more page
    p = ol.PoolModel(4, 16, 3, 4)
    a = p.admit()
    p.append(a, 15)
    assert p.free_pages() == 3
    p.append(a, 1)
    assert p.free_pages() == 3
    p.append(a, 1)
    assert p.free_pages() == 2
    with pytest.raises(OverflowError):
        p.append(a, 16 * 4)
    # slots: first free slot is reused, -1 when every slot is taken
    b, c = p.admit(), p.admit()
    assert (a, b, c) == (0, 1, 2) and p.admit() == -1
    p.release(b)
    assert p.admit() == 1
    # released pages come back in table order and are reused last-in first-out
    p = ol.PoolModel(6, 16, 2, 6)
    a = p.admit()
    p.append(a, 48)
    assert p.table(a).tolist() == [0, 1, 2]
    p.release(a)
    assert p.free_list().tolist() == [5, 4, 3, 0, 1, 2]
    a = p.admit()
    p.append(a, 32)
    assert p.table(a).tolist() == [2, 1]


def test_capacity_known_answers():
    # results/h100_capacity.csv of the reference: 1 GiB budget, 16-token pages, 8 kv heads, d 128
    for dtype, elem in ((0, 2), (1, 1)):
        bytes_per_page = 2 * 8 * 16 * 128 * elem
        pages = (1 << 30) // bytes_per_page
        assert pages == (16384 if dtype == 0 else 32768)
        for actual, want16 in ((256, 1024), (512, 512), (1024, 256), (2048, 128), (4096, 64), (8192, 32)):
            p = ol.PoolModel(pages, 16, pages, 8192 // 16)
            n = 0
            while True:
                s = p.admit()
                if s < 0 or not p.append(s, actual):
                    break
                n += 1
            assert n == want16 * (1 if dtype == 0 else 2)


@pytest.mark.skipif(not ol.have_ref(), reason="oracle/_ref not built here")
def test_live_against_reference_build():
    R = ol.ref()
    rng = np.random.default_rng(3)
    for T in (1, 7, 300):
        q, K, V = (rng.standard_normal(s).astype(np.float32) for s in (128, (T, 128), (T, 128)))
        assert np.array_equal(ol.cpu_attention(q, K, V), ol.cpu_attention(q, K, V, use_ref=True))
    allh = np.arange(65536, dtype=np.uint16)
    for scale in (1.0, 5.0 / 448.0, 1e-3, 100.0):
        assert (ol.quantize_e4m3(allh, scale) == ol.quantize_e4m3(allh, scale, R.ref_quantize_e4m3)).all()
    for _ in range(50):
        b = int(rng.integers(1, 9))
        hkv = int(rng.choice([1, 2, 4, 8]))
        lens = rng.integers(1, 6000, b)
        nc = int(rng.integers(1, 900))
        for dtype in (0, 1):
            c, tile, seg, cta, item = ol.ref_make_plan(dtype, lens, hkv * 4, hkv, 128, nc)
            c2, seg2, cta2, item2 = ol.make_plan(tile, nc, lens, hkv * 4, hkv)
            assert c == c2 and (seg == seg2).all() and (cta == cta2).all() and (item == item2).all()
