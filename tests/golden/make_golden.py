"""Generates the golden vectors under tests/golden/ from the reference itself.

Needs oracle/_ref/libpd_ref.so (the reference compiled from its own sources:
`make -C oracle ref REF=<checkout>`) and, for the planner known answers, the
reference's published results CSVs.  Run once where the reference is available:

    python tests/golden/make_golden.py [<reference checkout>]

Only CPU paths of the reference run here (cpu_attention, make_plan with an
explicit CTA count, the CUDA headers' host-side fp16/fp8 conversions).
"""
import csv
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402


def main():
    refdir = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    R = ol.ref()
    assert R is not None, "build oracle/_ref first"

    # 1. planner: published (ctas, segments) pairs + full plans from the reference's make_plan
    known = []
    for name in ("h100_sweep.csv", "h100_ctas.csv"):
        with open(os.path.join(refdir, "results", name)) as f:
            rows = list(csv.reader(f))
        for r in rows:
            if r[0] == "gpu":
                continue
            known.append({"source": "results/" + name, "dtype": 0 if r[1] == "fp16" else 1, "batch": int(r[2]),
                          "seq_len": int(r[3]), "hq": int(r[4]), "hkv": int(r[5]), "page": int(r[7]),
                          "ctas": int(r[8]), "segments": int(r[9])})
    plans = []
    rng = np.random.default_rng(2024)
    cases = [([8192] * 32, 32, 8, 264), ([1024] * 128, 32, 8, 396), ([5000, 90, 1, 700], 32, 8, 7),
             ([5000, 90, 1, 700], 32, 8, 1000), ([1, 15, 16, 17, 129, 1000, 4099], 32, 8, 296), ([1], 8, 8, 5),
             ([131072], 32, 8, 264)]
    for _ in range(12):
        b = int(rng.integers(1, 12))
        hkv = int(rng.choice([1, 2, 4, 8]))
        cases.append((rng.integers(1, 9000, b).tolist(), hkv * int(rng.choice([1, 2, 4, 8])), hkv, int(rng.integers(1, 600))))
    for lens, hq, hkv, nc in cases:
        for dtype in (0, 1):
            c, tile, seg, cta, item = ol.ref_make_plan(dtype, lens, hq, hkv, 128, nc)
            plans.append({"dtype": dtype, "seq_lens": lens, "hq": hq, "hkv": hkv, "num_ctas_in": nc, "tile": tile,
                          "num_ctas": c, "segments": seg.tolist() if len(seg) <= 64 else None,
                          "num_segments": len(seg), "segments_sum": int(seg.astype(np.int64).sum()),
                          "cta_seg_begin": cta.tolist() if len(cta) <= 64 else None,
                          "cta_seg_begin_sum": int(cta.astype(np.int64).sum()),
                          "item_seg_begin": item.tolist()})
    with open(os.path.join(HERE, "planner.json"), "w") as f:
        json.dump({"known_answers": known, "plans": plans}, f)

    # 2. storage conversions: every fp16 bit pattern through the fp8 quantiser at several scales,
    #    every e4m3 byte back to float, fp16 <-> fp32
    allh = np.arange(65536, dtype=np.uint16)
    scales = [1.0, 4.0 / 448.0, 2.0 / 448.0, 0.0123, 3.7]
    q = {f"q_{i}": ol.quantize_e4m3(allh, s, R.ref_quantize_e4m3) for i, s in enumerate(scales)}
    e2f = np.array([R.ref_e4m3_to_float(b) for b in range(256)], np.float32)
    h2f = np.array([R.ref_half_to_float(int(h)) for h in allh], np.float32)
    fs = np.concatenate([np.random.default_rng(5).standard_normal(4096).astype(np.float32) * s
                         for s in (1, 1e-3, 1e-6, 100, 1e4, 7e4)])
    f2h = np.array([R.ref_float_to_half(float(x)) for x in fs], np.uint16)
    np.savez_compressed(os.path.join(HERE, "conversions.npz"), scales=np.array(scales, np.float32), e4m3_to_float=e2f,
                        half_to_float=h2f, f2h_in=fs, f2h_out=f2h, **q)

    # 3. cpu_attention on seeded inputs (uniform(-1,1) like the reference's test helper, and N(0,1))
    att = {}
    rng = np.random.default_rng(11)
    for i, (T, d, dist) in enumerate([(1, 128, "n"), (17, 128, "n"), (64, 128, "u"), (333, 128, "n"), (256, 128, "n"),
                                      (16, 8, "u"), (100, 33, "u")]):
        gen = (lambda s: rng.standard_normal(s).astype(np.float32)) if dist == "n" else \
              (lambda s: rng.uniform(-1, 1, s).astype(np.float32))
        qv, K, V = gen(d), gen((T, d)), gen((T, d))
        att[f"q{i}"], att[f"K{i}"], att[f"V{i}"] = qv, K, V
        att[f"out{i}"] = ol.cpu_attention(qv, K, V, use_ref=True)
    np.savez_compressed(os.path.join(HERE, "cpu_attention.npz"), **att)

    # 4. config 1 of the benchmark spec (inputs are regenerated from their seed by golden_inputs.py;
    #    only their checksum and the reference's outputs are stored)
    from golden_inputs import config1_inputs
    c1 = config1_inputs()
    hq, hkv, d = c1["hq"], c1["hkv"], c1["d"]
    outs = np.zeros((4, hq, d), np.float32)     # cpu_attention on the fp32 inputs
    outs16 = np.zeros((4, hq, d), np.float32)   # same, on the inputs rounded to fp16 (what the cache stores)
    r16 = lambda a: a.astype(np.float16).astype(np.float32)
    for b in range(4):
        for h in range(hq):
            kv = h // (hq // hkv)
            outs[b, h] = ol.cpu_attention(c1["q"][b, h], c1["K"][b][:, kv], c1["V"][b][:, kv], use_ref=True)
            outs16[b, h] = ol.cpu_attention(r16(c1["q"][b, h]), r16(c1["K"][b][:, kv]), r16(c1["V"][b][:, kv]), use_ref=True)
    np.savez_compressed(os.path.join(HERE, "config1.npz"), seq_lens=c1["seq_lens"], block_table=c1["block_table"],
                        out_fp32_inputs=outs, out_fp16_inputs=outs16, inputs_sha256=np.array(c1["sha256"]))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
