"""Seeded random shapes against the oracle: kv-head counts, GQA groups, page sizes (also odd ones),
ragged lengths, forced CTA counts, both cache types, both schedules where the layer has 8 kv heads,
chunked appends.  Every case checks block tables, cache bytes (bit-exact) and outputs (tolerance), as
run_case does."""
import numpy as np
import pytest

from common import TOL, Case, run_case

pytestmark = pytest.mark.gpu


def _cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        hkv = int(rng.choice([1, 2, 4, 8, 8, 8]))
        group = int(rng.choice([1, 2, 4, 8]))
        ps = int(rng.choice([1, 2, 3, 8, 16, 16, 16, 24, 32, 64, 100]))
        batch = int(rng.integers(1, 40))
        top = int(rng.choice([40, 700, 6000]))
        lens = rng.integers(1, top + 1, batch).tolist()
        ctas = int(rng.choice([0, 0, 1, 3, 17, 90, 300, 700]))
        chunk = int(rng.choice([0, 0, 1, 37])) if sum(lens) < 3000 else 0
        out.append((int(rng.integers(0, 2)), hkv * group, hkv, ps, lens, ctas, chunk, int(rng.integers(0, 1 << 16))))
    return out


@pytest.mark.parametrize("index,spec", list(enumerate(_cases(20260, 36))))
def test_random_shapes_against_the_oracle(index, spec, torch_cuda, pa):
    dtype, hq, hkv, ps, lens, ctas, chunk, seed = spec
    before = pa.head_fused()
    try:
        for mode in ((2, 0) if hkv == 8 else (1,)):
            pa.set_head_fused(mode)
            case = Case(dtype, hq, hkv, ps, lens, num_ctas=ctas, chunk=chunk, seed=seed, shuffle=seed % 97)
            err, out, want, info = run_case(case, torch_cuda, pa)
            assert err <= TOL, (spec, mode, err)
    finally:
        pa.set_head_fused(before)
