"""The optional FlashInfer comparison harness (paged_attention_b200/compare_flashinfer.py, the counterpart of
the reference's scripts/compare_flashinfer.py): on a small shape it must run end to end, print the CSV it
documents, and show the engine within the path's tolerance of the fp32 reference the harness computes (the
same check the reference's script reports, scripts/compare_flashinfer.py:113-126,174-177) and of FlashInfer
itself where FlashInfer could be brought up.  FlashInfer is not a dependency: if it cannot be imported the
harness says so and the test is skipped."""
import contextlib
import io
import math

import pytest

pytestmark = pytest.mark.gpu


def test_inputs_follow_the_reference_harness(torch_cuda, pa):
    from paged_attention_b200 import compare_flashinfer as cf
    torch = torch_cuda
    for fp8 in (False, True):
        q, k, v, ks, vs, table = cf.make_inputs(torch, 3, 100, fp8)
        pages = math.ceil(100 / cf.PAGE)
        assert k.shape == (3 * pages, cf.HKV, cf.PAGE, cf.DIM) and table.shape == (3, pages)
        assert sorted(table.flatten().tolist()) == list(range(3 * pages)), "a permutation of the pool's pages"
        assert q.shape == (3, cf.HQ, cf.DIM) and q.dtype == torch.float16
        if fp8:
            assert k.dtype == torch.float8_e4m3fn and 0 < ks < 0.05 and abs(k.float().abs().max().item() - 448.0) < 1e-3
        else:
            assert k.dtype == torch.float16 and ks == 1.0 and vs == 1.0
        ref = cf.fp32_reference(torch, q, k, v, ks, vs, table, 100)
        assert ref.shape == (3, cf.HQ, cf.DIM) and torch.isfinite(ref).all()


def test_harness_runs_and_agrees(torch_cuda, pa):
    from paged_attention_b200 import compare_flashinfer as cf
    out = io.StringIO()
    with contextlib.redirect_stdout(out):
        assert cf.main(["--iters", "3", "--shapes", "4x600,16x2048"]) == 0
    lines = [ln for ln in out.getvalue().splitlines() if ln.strip()]
    if lines and lines[0].startswith("# flashinfer unavailable"):
        pytest.skip(lines[0])
    header = "dtype,batch,seq_len,ours_us,flashinfer_us,flashinfer_tc_us,ratio_fi_over_ours,max_abs_vs_fi,max_abs_vs_fp32"
    assert lines[0] == header
    rows = [dict(zip(header.split(","), ln.split(","))) for ln in lines[1:] if not ln.startswith("#")]
    assert len(rows) == 4, rows                           # two shapes x two cache dtypes
    for r in rows:
        assert float(r["ours_us"]) > 0
        assert float(r["max_abs_vs_fp32"]) <= 2e-3, r     # the engine against the harness's own fp32 reference
        if r["max_abs_vs_fi"] != "nan":
            assert float(r["max_abs_vs_fi"]) <= 2e-3, r   # and against FlashInfer on the same tensors
