"""bench.py's reference arm runs without a GPU: check that it prints one JSON line with the agreed keys
and that the byte model matches the figures stated for the headline configurations."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_algorithmic_bytes_of_the_headline_configs():
    sys.path.insert(0, ROOT)
    import bench
    # 2*sum(len)*Hkv*d*elem + 2*B*Hq*d*2 + 4*sum(ceil(len/page))
    assert bench.algorithmic_bytes(0, [8192] * 64, 32, 8, 16) == 2147483648 + 1048576 + 131072 == 2148663296
    assert bench.algorithmic_bytes(1, [4096] * 128, 32, 8, 16) == 1073741824 + 2097152 + 131072 == 1075970048
    assert bench.algorithmic_bytes(1, [16384] * 256, 64, 8, 16) == 8589934592 + 8388608 + 1048576


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "small",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    for key in ("metric", "value", "n_gpus", "steps", "warmup", "ms_per_step", "config", "cpu_baseline", "e2e"):
        assert key in d
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["value"] > 0


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--workload",
                        "small", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
