"""bench.py contract pieces that need no GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and "unavailable" in d and "\n" not in d["unavailable"]


def test_run_all_lists_every_experiment():
    r = subprocess.run([sys.executable, "-m", "tileccl_b200.bench.run_all", "--list", "--quick"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0
    for name in ("exp3_fused_m32768", "exp3_fused_native", "exp3_fused_nvls", "exp2_ag_gemm", "exp1_ce_interference", "nvls_bw", "peer_l2_probe", "signal_fanin"):
        assert name in r.stdout
