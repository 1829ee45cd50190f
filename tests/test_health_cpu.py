"""Failure detection on the host (gloo ranks on CPU, no GPU involved)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_peers_notice_a_missing_rank_before_the_next_step(mode):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29731" if mode == "leave" else "29732", os.path.join(HERE, "_health_worker.py"), mode]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    out = r.stdout + r.stderr
    assert out.count("HEALTH_OK") == 2 and "HEALTH_FAIL" not in out, out[-3000:]
