"""All ranks learn of a failure that one rank saw (gloo ranks on CPU)."""
import os
import subprocess
import sys

import pytest

from tileccl_b200.bench import _common as C

HERE = os.path.dirname(os.path.abspath(__file__))


def test_single_process_check():
    C.agree_no_failure(lambda: None)
    with pytest.raises(RuntimeError, match="rank 0: KeyError"):
        C.agree_no_failure(lambda: {}["x"], "warm-up")


def test_every_rank_raises_when_one_check_fails():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(HERE, "_agree_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    out = r.stdout + r.stderr
    assert r.returncode == 0 and out.count("AGREE_OK") == 3 and out.count("AGREE_CLEAN") == 3, out[-3000:]
    assert "AGREE_MISSED" not in out and "AGREE_BAD" not in out
