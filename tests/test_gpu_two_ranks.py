"""Context-sharded decode on two REAL GPUs, one process each: the fused exchange (peer
stores of epoch-tagged words, bounded spin on arrival) runs with both ranks live at the same
time, which the one-GPU tests cannot do. Skipped below two visible devices. No rank is
killed and every wait is bounded."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_sharded_decode_on_two_processes(cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(HERE, "two_rank_child.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-3000:])
    assert "RANK 0 OK" in out.stdout and "RANK 1 OK" in out.stdout
