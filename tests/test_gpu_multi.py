"""The row-sharded product on two or more GPUs (skipped on a one-GPU machine): one process per GPU,
every exchange variant, the whole C of every rank compared bit for bit with locally computed panel
products. Plain peer stores and NCCL only; NVLS is switched off for the child processes."""
import os
import re
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_peer_sharded_product_on_several_gpus(built_library, world):
    if not torch.cuda.is_available():
        pytest.fail("this test needs CUDA devices")
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this machine has {torch.cuda.device_count()}")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCHDYNAMO_DISABLE="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "peer_sharded_worker.py")]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "FAILED" not in out.stdout, out.stdout[-3000:]
    # the ranks print at the same moment: their lines may run into one another
    assert sorted(int(r) for r in re.findall(r"ok (\d+)", out.stdout)) == list(range(world)), out.stdout[-3000:]
