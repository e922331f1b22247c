"""The KV-split decode on real GPUs: one process a GPU under torch.distributed.run, partials pushed over NVLink into
IPC-opened mailboxes, every rank's combined rows against the CPU oracle and against the other ranks' (tests/kvsplit_worker.py).
Needs at least two GPUs; on a one-GPU box the same kernels are exercised by tests/test_kvsplit.py with all ranks on one GPU."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count():
    from nextsycl_b200 import api
    try:
        return int(api.load().ns_gpu_count())
    except Exception:
        return 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_agree_with_the_oracle(world):
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "kvsplit_worker.py")], cwd=ROOT, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:]
    assert "kvsplit multi-gpu: ok" in r.stdout
