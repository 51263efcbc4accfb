"""The expert-parallel layer on two (or more) GPUs, one process per GPU: the peer-memory exchange gives the all-to-all
form's results bit for bit and the plain layer's within 1e-5.  Skipped on a single GPU (kernels of different ranks
wait on one another, so every rank needs its own GPU)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_p2p_exchange_across_gpus():
    import torch
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(here, "ep_p2p_worker.py")],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "EP_P2P_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
