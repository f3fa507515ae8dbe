"""The two exchange steps (all-gather of decode partials, all-gather of the latent rows for a
context-parallel prefill) over real NCCL: one process per GPU through torch.distributed.run.
Needs at least two GPUs in the box; on a one-GPU box the same host logic is covered by the gloo
tests and the kernels by the single-process tests that run the ranks one after another."""
import os
import socket
import subprocess
import sys

import pytest
import torch


@pytest.mark.gpu
def test_exchange_steps_over_nccl(cuda):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("one GPU in this box")
    world = 4 if n >= 4 else 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(here, "nccl_rank.py")]
    # one of the cases keeps a rank away from a step of the peer exchange (nobody exits, nothing is killed); in-switch
    # reduction is switched off for the run all the same, so that no rank's memory is bound to a multicast object
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert out.stdout.count("exchange checks passed") == world
