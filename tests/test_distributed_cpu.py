"""Runs tests/mp_check.py scenarios under torchrun with the Gloo backend (no GPU needed)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = [29610]


def _run(name, nproc, timeout=420):
    _PORT[0] += 1
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_PORT[0]), os.path.join(HERE, "mp_check.py"), name]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert out.returncode == 0 and f"RESULT {name} ok" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]


@pytest.mark.slow
@pytest.mark.parametrize("name,nproc", [
    ("collectives", 2), ("ddp", 2), ("ddp_accum_offload", 2), ("fsdp", 2), ("fsdp_accum", 2), ("ep_ddp", 2),
    ("pp", 2), ("tp", 2), ("ep_equiv", 2), ("tp_equiv", 2), ("pp_equiv", 2), ("prefetch", 2), ("tp_ckpt", 2), ("flat_ep", 2), ("pp_ckpt", 2),
])
def test_two_ranks(name, nproc):
    _run(name, nproc)


@pytest.mark.slow
@pytest.mark.parametrize("name,nproc", [("hsdp", 4), ("tp_fsdp", 4), ("pp_fsdp", 4), ("flat_pp_dp", 4),
                                        ("3d_full", 8)])
def test_more_ranks(name, nproc):
    _run(name, nproc, timeout=600)
