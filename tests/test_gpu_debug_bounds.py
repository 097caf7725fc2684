"""The bounds-checked build (``_C_debug.so``, ``python -m forgeminds_b200.csrc.build --debug-bounds``).

It stands in for a memory checker: every access of the peer-memory kernels is validated against the table
of registered buffers; an address outside all of them is skipped and reported through the status word.
The tests run in child processes because the library variant is chosen at import time
(``FORGEMINDS_DEBUG_SO=1``). Nothing here faults: the point of the build is that a wrong index does not.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
DEBUG_SO = os.path.join(ROOT, "forgeminds_b200", "_C_debug.so")
needs_debug = pytest.mark.skipif(not os.path.exists(DEBUG_SO), reason="_C_debug.so is not built")

OUT_OF_RANGE = r"""
import sys, torch
sys.path.insert(0, %r)
from forgeminds_b200 import ops
C = ops.require()
assert C.debug_bounds()
dev = torch.device("cuda")
status = ops.status_word(dev)
master = torch.arange(4096, dtype=torch.float32, device=dev)
shadow = torch.zeros(2048, dtype=torch.bfloat16, device=dev)        # room for half of what the table asks for
guard = torch.full((4096,), 7.0, dtype=torch.bfloat16, device=dev)  # what lies behind it must stay untouched
ops.register_buffer(shadow)
off = torch.tensor([0, 2048], dtype=torch.int64, device=dev)
ln = torch.tensor([2048, 2048], dtype=torch.int32, device=dev)
C.comm_push_cast(master, [shadow.data_ptr()], off, ln)             # the second chunk ends past the buffer
torch.cuda.synchronize()
assert status.item() == 7, status.item()
assert torch.equal(shadow.float(), master[:2048].to(torch.bfloat16).float())   # the part in range was written
assert bool((guard == 7).all())
try:
    ops.check_status(dev)
except ops.BoundsError:
    pass
else:
    raise AssertionError("the skipped access was not reported")
assert status.item() == 0
C.comm_push_cast(master, [shadow.data_ptr()], off[:1], ln[:1])    # in range: clean
torch.cuda.synchronize()
assert status.item() == 0
print("BOUNDS_OK")
"""


def _child(code_or_args, env_extra=None, timeout=600):
    env = dict(os.environ, FORGEMINDS_DEBUG_SO="1", NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    env.update(env_extra or {})
    return subprocess.run(code_or_args, env=env, capture_output=True, text=True, timeout=timeout)


@needs_debug
def test_access_outside_the_registered_buffers_is_skipped_and_reported():
    out = _child([sys.executable, "-c", OUT_OF_RANGE % ROOT])
    assert out.returncode == 0 and "BOUNDS_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]


@needs_debug
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("scenario", ["peer_kernels", "gemm_peer", "ep_fused"])
def test_peer_scenarios_stay_inside_their_buffers(scenario):
    """The two-rank kernel scenarios under the checked build: no access leaves the symmetric buffers (each
    scenario ends with ``SymmGroup.check()``, which raises on code 7)."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "mp_gpu_check.py"), scenario]
    out = _child(cmd)
    assert out.returncode == 0 and f"OK {scenario}" in out.stdout, out.stdout[-2000:] + out.stderr[-5000:]
