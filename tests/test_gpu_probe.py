"""The awkward-shape probe (``python -m forgeminds_b200.cli probe``) on the real kernels: every case matches its
PyTorch statement and the device status word stays clear."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_probe_passes_on_the_device():
    from forgeminds_b200 import kernels as K
    from forgeminds_b200.cli import probe
    K.reset_stats()
    rows = probe.run(torch.device("cuda"), torch.bfloat16)
    bad = [r for r in rows if not r["ok"]]
    assert not bad, bad
    assert len(rows) >= 16                                   # the tensor-core cases ran too
    assert K.stats()["fast"] > 0                             # the kernels, not the fallbacks, were probed
