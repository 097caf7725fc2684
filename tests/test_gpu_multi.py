"""Peer-memory kernels on 2+ GPUs (child processes, one per GPU) and their single-GPU forms."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(scenario: str, nproc: int, port: int, timeout: int = 420):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_gpu_check.py"), scenario]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert out.returncode == 0 and f"OK {scenario}" in out.stdout, out.stdout[-3000:] + out.stderr[-6000:]


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
# number of ranks of the multi-process scenarios: 2, or FMB_TEST_RANKS (4 or 8) when the box has that many GPUs
_ASK = int(os.environ.get("FMB_TEST_RANKS", "2") or 2)
RANKS = _ASK if (_ASK in (4, 8) and torch.cuda.device_count() >= _ASK) else 2


@needs2
def test_peer_kernels_two_ranks():
    _run("peer_kernels", RANKS, 29611)


@needs2
def test_peer_trainer_two_ranks():
    _run("peer_trainer", RANKS, 29612)


@needs2
def test_gemm_with_gathered_operands_and_scattered_output_two_ranks():
    _run("gemm_peer", RANKS, 29613)


@needs2
def test_fused_tensor_parallel_gradients_two_ranks():
    _run("tp_grads", RANKS, 29615)


@needs2
def test_fused_tensor_parallel_two_ranks():
    _run("tp_fused", RANKS, 29614)


@needs2
def test_expert_parallel_over_peer_memory_two_ranks():
    _run("ep_fused", RANKS, 29616)


@needs2
def test_missing_rank_is_reported_not_waited_for_forever():
    _run("peer_failure", RANKS, 29617)


@needs2
def test_every_mesh_matches_the_whole_fp32_model():
    """2 ranks: dp, tp, pp (both schedules); 4: HSDP, tp x dp, pp x dp, pp x tp; 8: pp x dp x tp and HSDP 2 x 4."""
    _run("mesh_equiv", RANKS, 29619, timeout=900)


@needs2
def test_owner_computes_muon_over_peer_memory():
    _run("muon_peer", RANKS, 29620, timeout=600)


@needs2
def test_expert_parallel_trainer_on_the_flat_engine():
    _run("ep_trainer", RANKS, 29621, timeout=600)


@needs2
def test_mesh_and_feature_combinations_train():
    _run("mesh_smoke", RANKS, 29618, timeout=900)


def test_peer_step_single_rank(cuda_status):
    """World of one: the same kernels, peer tables of length one."""
    import forgeminds_b200 as fm
    from forgeminds_b200.parallel.flat import FlatParamStore, _adamw_reference
    from forgeminds_b200.parallel.peer import PeerAdamW, PeerReducer
    from forgeminds_b200.parallel.symm import SymmGroup
    dev = torch.device("cuda")
    torch.manual_seed(0)
    model = fm.GPT(fm.GPTConfig(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=128,
                                ffn_hidden=384)).to(dev)
    sg = SymmGroup(None, dev)
    store = FlatParamStore(model, dev, symm=sg)
    opt = PeerAdamW(store, lr=1e-2, weight_decay=0.1)
    red = PeerReducer(store)
    exp_p, exp_m, exp_v = store.master.clone(), torch.zeros_like(store.master), torch.zeros_like(store.master)
    exp_sh = torch.zeros_like(store.shadow)
    for step in range(2):
        store.grad.copy_(torch.randn(store.total, device=dev))
        g = store.grad.clone()
        red.launch(store.buckets[0])
        red.finish()
        stats = opt.reduce_step(red, torch.tensor(2.5, device=dev), max_norm=1.0, skip_nonfinite=True)
        opt.step()
        norm = g.norm()
        assert abs(stats[0].item() - norm.item()) < 1e-3 * norm.item()
        assert stats[1].item() == 2.5 and stats[2].item() == 1.0
        ctl = torch.stack([torch.clamp(1.0 / (norm + 1e-6), max=1.0), torch.ones((), device=dev)])
        for b in store.buckets:
            for off, n, dec in opt._segments(b):
                lo = b.start + off
                _adamw_reference(exp_p[lo:lo + n], g[lo:lo + n], exp_m[lo:lo + n], exp_v[lo:lo + n], exp_sh[lo:lo + n],
                                 1e-2, 0.9, 0.95, 1e-8, 0.1 if dec else 0.0, 1 - 0.9 ** (step + 1),
                                 1 - 0.95 ** (step + 1), ctl)
        assert (store.master - exp_p).abs().max() < 2e-5
        assert (store.shadow.float() - exp_sh.float()).abs().max() < 1e-3
    # a non-finite gradient leaves everything untouched
    store.grad[5] = float("inf")
    red.finish()
    stats = opt.reduce_step(red, torch.tensor(1.0, device=dev), max_norm=1.0, skip_nonfinite=True)
    before = store.master.clone()
    opt.step()
    assert stats[2].item() == 0.0 and torch.equal(before, store.master)


def test_barrier_wait_runs_out_and_reports(cuda_status):
    """A flag that nobody sets: the wait gives up after its limit and the host sees the code."""
    from forgeminds_b200 import ops
    C = ops.require()
    dev = torch.device("cuda")
    flags = torch.zeros(16, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # a "world" of two whose second rank is this same buffer: rank 1 never signals slot 0
    C.comm_barrier([flags.data_ptr(), flags.data_ptr()], 0, 1, 0, 200.0, status)
    torch.cuda.synchronize()
    assert status.item() == 5            # ERR_WAIT_PEER
    assert flags[0].item() == 1          # this rank's own arrival was recorded
    x = torch.ones(4, device=dev) * 2    # the context is still usable
    assert x.sum().item() == 8.0
