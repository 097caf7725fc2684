"""Run by tests/test_muon.py in a subprocess under torchrun (2 CPU ranks, Gloo): Muon with the
Newton-Schulz work split over the ranks gives bit-identical replicas and the same parameters as a
single-process run on the averaged gradients."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import forgeminds_b200 as fm  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    def build():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 32), nn.Tanh(), nn.Linear(32, 4))
    model, solo = build(), build()
    opt = fm.Muon(model.parameters(), lr=0.02, weight_decay=0.01, ns_dtype=torch.float32, adam_lr=1e-3)
    ref = fm.Muon(solo.parameters(), lr=0.02, weight_decay=0.01, ns_dtype=torch.float32, adam_lr=1e-3, group=None)
    ref._dist_group = "solo"
    x_all = torch.randn(3, world, 8, 16, generator=torch.Generator().manual_seed(5))
    y_all = torch.randn(3, world, 8, 4, generator=torch.Generator().manual_seed(6))
    for step in range(3):
        opt.zero_grad()
        nn.functional.mse_loss(model(x_all[step, rank]), y_all[step, rank]).backward()
        for p in model.parameters():                       # data-parallel average, as DDP would leave it
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step()
        # the single-process twin: whole batch, no process group
        ref.zero_grad()
        (sum(nn.functional.mse_loss(solo(x_all[step, r]), y_all[step, r]) for r in range(world)) / world).backward()
        _solo_step(ref)
    for p, q in zip(model.parameters(), solo.parameters()):
        assert torch.allclose(p, q, atol=1e-5), (p - q).abs().max()
        mine = p.detach().clone()
        dist.broadcast(mine, src=0)
        assert torch.equal(mine, p.detach()), "replicas diverged"
    dist.barrier()
    if rank == 0:
        print("MUON_MP_OK", flush=True)
    dist.destroy_process_group()


def _solo_step(opt):
    """Step ``opt`` as if no process group existed (every matrix orthogonalised here)."""
    real_init, real_size = dist.is_initialized, dist.get_world_size
    dist.is_initialized = lambda: False
    try:
        opt.step()
    finally:
        dist.is_initialized, dist.get_world_size = real_init, real_size


if __name__ == "__main__":
    main()
