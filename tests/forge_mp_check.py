"""Run by tests/test_forge.py in a subprocess: ``fm.launch`` spawns two CPU ranks, each trains the same
model on its own data with ``Forge`` (DDP is applied because a process group exists), and the replicas
must stay bit-identical; rank 0 writes the checkpoint and both ranks restore it."""
import os
import sys
import tempfile

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import forgeminds_b200 as fm  # noqa: E402

PATH = os.path.join(tempfile.gettempdir(), f"forge_mp_{os.getppid()}.pt")


def work():
    import torch.distributed as dist
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == 2
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 1))
    forge = fm.Forge(model, torch.optim.SGD(model.parameters(), lr=0.05), precision="fp32", quiet=True,
                     async_batches=False, accum=2, loss_fn=lambda out, b: nn.functional.mse_loss(out, b[1]),
                     forward_fn=lambda m, b: m(b[0]))
    assert isinstance(forge.model, nn.parallel.DistributedDataParallel)
    gen = torch.Generator().manual_seed(100 + rank)                 # every rank sees different data
    for _ in range(6):
        forge.step((torch.randn(4, 8, generator=gen), torch.randn(4, 1, generator=gen)))
    assert forge.step_count == 3
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    everyone = fm.all_gather(flat.unsqueeze(0))
    assert everyone.shape[0] == 2 and torch.equal(everyone[0], everyone[1]), "replicas diverged"
    forge.save(PATH)                                               # rank 0 writes, both wait
    assert os.path.exists(PATH)
    blob = torch.load(PATH, weights_only=False)
    assert all(not k.startswith("module.") for k in blob["model"])
    for p in model.parameters():
        p.data.zero_()
    forge.load(PATH)
    again = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    assert torch.equal(again, flat)
    mean = fm.all_reduce(torch.tensor([float(rank)]), "sum")
    assert mean.item() == 1.0
    fm.barrier()
    if rank == 0:
        os.remove(PATH)
        print("FORGE_MP_OK", flush=True)


if __name__ == "__main__":
    fm.launch(nproc=2, port=int(sys.argv[1]) if len(sys.argv) > 1 else 29641)(work)()
