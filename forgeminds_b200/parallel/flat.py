"""Flat parameter store and the fused optimizer that runs on it.

:class:`FlatParamStore` re-homes a model's parameters into three flat device buffers --
fp32 master weights, fp32 gradients ("main grads") and bf16 working weights -- laid out bucket by
bucket in module order (one bucket per transformer block, plus one for everything outside the
blocks). Every ``nn.Parameter`` keeps its name and shape and becomes a view of the master buffer;
its ``.grad`` is a view of the gradient buffer and never goes back to ``None``; its bf16 shadow
(used by the GEMMs) is a view of the working buffer. Because the q|k|v and the gate|up weights of a
block are neighbours in these buffers, the fused projections need no concatenation at all.

What this buys on a B200:

* the weight-gradient GEMMs accumulate straight into the main-grad buffer (no ``grad +=`` pass);
* zeroing gradients is one memset, the global norm one reduction, AdamW one kernel per bucket that
  also refreshes the bf16 weights (no per-forward casts) and takes the clip coefficient and the
  skip flag from device memory (no host round trip);
* data-parallel reduction works on whole buckets: ``all_reduce`` (replicated) or
  ``reduce_scatter`` + sharded update + ``all_gather`` of the bf16 weights (sharded), each bucket on a
  side stream as soon as its block has finished its last backward.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import ops

ALIGN = 256          # elements; keeps every parameter 512-byte aligned in all three buffers


@dataclass
class Bucket:
    name: str
    start: int                  # offset of the bucket in the flat buffers (elements)
    size: int                   # padded size, a multiple of ALIGN * shard world
    params: list = field(default_factory=list)
    decay: list = field(default_factory=list)     # (offset_in_bucket, numel, weight_decay on/off)
    ready: "torch.cuda.Event | None" = None
    local: bool = False         # parameters that only this rank holds (its experts): never reduced over the group,
                                # optimizer state kept whole
    moff: int = 0               # offset of this bucket's part of the optimizer moments (elements)
    msize: int = 0              # its length: size / shard_world, or size for a local bucket


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class DpLayout:
    """Place of this rank in the data-parallel group of its (pipeline stage, tensor-parallel rank).

    The group has ``replicas * shard_world`` ranks, numbered ``replica * shard_world + shard_rank``
    (the mesh order of ``forgemind/distributed.py:146-169``). Gradients are averaged over all of
    them; optimizer state is split over the ``shard_world`` ranks of one replica and repeated in
    every replica (HSDP), so ``replicas == 1`` is plain sharded data parallelism and
    ``shard_world == 1`` plain replication."""
    rank: int = 0
    world: int = 1
    shard_rank: int = 0
    shard_world: int = 1
    shard_group: object = None          # process group of the ranks of this replica (None: the whole group)

    @property
    def replicas(self) -> int:
        return self.world // self.shard_world

    @property
    def replica(self) -> int:
        return self.rank // self.shard_world

    def replica_peers(self) -> range:
        """Group ranks that hold the other shards of this replica (they receive this rank's weights)."""
        lo = self.replica * self.shard_world
        return range(lo, lo + self.shard_world)

    @classmethod
    def of(cls, ctx) -> "DpLayout":
        pc = ctx.pc
        s = max(1, int(pc.dp_shard))
        if ctx.dp_world <= 1:
            return cls()
        if s == 1:                      # pure replication: the optimizer state is still split (ZeRO-1 style)
            return cls(rank=ctx.dp_rank, world=ctx.dp_world, shard_rank=ctx.dp_rank, shard_world=ctx.dp_world,
                       shard_group=ctx.dp_group)
        grp = ctx.dp_group if pc.dp_replicate == 1 else ctx.shard_group
        return cls(rank=ctx.dp_rank, world=ctx.dp_world, shard_rank=ctx.shard_rank, shard_world=s, shard_group=grp)


class FlatParamStore:
    def __init__(self, model, device, shard_world: int = 1, block_attr: str = "layers", symm=None,
                 layout: "DpLayout | None" = None, apart=None):
        """``symm`` (a :class:`~forgeminds_b200.parallel.symm.SymmGroup`) puts the gradient and the bf16
        buffers into symmetric memory so that the peer-memory kernels can read / write them on every
        rank; the buckets are then padded so that they split evenly over the shard ranks of ``layout``
        (default: every rank of the group holds a different shard).

        ``apart(param) -> bool`` moves matching parameters out of their block's bucket into the last
        bucket (``rest``). Tensor parallelism uses it for parameters that are replicated over the
        tensor-parallel ranks (block norms): the ``rest`` bucket then holds exactly the replicated
        part of the model, whose share of the gradient norm is counted once, not once per rank."""
        self.device = torch.device(device)
        self.symm = symm
        if layout is None:
            w = max(1, int(symm.world if symm is not None else shard_world))
            layout = DpLayout(rank=symm.rank if symm is not None else 0, world=w,
                              shard_rank=symm.rank if symm is not None else 0, shard_world=w,
                              shard_group=symm.group if symm is not None else None)
        self.layout = layout
        self.shard_world = layout.shard_world
        groups: list = []
        seen = set()
        blocks = getattr(model, block_attr, None)
        block_list = list(blocks.values()) if hasattr(blocks, "values") else list(blocks or [])
        moved = []
        for i, blk in enumerate(block_list):
            ps = [p for p in blk.parameters() if p.requires_grad and id(p) not in seen]
            for p in ps:
                seen.add(id(p))
            if apart is not None:
                moved += [p for p in ps if apart(p)]
                ps = [p for p in ps if not apart(p)]
            own = [p for p in ps if getattr(p, "_fm_local", False)]       # this rank's experts
            ps = [p for p in ps if not getattr(p, "_fm_local", False)]
            if ps:
                groups.append((f"block{i}", ps, False))
            if own:
                groups.append((f"experts{i}", own, True))
        rest = moved + [p for p in model.parameters() if p.requires_grad and id(p) not in seen]
        if rest:
            groups.append(("rest", rest, False))
        self.buckets: list = []
        cursor = mcursor = 0
        for name, ps, local in groups:
            b = Bucket(name=name, start=cursor, size=0, params=ps, local=local)
            off = 0
            for p in ps:
                b.decay.append((off, p.numel(), p.ndim >= 2))
                off += _round_up(p.numel(), ALIGN)
            b.size = _round_up(off, ALIGN * (1 if local else self.shard_world))
            b.moff, b.msize = mcursor, (b.size if local else b.size // self.shard_world)
            cursor += b.size
            mcursor += b.msize
            self.buckets.append(b)
        self.total = cursor
        self.moment_total = mcursor
        self.reduced = None          # compact buffer of reduced gradient shards (hybrid sharding only, see peer.py)
        self.master = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        if symm is not None:
            self.grad_symm = symm.alloc(self.total, torch.float32)
            self.shadow_symm = symm.alloc(self.total, torch.bfloat16)
            self.grad, self.shadow = self.grad_symm.local, self.shadow_symm.local
        else:
            self.grad = torch.zeros(self.total, dtype=torch.float32, device=self.device)
            self.shadow = torch.zeros(self.total, dtype=torch.bfloat16, device=self.device)
        self.params: list = []
        self._offset: dict = {}
        with torch.no_grad():
            for b in self.buckets:
                for p, (off, n, _) in zip(b.params, b.decay):
                    lo = b.start + off
                    self.master[lo:lo + n].copy_(p.detach().reshape(-1).to(torch.float32))
                    p.data = self.master[lo:lo + n].view(p.shape)
                    g = self.grad[lo:lo + n].view(p.shape)
                    p.grad = g
                    p._fm_main_grad = g
                    p._fm_shadow = (self.shadow[lo:lo + n].view(p.shape), p._version)
                    self._offset[p] = lo
                    self.params.append(p)
            self.refresh_shadow()
        self._scratch = torch.empty(1024, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ views
    def bucket_view(self, buf: torch.Tensor, b: Bucket) -> torch.Tensor:
        return buf[b.start:b.start + b.size]

    def refresh_shadow(self) -> None:
        """bf16 working weights <- fp32 masters (after a load_state_dict or any external edit)."""
        if self.device.type == "cuda" and ops.available():
            ops.require().scale_cast(self.master, self.shadow, 1.0)
        else:
            self.shadow.copy_(self.master)
        for p in self.params:
            p._fm_shadow = (p._fm_shadow[0], p._version)

    def shard_range(self, b: Bucket, rank: int):
        """(flat offset, length) of ``rank``'s part of bucket ``b`` (all of it for a local bucket)."""
        if b.local:
            return b.start, b.size
        n = b.size // self.shard_world
        return b.start + rank * n, n

    def sync_master(self) -> None:
        """Make the fp32 masters whole again on every rank. With a sharded optimizer each rank only
        updates its own part of every bucket (the bf16 working weights are complete everywhere); call
        this before reading parameters as fp32: checkpoints, ``state_dict``, evaluation on the
        PyTorch path."""
        lay = self.layout
        if self.symm is None or lay.shard_world == 1:
            return
        for b in self.buckets:
            if b.local:
                continue
            lo, n = self.shard_range(b, lay.shard_rank)
            whole = self.bucket_view(self.master, b)
            if all(self.shard_range(b, r)[1] == n for r in range(lay.shard_world)):
                dist.all_gather_into_tensor(whole, self.master[lo:lo + n].clone(), group=lay.shard_group)
            else:                      # shards of unequal length (cut along parameter boundaries): sum of disjoint parts
                mine = self.master[lo:lo + n].clone()
                whole.zero_()
                self.master[lo:lo + n].copy_(mine)
                dist.all_reduce(whole, group=lay.shard_group)

    def reduced_shard(self, b: Bucket, rank: int) -> torch.Tensor:
        """This rank's reduced gradients of bucket ``b`` after the reduce-scatter: a slice of the gradient
        buffer itself, or of the compact buffer when replicas share shards (hybrid sharding)."""
        lo, n = self.shard_range(b, rank)
        if self.reduced is not None and not b.local:
            return self.reduced[b.moff:b.moff + n]
        return self.grad[lo:lo + n]

    def rebind(self) -> None:
        """Re-attach ``.grad`` views (something set them to ``None``)."""
        for p in self.params:
            if p.grad is None or p.grad.data_ptr() != p._fm_main_grad.data_ptr():
                p.grad = p._fm_main_grad

    def zero_grad(self) -> None:
        self.grad.zero_()
        self.rebind()

    def grad_sq_norm(self, out: torch.Tensor, view: "torch.Tensor | None" = None) -> torch.Tensor:
        """``out[0] = sum(grad^2)`` over the whole buffer (or ``view``), on the device."""
        g = self.grad if view is None else view
        if self.device.type == "cuda" and ops.available():
            ops.require().sqnorm(g, self._scratch, out, False)
        else:
            out.copy_(g.float().square().sum().reshape(1))
        return out


class FlatAdamW(torch.optim.Optimizer):
    """AdamW over a :class:`FlatParamStore`: one fused kernel per (bucket, decay class).

    ``ctl`` is a 2-float device tensor ``[clip coefficient, apply flag]`` read by the kernel, so the
    global-norm clipping and the unanimous skip decision never need the host. Weight decay is applied
    to parameters with ``ndim >= 2`` only (``forgemind/trainer.py:103-107``). The per-parameter state
    (``exp_avg``, ``exp_avg_sq``, ``step``) is exposed as views, so ``state_dict()`` has the layout of
    ``torch.optim.AdamW``.
    """

    def __init__(self, store: FlatParamStore, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 shard_rank: int = 0, shard_world: int = 1):
        self.store = store
        decay = [p for p in store.params if p.ndim >= 2]
        rest = [p for p in store.params if p.ndim < 2]
        groups = [g for g in ({"params": decay, "weight_decay": weight_decay},
                              {"params": rest, "weight_decay": 0.0}) if g["params"]]
        super().__init__(groups, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.shard_rank, self.shard_world = shard_rank, shard_world
        n = store.moment_total if shard_world > 1 else store.total
        dev = store.device
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.ctl = torch.tensor([1.0, 1.0], dtype=torch.float32, device=dev)
        self.steps = 0
        self._step_t = torch.zeros((), dtype=torch.float32)
        if shard_world == 1:
            for p in store.params:
                lo = store._offset[p]
                self.state[p] = {"step": self._step_t,
                                 "exp_avg": self.exp_avg[lo:lo + p.numel()].view(p.shape),
                                 "exp_avg_sq": self.exp_avg_sq[lo:lo + p.numel()].view(p.shape)}

    def _segments(self, b: Bucket):
        """Runs of equal weight-decay class inside a bucket: (offset, length, decay?)."""
        runs = []
        for off, n, dec in b.decay:
            padded = _round_up(n, ALIGN)
            if runs and runs[-1][2] == dec and runs[-1][0] + runs[-1][1] == off:
                runs[-1] = (runs[-1][0], runs[-1][1] + padded, dec)
            else:
                runs.append((off, padded, dec))
        return runs

    @torch.no_grad()
    def step(self, closure=None):
        st = self.store
        self.steps += 1
        self._step_t.fill_(self.steps)
        lr = self.param_groups[0]["lr"]
        b1, b2 = self.defaults["betas"]
        eps = self.defaults["eps"]
        wd = max(float(g["weight_decay"]) for g in self.param_groups)
        bc1, bc2 = 1 - b1 ** self.steps, 1 - b2 ** self.steps
        native = st.device.type == "cuda" and ops.available()
        C = ops.require() if native else None
        for b in st.buckets:
            for off, n, dec in self._segments(b):
                lo = b.start + off
                p, g = st.master[lo:lo + n], st.grad[lo:lo + n]
                m, v = self.exp_avg[lo:lo + n], self.exp_avg_sq[lo:lo + n]
                sh = st.shadow[lo:lo + n]
                w = wd if dec else 0.0
                if native:
                    C.adamw_flat(p, g, m, v, sh, lr, b1, b2, eps, w, bc1, bc2, self.ctl)
                else:
                    _adamw_reference(p, g, m, v, sh, lr, b1, b2, eps, w, bc1, bc2, self.ctl)
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.store.zero_grad()

    def load_state_dict(self, state_dict) -> None:
        """Loads like ``torch.optim.AdamW`` and then moves the moments back into the flat buffers
        (``Optimizer.load_state_dict`` replaces the state tensors by copies)."""
        super().load_state_dict(state_dict)
        if self.shard_world != 1:
            return
        steps = 0
        with torch.no_grad():
            for p in self.store.params:
                st = self.state.get(p)
                if not st:
                    continue
                lo, n = self.store._offset[p], p.numel()
                for key, flat in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                    view = flat[lo:lo + n].view(p.shape)
                    if key in st and st[key].data_ptr() != view.data_ptr():
                        view.copy_(st[key])
                    st[key] = view
                if "step" in st:
                    steps = max(steps, int(float(st["step"])))
                st["step"] = self._step_t
        self.steps = steps
        self._step_t.fill_(steps)


def _adamw_reference(p, g, m, v, shadow, lr, b1, b2, eps, wd, bc1, bc2, ctl):
    """PyTorch statement of the fused kernel (CPU path and test oracle)."""
    clip, ok = ctl[0], ctl[1]
    if float(ok) < 0.5:
        return
    gg = g * clip
    m.lerp_(gg, 1 - b1)
    v.mul_(b2).addcmul_(gg, gg, value=1 - b2)
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p.mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
    shadow.copy_(p)


class BucketReducer:
    """Averages gradient buckets over the data-parallel group on a side stream.

    ``launch(bucket)`` is called when a block has finished its last backward of the step (module
    backward hook): the reduction of that bucket then overlaps the backward of the earlier blocks.
    ``finish()`` makes the compute stream wait for all of them. Uses NCCL/Gloo ``all_reduce``. Inside
    one NVSwitch domain the trainer uses :class:`forgeminds_b200.parallel.peer.PeerReducer` (same
    interface, pull reduce-scatter over symmetric memory) instead; this class serves larger groups,
    CPU runs and ``fused_comm=False``.
    """

    def __init__(self, store: FlatParamStore, group, world: int, local_group=None):
        """``local_group``: ranks that hold replicas of this rank's local buckets (the same expert shard in
        other expert-parallel groups), or ``None`` when there are none."""
        self.store, self.group, self.world = store, group, world
        self.local_group = local_group
        self.cuda = store.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=store.device) if self.cuda else None
        self._launched: list = []
        self.enabled = True

    def _finish_local(self, b: Bucket) -> None:
        """A bucket that only this rank (and its replicas) holds already sums the tokens of every rank that
        routed to it: add the replicas, then scale like every other gradient (mean over the group)."""
        view = self.store.bucket_view(self.store.grad, b)
        if self.local_group is not None and dist.get_world_size(self.local_group) > 1:
            dist.all_reduce(view, group=self.local_group)
        view.div_(self.world)

    def launch(self, b: Bucket) -> None:
        if not self.enabled or self.world <= 1:
            return
        if b.local:
            self._finish_local(b)
            self._launched.append(b.name)
            return
        view = self.store.bucket_view(self.store.grad, b)
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                dist.all_reduce(view, op=dist.ReduceOp.AVG, group=self.group)
        else:
            dist.all_reduce(view, group=self.group)
            view.div_(self.world)
        self._launched.append(b.name)

    def finish(self) -> None:
        if self.cuda and self._launched:
            torch.cuda.current_stream().wait_stream(self.stream)
        done = set(self._launched)
        self._launched.clear()
        if self.enabled and self.world > 1:
            for b in self.store.buckets:         # anything whose hook did not fire (unused parameters)
                if b.name not in done and b.local:
                    self._finish_local(b)
                elif b.name not in done:
                    view = self.store.bucket_view(self.store.grad, b)
                    if self.cuda:
                        dist.all_reduce(view, op=dist.ReduceOp.AVG, group=self.group)
                    else:
                        dist.all_reduce(view, group=self.group)
                        view.div_(self.world)
