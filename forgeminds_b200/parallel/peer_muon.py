"""Muon over peer memory: every matrix has one owner rank that orthogonalises it.

Newton-Schulz needs whole matrices, so the even split of a gradient bucket that the sharded AdamW uses
does not work for Muon. Here every block's bucket is cut along parameter boundaries into one contiguous
run of whole parameters per shard rank (balanced by size). The step is then the peer-memory step of
:mod:`forgeminds_b200.parallel.peer` with those runs as the shards:

1. the pull reduce-scatter of a bucket sums, on each rank, the run that the rank owns;
2. the scalar exchange produces the global norm, the clip coefficient and the apply flag on the device;
3. the owner updates what it owns -- Muon (momentum, Nesterov blend, batched Newton-Schulz on the
   tcgen05 GEMM, ``sqrt(max(1, rows/cols))`` scale, decoupled weight decay) for the matrices, the fused
   AdamW kernel for the vectors in its run and for its even share of the non-block parameters -- and the
   new weights go to every rank's bf16 working copy (``adamw_push_kernel`` / ``push_cast_kernel``).

Momentum buffers exist only on the owner (optimizer state is 1/S per rank, like the sharded AdamW). The
clip coefficient and the apply flag are read on the device, so the step is enqueued before the host has
seen the norm. The reference's Muon is replicated: every rank keeps every momentum buffer, the
Newton-Schulz work is split ``rank::world`` and recombined with an all-reduce
(``forgemind/muon.py:203-255``); its trainer cannot select Muon at all (``forgemind/trainer.py:113-124``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from .flat import ALIGN, Bucket, FlatParamStore, _round_up
from .peer import PeerAdamW


def split_whole_params(sizes: list, parts: int) -> list:
    """Cut ``sizes`` (padded parameter lengths, in order) into ``parts`` contiguous runs of whole
    parameters with sums as even as a left-to-right greedy cut gets them. Returns the index where each
    run starts, plus the end: ``parts + 1`` non-decreasing numbers."""
    total = sum(sizes)
    cuts, acc, i = [0], 0, 0
    for k in range(1, parts):
        goal = total * k / parts
        while i < len(sizes) and acc + sizes[i] / 2 <= goal:
            acc += sizes[i]
            i += 1
        cuts.append(i)
    cuts.append(len(sizes))
    return cuts


class PeerMuon(PeerAdamW):
    def __init__(self, store: FlatParamStore, model, tc, scalars=None):
        lay = store.layout
        # ownership has to exist before the base class sizes the moments: a Muon bucket's share of the
        # moment buffers is the longest run of any rank (the layout must not depend on the rank)
        self.muon_lr, self.mu, self.ns_steps = float(tc.muon_lr), float(tc.muon_momentum), int(tc.muon_ns_steps)
        self.base_lr = float(tc.lr)
        names = {id(p): n for n, p in model.named_parameters()}
        self._is_matrix = {id(p): (p.ndim >= 2 and ".layers." in f".{names.get(id(p), '')}") for p in store.params}
        self.runs: dict = {}                       # bucket name -> [(lo, n)] per shard rank
        mcursor = 0
        for b in store.buckets:
            if b.local or not b.name.startswith("block"):
                b.moff, b.msize = mcursor, (b.size if b.local else b.size // lay.shard_world)
            else:
                sizes = [_round_up(n, ALIGN) for _, n, _ in b.decay]
                cuts = split_whole_params(sizes, lay.shard_world)
                starts = [sum(sizes[:c]) for c in cuts]
                self.runs[b.name] = [(b.start + starts[r], starts[r + 1] - starts[r]) for r in range(lay.shard_world)]
                b.moff, b.msize = mcursor, max(n for _, n in self.runs[b.name])
            mcursor += b.msize
        store.moment_total = mcursor
        store.shard_range = self._shard_range          # the reducer asks the store
        super().__init__(store, lr=tc.lr, betas=tc.betas, eps=tc.eps, weight_decay=tc.weight_decay, scalars=scalars)
        self.weight_decay = float(tc.weight_decay)
        self._mine = self._owned_matrices()
        self._push = None

    # ------------------------------------------------------------------ ownership
    def _shard_range(self, b: Bucket, rank: int):
        runs = self.runs.get(b.name)
        if runs is not None:
            return runs[rank]
        return FlatParamStore.shard_range(self.store, b, rank)

    def _owned_matrices(self) -> list:
        """(parameter, flat offset, offset in the moment buffers) of the matrices this rank orthogonalises."""
        st, r = self.store, self.layout.shard_rank
        out = []
        for b in st.buckets:
            runs = self.runs.get(b.name)
            if runs is None:
                continue
            lo, n = runs[r]
            for p in b.params:
                off = st._offset[p]
                if self._is_matrix[id(p)] and lo <= off < lo + n:
                    out.append((p, off, b.moff + off - lo))
        return out

    def _segments(self, b: Bucket):
        """Runs of equal weight-decay class for the fused AdamW kernel; matrices that Muon updates are left out."""
        segs = []
        for (off, n, _dec), p in zip(b.decay, b.params):
            if b.name in self.runs and self._is_matrix[id(p)]:
                continue
            # no weight decay outside the Muon group (as in the replicated form, Trainer._muon)
            if segs and segs[-1][0] + segs[-1][1] == off:
                segs[-1] = (segs[-1][0], segs[-1][1] + _round_up(n, ALIGN), False)
            else:
                segs.append((off, _round_up(n, ALIGN), False))
        return segs

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, closure=None):
        st, sg = self.store, self.sg
        lr = self.param_groups[0]["lr"]
        shape = lr / self.base_lr if self.base_lr else 1.0
        self._muon_update(self.muon_lr * shape)
        return super().step()                    # AdamW shares, their pushes and the closing barrier

    def _muon_update(self, lr: float) -> None:
        from ..kernels import newton_schulz
        st = self.store
        clip, go = self.ctl[0], self.ctl[1] > 0.5
        by_shape: dict = {}
        for item in self._mine:
            p = item[0]
            by_shape.setdefault((p.shape[0], p.numel() // p.shape[0]), []).append(item)
        for (rows, cols), items in by_shape.items():
            stack = []
            for p, off, moff in items:
                n = p.numel()
                src = st.reduced[moff:moff + n] if st.reduced is not None else st.grad[off:off + n]
                g = src * clip
                buf = self.exp_avg[moff:moff + n]
                buf.copy_(torch.where(go, buf.lerp(g, 1 - self.mu), buf))
                stack.append(g.lerp(buf, self.mu).view(rows, cols))
            ortho = newton_schulz(torch.stack(stack), steps=self.ns_steps, dtype=torch.bfloat16)
            gain = max(1.0, rows / cols) ** 0.5
            for i, (p, off, moff) in enumerate(items):
                w = st.master[off:off + p.numel()]
                moved = w * (1 - lr * self.weight_decay) - ortho[i].reshape(-1).to(torch.float32) * (lr * gain)
                w.copy_(torch.where(go, moved, w))
        if self._mine:
            if self._push is None:
                chunk = int(ops.require().comm_adam_chunk())
                offs, lens = [], []
                for p, off, _ in self._mine:
                    n = _round_up(p.numel(), 8)
                    for a in range(0, n, chunk):
                        offs.append(off + a)
                        lens.append(min(chunk, n - a))
                self._push = (torch.tensor(offs, dtype=torch.int64, device=st.device),
                              torch.tensor(lens, dtype=torch.int32, device=st.device))
            ptrs = st.shadow_symm.ptrs
            if self.local_only:
                ptrs = [ptrs[self.sg.rank]]
            elif self.layout.replicas > 1:
                ptrs = [ptrs[r] for r in self.layout.replica_peers()]
            ops.require().comm_push_cast(st.master, ptrs, *self._push)

    # ------------------------------------------------------------------ checkpoints
    def gather_full(self) -> None:
        """Expose the whole state per parameter: ``momentum_buffer`` for Muon's matrices, the AdamW entries
        for everything else. Every rank fills in what it owns; one sum over the shard group completes it."""
        st, lay = self.store, self.layout
        full_m = torch.zeros(st.total, dtype=torch.float32, device=st.device)
        full_v = torch.zeros(st.total, dtype=torch.float32, device=st.device)
        for b in st.buckets:
            lo, n = st.shard_range(b, lay.shard_rank)
            full_m[lo:lo + n] = self.exp_avg[b.moff:b.moff + n]
            full_v[lo:lo + n] = self.exp_avg_sq[b.moff:b.moff + n]
        if lay.shard_world > 1:
            local = [b for b in st.buckets if b.local]
            keep = [(st.bucket_view(full_m, b).clone(), st.bucket_view(full_v, b).clone()) for b in local]
            dist.all_reduce(full_m, group=lay.shard_group)
            dist.all_reduce(full_v, group=lay.shard_group)
            for b, (m, v) in zip(local, keep):         # a rank's own experts are not shared
                st.bucket_view(full_m, b).copy_(m)
                st.bucket_view(full_v, b).copy_(v)
        self._full = (full_m, full_v)
        for p in st.params:
            lo, n = st._offset[p], p.numel()
            if self._is_matrix[id(p)]:
                self.state[p] = {"momentum_buffer": full_m[lo:lo + n].view(p.shape)}
            else:
                self.state[p] = {"step": self._step_t, "exp_avg": full_m[lo:lo + n].view(p.shape),
                                 "exp_avg_sq": full_v[lo:lo + n].view(p.shape)}

    def scatter_full(self) -> None:
        if self._full is None:
            return
        st, lay = self.store, self.layout
        full_m, full_v = self._full
        steps = 0
        for p in st.params:                      # load_state_dict replaced the views by copies
            state = self.state.get(p)
            if not state:
                continue
            lo, n = st._offset[p], p.numel()
            pairs = (("momentum_buffer", full_m),) if self._is_matrix[id(p)] else \
                (("exp_avg", full_m), ("exp_avg_sq", full_v))
            for key, flat in pairs:
                view = flat[lo:lo + n].view(p.shape)
                if key in state and state[key].data_ptr() != view.data_ptr():
                    view.copy_(state[key])
            if "step" in state:
                steps = max(steps, int(float(state["step"])))
        for b in st.buckets:
            lo, n = st.shard_range(b, lay.shard_rank)
            self.exp_avg[b.moff:b.moff + n].copy_(full_m[lo:lo + n])
            self.exp_avg_sq[b.moff:b.moff + n].copy_(full_v[lo:lo + n])
        self.steps = steps
        self._step_t.fill_(steps)
        self.release_full()

    def load_state_dict(self, state_dict) -> None:
        if self._full is None:
            self.gather_full()
        torch.optim.Optimizer.load_state_dict(self, state_dict)
        self.scatter_full()
