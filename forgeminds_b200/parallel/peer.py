"""Data-parallel training step over peer memory: no NCCL call between backward and the next forward.

With ``W`` ranks on one NVSwitch domain the step after the last backward is three kinds of kernel
(``csrc/comm.cu``), all working on the symmetric buffers of a :class:`FlatParamStore`:

1. per gradient bucket, on a side stream as soon as its block has finished backward:
   **reduce-scatter by pulling** -- each rank sums ITS 1/W of the bucket over all ranks' buffers
   with plain peer loads, scales, writes the result in place and leaves per-block sums of squares;
2. once per step, one CTA: sum the partials, exchange ``{sum of squares, loss}`` with the peers and
   leave the global norm, the mean loss, the "all finite" flag and the clip coefficient in device
   memory -- this replaces the norm all-reduce, the loss all-reduce and the unanimous-skip
   all-reduce of the reference step (``forgemind/trainer.py:213-250,299,329``);
3. **AdamW on the shard + all-gather by pushing**: one kernel updates this rank's fp32 masters and
   moments (1/W of the optimizer state lives on each rank) and stores the bf16 result straight into
   every rank's working weights; a flag barrier then tells everybody that all pushes have landed.

Weights stay resident in bf16 on every GPU (a 354 M-parameter model is 0.7 GB of 180 GB), so the
forward needs no all-gather at all; the reference's FSDP2 gathers every block's parameters before
its forward and again before its backward (``forgemind/parallel/native.py:52-68``).

Hybrid sharding (``dp_replicate x dp_shard``, the reference's 2-D ``fully_shard`` mesh,
``forgemind/parallel/native.py:54-57``) uses the same three kernels on the whole data-parallel group:
rank ``(r, s)`` pulls shard ``s`` of every bucket from all ``R * S`` buffers (reduce-scatter inside
the shard group and the sum over the replicas are one pass, fixed rank order), keeps the moments of
shard ``s`` only, and pushes the new bf16 weights to the ``S`` ranks of its own replica.

With pipeline or tensor parallelism every (stage, tensor rank) coordinate runs this over its own
data-parallel group; the end-of-step scalars are exchanged over a second, world-wide group so that
the norm covers the whole model (see :class:`PeerAdamW.reduce_step`).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from .flat import ALIGN, Bucket, FlatAdamW, FlatParamStore, _round_up

BLOCKS_PER_BUCKET = 296          # grid of one bucket's pull-reduce (also its number of partial sums)


class PeerReducer:
    """Drop-in for :class:`BucketReducer` that runs step 1 above."""

    def __init__(self, store: FlatParamStore, local_group=None):
        """``local_group``: ranks holding replicas of this rank's local buckets (same experts, other
        expert-parallel group); their gradients are summed with one ``all_reduce`` per bucket."""
        if store.symm is None:
            raise ValueError("PeerReducer needs a FlatParamStore built on a SymmGroup")
        self.local_group = local_group
        self.store, self.sg = store, store.symm
        self.world = self.sg.world
        self.layout = store.layout
        self.stream = torch.cuda.Stream(device=store.device, priority=-1)
        self.partials = torch.zeros(len(store.buckets) * BLOCKS_PER_BUCKET, dtype=torch.float32, device=store.device)
        self.slot0 = self.sg.reserve_slots(len(store.buckets))
        self._index = {b.name: i for i, b in enumerate(store.buckets)}
        self._launched: list = []
        self.enabled = True
        self.local_only = False      # timing diagnostics: same kernels, this rank's memory only (see detach)
        # Hybrid sharding: the replicas of a shard all read that shard from every rank, so none of them may
        # overwrite it. Their sums go to a compact buffer laid out like the optimizer moments instead.
        if self.layout.replicas > 1 and getattr(store, "reduced", None) is None:
            store.reduced = torch.zeros(store.moment_total, dtype=torch.float32, device=store.device)
            ops.register_buffer(store.reduced)

    def _reduce(self, b: Bucket) -> None:
        C = ops.require()
        st, sg = self.store, self.sg
        i = self._index[b.name]
        lo, n = st.shard_range(b, self.layout.shard_rank)
        part = self.partials[i * BLOCKS_PER_BUCKET:(i + 1) * BLOCKS_PER_BUCKET]
        slot = self.slot0 + i
        if b.local and self.local_group is not None and dist.get_world_size(self.local_group) > 1:
            dist.all_reduce(st.bucket_view(st.grad, b), group=self.local_group)
        if self.local_only or b.local:
            # this rank's memory only: scale, sum of squares (a local bucket holds the rank's own experts,
            # whose gradient already covers the tokens of every rank that routed to them)
            C.comm_rs_reduce([st.grad_symm.ptrs[sg.rank]], lo, n, 1.0 / self.world, part, [sg.flags.ptrs[sg.rank]], slot,
                             sg.next_epoch(slot), 0, sg.timeout_ms, sg.status)
            return
        dst = None
        if getattr(st, "reduced", None) is not None:
            dst = st.reduced[b.moff:b.moff + n]
        C.comm_rs_reduce(st.grad_symm.ptrs, lo, n, 1.0 / self.world, part, sg.flags.ptrs, slot, sg.next_epoch(slot),
                         sg.rank, sg.timeout_ms, sg.status, dst)

    def launch(self, b: Bucket) -> None:
        if not self.enabled:
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self._reduce(b)
        self._launched.append(b.name)

    def finish(self) -> None:
        done = set(self._launched)
        self._launched.clear()
        if not self.enabled:
            return
        if done:
            torch.cuda.current_stream().wait_stream(self.stream)
        for b in self.store.buckets:             # buckets whose hook did not fire (embedding, head, unused)
            if b.name not in done:
                self._reduce(b)

    def weigh(self, factors: dict) -> None:
        """Multiply the sum-of-squares partials of the named buckets (``{bucket name: factor}``, ``"*"`` for
        all others). Used when several ranks hold the same reduced values (replicas of a hybrid-sharded
        group, parameters replicated over tensor-parallel ranks) and the norm is then summed over all
        of them."""
        default = factors.get("*", 1.0)
        for i, b in enumerate(self.store.buckets):
            f = factors.get(b.name, default)
            if f != 1.0:
                self.partials[i * BLOCKS_PER_BUCKET:(i + 1) * BLOCKS_PER_BUCKET].mul_(f)


class PeerAdamW(FlatAdamW):
    """AdamW whose state is sharded over the ranks of the store's :class:`SymmGroup` (steps 2 and 3)."""

    def __init__(self, store: FlatParamStore, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 scalars=None):
        """``scalars``: the :class:`SymmGroup` over which the end-of-step scalars are exchanged (default:
        the store's own group). Pass a world-wide group when the model is also split over pipeline
        stages or tensor-parallel ranks."""
        sg = store.symm
        if sg is None:
            raise ValueError("PeerAdamW needs a FlatParamStore built on a SymmGroup")
        lay = store.layout
        super().__init__(store, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, shard_rank=lay.shard_rank,
                         shard_world=max(lay.shard_world, 1))
        self.sg, self.layout = sg, lay
        self.sx = scalars if scalars is not None else sg
        self.stats = torch.zeros(4, dtype=torch.float32, device=store.device)
        self.slot_step = self.sx.reserve_slots(1)
        self.slot_done = sg.reserve_slots(1)
        self._tables = None
        self._tables_wd = None
        self._full = None

    # ------------------------------------------------------------------ chunk tables
    def _build_tables(self, wd: float):
        st, lay = self.store, self.layout
        chunk = int(ops.require().comm_adam_chunk())
        dev = st.device
        tables = []
        for local in (False, True):            # shards whose result goes to every peer; buckets only this rank holds
            off, soff, ln, wds = [], [], [], []
            for b in st.buckets:
                if b.local != local:
                    continue
                lo, n = st.shard_range(b, lay.shard_rank)
                for seg_off, seg_n, dec in self._segments(b):
                    a = max(b.start + seg_off, lo)
                    e = min(b.start + seg_off + seg_n, lo + n)
                    while a < e:
                        step = min(chunk, e - a)
                        off.append(a)
                        soff.append(b.moff + (a - lo))
                        ln.append(step)
                        wds.append(wd if dec else 0.0)
                        a += step
            tables.append((torch.tensor(off, dtype=torch.int64, device=dev), torch.tensor(soff, dtype=torch.int64, device=dev),
                           torch.tensor(ln, dtype=torch.int32, device=dev), torch.tensor(wds, dtype=torch.float32, device=dev)))
        self._tables = tables
        self._tables_wd = wd

    # ------------------------------------------------------------------ step 2
    def reduce_step(self, reducer: PeerReducer, loss: torch.Tensor, max_norm: float, skip_nonfinite: bool,
                    loss_weight: float = 1.0):
        """Enqueue the end-of-step exchange. Returns the device tensor ``[norm, mean loss, finite]``
        and fills ``ctl`` for :meth:`step`.

        The kernel adds the ranks' sums of squares and averages their losses over the ``scalars``
        group. When that group is wider than the data-parallel one, the caller weighs the partials
        (:meth:`PeerReducer.weigh`) so that every gradient element is counted once, and passes
        ``loss_weight`` so that the average comes out as the mean over the data-parallel ranks
        (0 on ranks that hold no loss, e.g. all but the last pipeline stage)."""
        sx = self.sx
        loss32 = loss.detach().to(torch.float32).reshape(1)
        if loss_weight != 1.0:
            loss32 = loss32 * float(loss_weight)
        xchg, flags, me = sx.xchg.ptrs, sx.flags.ptrs, sx.rank
        if self.local_only:
            xchg, flags, me = [xchg[sx.rank]], [flags[sx.rank]], 0
        ops.require().comm_step_reduce(reducer.partials, None, loss32, xchg, flags, self.slot_step,
                                       sx.next_epoch(self.slot_step), me, float(max_norm or 0.0),
                                       bool(skip_nonfinite), self.stats, self.ctl, sx.timeout_ms, sx.status)
        return self.stats[:3]

    local_only = False

    def detach(self, reducer: PeerReducer) -> None:
        """Timing diagnostics, one way: from now on the three kernels of the step touch this rank's
        memory only (peer tables of length one), so a step costs what it would cost with free
        communication. The ranks' weights drift apart afterwards; use it last."""
        self.local_only = reducer.local_only = True

    # ------------------------------------------------------------------ step 3
    @torch.no_grad()
    def step(self, closure=None):
        st, sg = self.store, self.sg
        self.steps += 1
        self._step_t.fill_(self.steps)
        lr = self.param_groups[0]["lr"]
        b1, b2 = self.defaults["betas"]
        wd = max(float(g["weight_decay"]) for g in self.param_groups)
        if self._tables is None or self._tables_wd != wd:
            self._build_tables(wd)
        bc1, bc2 = 1 - b1 ** self.steps, 1 - b2 ** self.steps
        everyone = st.shadow_symm.ptrs
        me = [everyone[sg.rank]]
        if self.local_only:
            everyone = me
        elif self.layout.replicas > 1:           # hybrid sharding: the other replicas compute the same shard themselves
            everyone = [everyone[r] for r in self.layout.replica_peers()]
        compact = getattr(st, "reduced", None)      # hybrid sharding: reduced gradients live in their own buffer
        for (off, soff, ln, wds), ptrs, shared in zip(self._tables, (everyone, me), (True, False)):
            if off.numel():
                from_compact = shared and compact is not None
                ops.require().comm_adamw_push(st.master, compact if from_compact else st.grad, self.exp_avg,
                                              self.exp_avg_sq, ptrs, off, soff, ln, wds, lr, b1, b2,
                                              self.defaults["eps"], bc1, bc2, self.ctl, from_compact)
        if not self.local_only:
            sg.barrier(self.slot_done)
        return None

    # ------------------------------------------------------------------ checkpoints
    def gather_full(self) -> None:
        """Expose the whole optimizer state per parameter (``torch.optim.AdamW`` layout) by gathering
        the moment shards into temporary full-size buffers. Pair with :meth:`release_full` (after a
        save) or :meth:`scatter_full` (after a load)."""
        st, lay = self.store, self.layout
        if lay.shard_world == 1:
            return
        full_m = torch.zeros(st.total, dtype=torch.float32, device=st.device)
        full_v = torch.zeros(st.total, dtype=torch.float32, device=st.device)
        for b in st.buckets:
            n, s0 = b.msize, b.moff
            if b.local:
                st.bucket_view(full_m, b).copy_(self.exp_avg[s0:s0 + n])
                st.bucket_view(full_v, b).copy_(self.exp_avg_sq[s0:s0 + n])
                continue
            dist.all_gather_into_tensor(st.bucket_view(full_m, b), self.exp_avg[s0:s0 + n], group=lay.shard_group)
            dist.all_gather_into_tensor(st.bucket_view(full_v, b), self.exp_avg_sq[s0:s0 + n], group=lay.shard_group)
        self._full = (full_m, full_v)
        for p in st.params:
            lo = st._offset[p]
            self.state[p] = {"step": self._step_t, "exp_avg": full_m[lo:lo + p.numel()].view(p.shape),
                             "exp_avg_sq": full_v[lo:lo + p.numel()].view(p.shape)}

    def release_full(self) -> None:
        if self._full is not None:
            self._full = None
            self.state.clear()

    def scatter_full(self) -> None:
        """Take this rank's shard back out of the full-size state (after ``load_state_dict``)."""
        if self._full is None:
            return
        st, lay = self.store, self.layout
        full_m, full_v = self._full
        steps = 0
        for p in st.params:                      # load_state_dict replaced the views by copies
            state = self.state.get(p)
            if not state:
                continue
            lo = st._offset[p]
            for key, flat in (("exp_avg", full_m), ("exp_avg_sq", full_v)):
                view = flat[lo:lo + p.numel()].view(p.shape)
                if key in state and state[key].data_ptr() != view.data_ptr():
                    view.copy_(state[key])
            if "step" in state:
                steps = max(steps, int(float(state["step"])))
        for b in st.buckets:
            lo, n = st.shard_range(b, lay.shard_rank)
            s0 = b.moff
            self.exp_avg[s0:s0 + n].copy_(full_m[lo:lo + n])
            self.exp_avg_sq[s0:s0 + n].copy_(full_v[lo:lo + n])
        self.steps = steps
        self._step_t.fill_(steps)
        self.release_full()

    def load_state_dict(self, state_dict) -> None:
        if self.layout.shard_world == 1:
            return super().load_state_dict(state_dict)
        if self._full is None:
            self.gather_full()
        torch.optim.Optimizer.load_state_dict(self, state_dict)
        self.scatter_full()
