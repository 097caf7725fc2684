"""The sm_100a training engine: one flat parameter store per rank, whatever the mesh.

Every rank holds the parameters of its (pipeline stage, tensor-parallel rank) coordinate in a
:class:`~forgeminds_b200.parallel.flat.FlatParamStore`; the weight-gradient GEMMs of the dense blocks
and of the fused tensor-parallel blocks accumulate straight into its fp32 gradient buffer. What
happens to a finished gradient bucket depends on the data-parallel group of that coordinate:

* inside one NVSwitch domain (up to 8 ranks): the peer-memory step of
  :mod:`forgeminds_b200.parallel.peer` -- pull reduce-scatter on a side stream while the backward
  is still running, one kernel for norm / loss / finite flag / clip coefficient, AdamW on the shard
  with the bf16 result pushed into the peers' working weights. ``dp_replicate x dp_shard`` (HSDP) is
  the same kernels with the shard index taken modulo ``dp_shard``. No NCCL call between the last
  backward and the next forward when the mesh is data-parallel only; with pipeline stages or tensor
  parallelism the scalars are exchanged over a second, world-wide symmetric group, so that is still
  true as long as the world fits one domain;
* otherwise: bucket-wise ``all_reduce`` (:class:`~forgeminds_b200.parallel.flat.BucketReducer`) and a
  replicated fused AdamW.

Muon (``TrainConfig.optimizer = "muon"``) runs owner-computes on the peer path
(:class:`~forgeminds_b200.parallel.peer_muon.PeerMuon`) and replicated otherwise.

The update is enqueued before the step's single host read: the optimizer kernels take the clip
coefficient and the apply flag from device memory (``ctl``). The reference reads the norm on the host
first (``forgemind/trainer.py:297-310``).
"""
from __future__ import annotations

import contextlib
import os

import torch
import torch.distributed as dist

from ..distributed import log
from ..parallel.flat import BucketReducer, DpLayout, FlatAdamW, FlatParamStore


PEER_MUON = True          # owner-computes Muon over peer memory (parallel/peer_muon.py)


def same_host(ctx) -> bool:
    """True when every rank of the job runs on this host (one NVSwitch domain)."""
    if ctx.world <= 1:
        return True
    local = os.environ.get("LOCAL_WORLD_SIZE")
    if local is not None:
        return int(local) == ctx.world
    return ctx.world <= torch.cuda.device_count()


class NativeEngine:
    name = "native"

    def __init__(self, owner, model):
        self.t = owner
        cfg, ctx = owner.cfg, owner.ctx
        tc, pc = cfg.train, cfg.parallel
        self.ctx, self.tc, self.pc = ctx, tc, pc
        self.model = model
        dp = ctx.dp_world > 1
        self.layout = DpLayout.of(ctx)
        tp_state = getattr(model, "_fm_tp", None)
        self.tp_state = tp_state if (tp_state is not None and not isinstance(tp_state, str)) else None
        self.tp = pc.tp if self.tp_state is not None else 1
        self.wide = ctx.world > ctx.dp_world            # model-parallel dimensions besides data parallelism
        self._sync_now = True
        self.muon = None
        # expert parallelism: a rank's experts are its own -- their gradients already cover the tokens of the
        # whole expert-parallel group and are only summed over the ranks that hold the same experts
        self.edp_group, self.edp_size = None, 1
        if pc.ep > 1:
            for name, p in model.named_parameters():
                if ".experts." in name:
                    p._fm_local = True
            if ctx.edp_group is not None and dist.get_world_size(ctx.edp_group) > 1:
                self.edp_group, self.edp_size = ctx.edp_group, dist.get_world_size(ctx.edp_group)
        self.peer = self._try_peer(model, dp)
        if not self.peer:
            self.store = FlatParamStore(model, ctx.device, apart=self._apart())
            self.opt = FlatAdamW(self.store, lr=tc.lr, betas=tc.betas, eps=tc.eps, weight_decay=tc.weight_decay)
            self.reducer = BucketReducer(self.store, ctx.dp_group, ctx.dp_world, local_group=self.edp_group) \
                if dp else None
            if tc.optimizer == "muon":
                self.muon = owner._muon(model, tc)
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=ctx.device)
        self._rest_sq = torch.zeros(1, dtype=torch.float32, device=ctx.device)
        self._hook_blocks(model)

    # ------------------------------------------------------------------ set-up
    def _apart(self):
        if self.tp_state is None:
            return None
        return lambda p: getattr(p, "_tp_partial", False)

    def _try_peer(self, model, dp: bool) -> bool:
        """Build the peer-memory step when the groups allow it; report and fall back otherwise."""
        ctx, tc, pc = self.ctx, self.tc, self.pc
        if ctx.device.type != "cuda" or not pc.fused_comm or ctx.dp_world > 8 or not same_host(ctx) \
                or (self.wide and ctx.world > 8):
            return False
        if tc.optimizer == "muon" and not PEER_MUON:
            return False
        from ..parallel.peer import PeerAdamW, PeerReducer
        from ..parallel.symm import SymmGroup
        try:
            sg = SymmGroup(ctx.dp_group if dp else None, ctx.device, timeout_ms=pc.comm_timeout_ms, solo=not dp)
            self.sx = SymmGroup(None, ctx.device, timeout_ms=pc.comm_timeout_ms) if self.wide else sg
            self.store = FlatParamStore(model, ctx.device, symm=sg, layout=self.layout, apart=self._apart())
        except (RuntimeError, ValueError, OSError) as exc:           # no peer mapping on this machine
            log(ctx, f"[forgeminds_b200] peer-memory step unavailable ({exc!r}); reducing with all_reduce")
            return False
        if tc.optimizer == "muon":
            from ..parallel.peer_muon import PeerMuon
            self.opt = PeerMuon(self.store, model, tc, scalars=self.sx)
            self.muon = None
        else:
            self.opt = PeerAdamW(self.store, lr=tc.lr, betas=tc.betas, eps=tc.eps, weight_decay=tc.weight_decay,
                                 scalars=self.sx)
        self.reducer = PeerReducer(self.store, local_group=self.edp_group)
        return True

    def _hook_blocks(self, model) -> None:
        if self.reducer is None:
            return
        by_name = {b.name: b for b in self.store.buckets}
        for i, blk in enumerate(model.layers.values()):
            mine = [by_name[n] for n in (f"block{i}", f"experts{i}") if n in by_name]
            if mine:
                blk.register_full_backward_hook(self._on_block_done(mine))

    def _on_block_done(self, buckets):
        def fire(module, grad_in, grad_out):
            if self._sync_now:
                for bucket in buckets:
                    self.reducer.launch(bucket)
        return fire

    # ------------------------------------------------------------------ micro-batches
    def sync_scope(self, final: bool, forward: bool = False):
        """Bracket of one backward: gradient buckets may be reduced only in the very last one."""
        if not forward:
            self._sync_now = bool(final)
        return contextlib.nullcontext()

    def micro_step(self, ids, y, last: bool):
        t = self.t
        if t.pp is not None:
            self._sync_now = False
            loss = t.pp.step(ids, y, last_sync=last)
            self._sync_now = True
            return loss if loss is not None else torch.zeros((), device=self.ctx.device)
        self._sync_now = last
        with t._autocast(), t.quant.autocast():
            ce, aux = self.model(ids, labels=y)
            loss = ce if aux is None else ce + aux
        (loss / self.tc.grad_accum).backward()
        return ce.detach().float()

    def begin_step(self, lr: float) -> None:
        for g in self.opt.param_groups:
            g["lr"] = lr
        if self.muon is not None:
            self.t._schedule_muon(self.muon, lr)

    # ------------------------------------------------------------------ end of the step
    def _sum_partial_grads(self) -> None:
        """Tensor parallelism: replicated parameters that saw only this rank's rows (block norms, the
        embedding) get the other ranks' contributions before the data-parallel reduction."""
        if self.tp_state is None:
            return
        from ..parallel import tp as fused_tp
        fused_tp.sync_partial_grads(self.model, self.tp_state)

    def clip(self):
        """Global gradient norm as a 0-dim device tensor; leaves the clip coefficient in ``ctl[0]``
        (all_reduce path; the peer path gets both from :meth:`settle`)."""
        tc, ctx, st = self.tc, self.ctx, self.store
        sq = st.grad_sq_norm(self._norm_sq)[0]
        if self.tp > 1:
            rest = next((b for b in st.buckets if b.name == "rest"), None)
            if rest is not None:        # replicated over the tensor-parallel ranks: count it once
                r_sq = st.grad_sq_norm(self._rest_sq, st.bucket_view(st.grad, rest))[0]
                sq = sq - r_sq * (1.0 - 1.0 / self.tp)
            sq = sq.clone()
            dist.all_reduce(sq, group=ctx.tp_group)
        if self.pc.ep > 1 and ctx.world > 1:
            # every expert-parallel rank holds different experts: their squares add up over the group
            own = torch.zeros((), dtype=torch.float32, device=ctx.device)
            for b in st.buckets:
                if b.local:
                    own = own + st.grad_sq_norm(self._rest_sq, st.bucket_view(st.grad, b))[0]
            spread = own.clone()
            dist.all_reduce(spread, group=ctx.ep_group)
            sq = sq - own + spread
        if self.pc.pp > 1:
            sq = ctx.sum_over_pp(sq)
        norm = sq.clamp(min=0).sqrt()
        if tc.grad_clip and tc.grad_clip > 0:
            coef = torch.clamp(tc.grad_clip / (norm + 1e-6), max=1.0)
        else:
            coef = torch.ones_like(norm)
        self.opt.ctl[0:1].copy_(coef.reshape(1))
        return norm

    def settle(self, loss):
        """Reduce what is left, produce ``[flag, norm, loss(, status)]`` on the device and, unless a
        spike guard needs the host's opinion first, enqueue the update. Returns ``(tensor, early)``."""
        t, tc, ctx = self.t, self.tc, self.ctx
        self._sum_partial_grads()
        if self.reducer is not None:
            self.reducer.finish()
        early = not (tc.skip_spike_factor > 0)
        if self.peer:
            lay = self.layout
            if self.wide or lay.replicas > 1 or self.edp_size > 1:
                f = 1.0 / lay.replicas
                factors = {"*": f, "rest": f / self.tp}
                for b in self.store.buckets:
                    if b.local:                      # as many copies as ranks holding the same experts
                        factors[b.name] = 1.0 / self.edp_size
                self.reducer.weigh(factors)
            weight = 1.0
            if self.wide:
                # the kernel averages over the world: the ranks of the last stage hold the loss, once per
                # tensor-parallel rank; everybody else contributes zero
                has_loss = self.pc.pp == 1 or ctx.pp_rank == self.pc.pp - 1
                weight = ctx.world / float(ctx.dp_world * self.pc.tp) if has_loss else 0.0
            stats = self.opt.reduce_step(self.reducer, loss, tc.grad_clip, tc.skip_nonfinite, loss_weight=weight)
            if early:
                self.apply()
            words = [self.store.symm.status.to(torch.float32)]
            out = torch.cat([stats[2:3], stats[0:1], stats[1:2], *words])
            return out, early
        gn = t._clip().to(ctx.device)
        loss = t._reduce_loss(loss)
        if tc.skip_nonfinite:
            finite = (torch.isfinite(gn) & torch.isfinite(loss)).to(torch.int32)
        else:
            finite = torch.ones((), dtype=torch.int32, device=loss.device)
        flag = ctx.all_min_int(finite).to(torch.float32)
        self.opt.ctl[1:2].copy_(flag.reshape(1))
        if early:
            self.apply()
        return torch.stack([flag, gn.to(torch.float32), loss]), early

    def check(self, values) -> None:
        if self.peer and len(values) > 3:
            self.store.symm.check(int(values[3]))

    def apply(self) -> None:
        """Enqueue the parameter update; it reads ``ctl`` (clip coefficient, apply flag) on the device."""
        if self.muon is not None:
            self.muon.step(ctl=self.opt.ctl)
            self.store.refresh_shadow()
            self.opt.steps += 1
        else:
            self.opt.step()

    def approve(self) -> None:
        """The host decided (spike guard) that a late update goes ahead."""
        self.opt.ctl[1:2].fill_(1.0)
        self.apply()

    def rejected(self, early: bool) -> None:
        if early and isinstance(getattr(self.opt, "steps", None), int):
            self.opt.steps -= 1                    # the kernels left everything untouched

    def zero_grad(self) -> None:
        self.opt.zero_grad(set_to_none=True)

    def detach_peers(self) -> bool:
        """Benchmark diagnostics (irreversible): run the data-parallel step on local memory only, to time
        a step whose communication is free. False when the engine has no peer step to detach (or tensor
        parallel kernels, whose collectives cannot be taken out of their GEMMs)."""
        if not self.peer or self.tp_state is not None or not hasattr(self.opt, "detach"):
            return False
        self.opt.detach(self.reducer)
        return True

    # ------------------------------------------------------------------ checkpoints
    def state_for_dcp(self):
        from torch.distributed.checkpoint.state_dict import get_state_dict
        if self.peer:
            self.store.sync_master()
            self.opt.gather_full()
        msd, osd = get_state_dict(self.model, self.opt)
        if self.muon is not None:
            self.muon.init_state()         # gradients are never None here, so torch would not create it
            _, extra = get_state_dict(self.model, self.muon)
            osd = {"flat": osd, "muon": extra}
        return msd, osd

    def after_save(self) -> None:
        if self.peer:
            self.opt.release_full()

    def load_from_dcp(self, msd, osd) -> None:
        from torch.distributed.checkpoint.state_dict import set_state_dict
        if self.muon is not None:
            set_state_dict(self.model, self.opt, model_state_dict=msd, optim_state_dict=osd["flat"])
            set_state_dict(self.model, self.muon, model_state_dict=msd, optim_state_dict=osd["muon"])
        else:
            set_state_dict(self.model, self.opt, model_state_dict=msd, optim_state_dict=osd)
        if self.peer:
            self.opt.scatter_full()
        self.store.refresh_shadow()

    def sync_params(self) -> None:
        if self.peer:
            self.store.sync_master()
