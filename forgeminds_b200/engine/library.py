"""The portable training engine: ``torch.distributed`` wrappers and ``torch.optim`` optimizers.

Runs everywhere (CPU + Gloo in the test-suite, fp32, quantisation back ends that bring their own
modules, optimizer offload, 8-bit optimizer state, DeepSpeed, ``torch.compile``) and is the path
the sm_100a engine is measured against. What it must do is fixed by the reference's training step
(``forgemind/trainer.py:213-323``):

* data parallelism through FSDP2 (``dp_shard``), HSDP (2-D mesh) or DDP (``dp_replicate``), with
  gradient synchronisation held back until the last micro-batch of an accumulation window;
* a global L2 gradient norm computed on the device that is correct for every mesh -- DTensor
  gradients are reduced per mesh, expert gradients are summed over the expert-parallel group, fused
  tensor-parallel shards over the tensor-parallel group, stages over the pipeline group -- and a
  clip coefficient ``min(1, clip / (norm + 1e-6))`` that is always multiplied in;
* a unanimous finite check (MIN all-reduce over the world) so that either every rank applies the
  update or none does.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel import native as wrappers


def _sq_norm(grads, device):
    if not grads:
        return torch.zeros((), device=device, dtype=torch.float32)
    return torch.nn.utils.get_total_norm(grads).float().square()


class LibraryEngine:
    name = "library"
    store = None
    reducer = None
    peer = False

    def __init__(self, owner, model):
        self.t = owner
        cfg, ctx = owner.cfg, owner.ctx
        self.ctx, self.tc, self.pc = ctx, cfg.train, cfg.parallel
        tc, pc, oc = cfg.train, cfg.parallel, cfg.offload
        self.off_opt = None
        self.off_overlap = False
        self.ds = None
        multi = ctx.dp_world > 1
        if owner.use_ds:
            from ..parallel.deepspeed_backend import init_deepspeed
            params = [p for p in model.parameters() if p.requires_grad]
            self.ds, self.opt = init_deepspeed(model, owner._param_groups(params, tc), cfg, ctx.world,
                                               owner.micro_batch)
            self.model = model
        else:
            if multi and pc.dp_shard > 1:
                model = wrappers.apply_fsdp(model, ctx, tc.bf16, pc.fsdp_cpu_offload, pc.fsdp_reshard_after_forward)
            elif multi and pc.dp_replicate > 1:
                model = wrappers.apply_ddp(model, ctx)
            self.model = model
            self.opt = self._make_optimizer(model, cfg)
        self.is_ddp = isinstance(self.model, nn.parallel.DistributedDataParallel)
        self.is_fsdp = hasattr(self.model, "set_requires_gradient_sync") and not self.is_ddp
        self.params = [p for p in self.model.parameters() if p.requires_grad]
        self.expert_params = wrappers.expert_params(self.model) if pc.ep > 1 else []
        self.sharded_grads = any(hasattr(p, "to_local") for p in self.params)
        tp_state = getattr(owner.raw, "_fm_tp", None)
        self.fused_tp = tp_state if (tp_state is not None and not isinstance(tp_state, str)) else None

    # ------------------------------------------------------------------ optimizer
    def _make_optimizer(self, model, cfg):
        tc, oc, ctx = cfg.train, cfg.offload, self.ctx
        params = [p for p in model.parameters() if p.requires_grad]
        groups = self.t._param_groups(params, tc)
        if oc.optimizer:
            if self.pc.pp > 1:
                raise AssertionError("optimizer offload + pipeline parallelism is not supported")
            from ..offload import OffloadedAdamW
            wrapped = isinstance(model, nn.parallel.DistributedDataParallel) or hasattr(model, "set_requires_gradient_sync")
            self.off_overlap = not wrapped
            self.off_opt = OffloadedAdamW(groups, tc.lr, tc.betas, tc.eps, oc, overlap=self.off_overlap)
            return self.off_opt
        if cfg.quant.optimizer_8bit:
            from ..quant import make_optimizer_8bit
            return make_optimizer_8bit(groups, tc.lr, tc.betas, tc.eps)
        if tc.optimizer == "muon":
            return self.t._muon(model, tc)
        # torch's fused kernel refuses a mix of DTensor and plain parameters (tensor-parallel blocks next to
        # a replicated embedding): such models take the foreach implementation
        uniform = len({hasattr(p, "to_local") for p in params}) == 1
        return torch.optim.AdamW(groups, lr=tc.lr, betas=tc.betas, eps=tc.eps,
                                 fused=ctx.device.type == "cuda" and uniform)

    # ------------------------------------------------------------------ micro-batches
    def sync_scope(self, final: bool, forward: bool = False):
        """Pipeline schedules: brackets of each micro-batch's forward and backward."""
        from ..parallel.pipeline import ddp_or_fsdp_scope
        return ddp_or_fsdp_scope(self.model, self.is_ddp, self.is_fsdp, final, forward)

    def micro_step(self, ids, y, last: bool):
        t = self.t
        if t.pp is not None:
            loss = t.pp.step(ids, y, last_sync=last)
            return loss if loss is not None else torch.zeros((), device=self.ctx.device)
        if self.is_fsdp:
            self.model.set_requires_gradient_sync(last)
        hold = self.model.no_sync() if (self.is_ddp and not last) else contextlib.nullcontext()
        with hold, t._autocast(), t.quant.autocast():
            ce, aux = self.model(ids, labels=y)
            objective = ce if aux is None else ce + aux
        if self.ds is not None:
            self.ds.backward(objective)
        else:
            (objective / self.tc.grad_accum).backward()
        if self.off_opt is not None and (self.off_overlap or last):
            self.off_opt.collect()
        return ce.detach().float()

    def begin_step(self, lr: float) -> None:
        if self.tc.optimizer == "muon" and hasattr(self.opt, "init_state"):
            self.t._schedule_muon(self.opt, lr)
        else:
            for g in self.opt.param_groups:
                g["lr"] = lr
        if self.off_opt is not None:
            self.off_opt.begin_step()

    # ------------------------------------------------------------------ norm and clipping
    def clip(self):
        tc, pc, ctx = self.tc, self.pc, self.ctx
        if self.off_opt is not None:
            return self.off_opt.clip_grad_norm_(tc.grad_clip).float()
        grads = [p.grad for p in self.params if p.grad is not None]
        dev = ctx.device
        if not grads:
            return torch.zeros((), device=dev, dtype=torch.float32)
        if self.sharded_grads:
            # one reduction per device mesh: DTensor norms are partial sums over their own mesh only
            meshes: dict = {}
            for g in grads:
                key = id(g.device_mesh) if hasattr(g, "to_local") else None
                meshes.setdefault(key, []).append(g)
            sq = torch.zeros((), device=dev, dtype=torch.float32)
            for key, members in meshes.items():
                part = torch.nn.utils.get_total_norm(members)
                if key is not None and hasattr(part, "full_tensor"):
                    part = part.full_tensor()
                sq = sq + part.float().square()
        else:
            sq = _sq_norm(grads, dev)
        if self.fused_tp is not None:
            # plain tensors holding this rank's slice: their squares add up over the tensor-parallel ranks
            own = _sq_norm([p.grad for p in self.params if p.grad is not None and hasattr(p, "_tp_shard_dim")], dev)
            spread = own.clone()
            dist.all_reduce(spread, group=ctx.tp_group)
            sq = sq - own + spread
        if pc.ep > 1 and ctx.world > 1:
            own = _sq_norm([p.grad for p in self.expert_params if p.grad is not None], dev)
            spread = own.clone()
            dist.all_reduce(spread, group=ctx.ep_group)
            sq = sq - own + spread
        if pc.pp > 1:
            sq = ctx.sum_over_pp(sq)
        norm = sq.clamp(min=0).sqrt()
        if tc.grad_clip and tc.grad_clip > 0:
            coef = torch.clamp(tc.grad_clip / (norm + 1e-6), max=1.0)
            if self.sharded_grads:
                for g in grads:
                    g.mul_(coef)
            else:
                torch._foreach_mul_(grads, coef)
        return norm

    # ------------------------------------------------------------------ end of the step
    def settle(self, loss):
        t, tc, ctx = self.t, self.tc, self.ctx
        wrappers.sync_expert_grads(self.model, ctx, self.expert_params)
        if self.fused_tp is not None:
            from ..parallel import tp as fused_tp
            fused_tp.sync_partial_grads(t.raw, self.fused_tp)
        gn = t._clip().to(ctx.device)
        loss = t._reduce_loss(loss)
        if tc.skip_nonfinite:
            vote = (torch.isfinite(gn) & torch.isfinite(loss)).to(torch.int32)
        else:
            vote = torch.ones((), dtype=torch.int32, device=loss.device)
        flag = ctx.all_min_int(vote).to(torch.float32)
        return torch.stack([flag, gn.to(torch.float32), loss]), False

    def check(self, values) -> None:
        pass

    def apply(self) -> None:
        self.opt.step()

    approve = apply

    def rejected(self, early: bool) -> None:
        pass

    def zero_grad(self) -> None:
        self.opt.zero_grad(set_to_none=True)

    # ------------------------------------------------------------------ DeepSpeed runs its own step
    def ds_step(self, loss):
        self.ds.step()
        return float(self.ds.get_global_grad_norm() or 0.0), float(loss)

    # ------------------------------------------------------------------ checkpoints
    def state_for_dcp(self):
        from torch.distributed.checkpoint.state_dict import get_state_dict
        return get_state_dict(self.model, () if self.off_opt is not None else self.opt)

    def after_save(self) -> None:
        pass

    def load_from_dcp(self, msd, osd) -> None:
        from torch.distributed.checkpoint.state_dict import set_state_dict
        if self.off_opt is not None:
            set_state_dict(self.model, (), model_state_dict=msd, optim_state_dict={})
        else:
            set_state_dict(self.model, self.opt, model_state_dict=msd, optim_state_dict=osd)

    def sync_params(self) -> None:
        pass
