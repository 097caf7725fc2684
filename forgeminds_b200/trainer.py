"""Config-driven training loop with one host<->device synchronisation per optimizer step.

Public behaviour follows the reference's ``forgemind/trainer.py:41-459``: the same constructor, the
same set-up order (quantisation -> tensor parallel -> activation checkpointing / offload -> fused
ops -> cache warm-up -> compile -> data-parallel wrapper -> optimizer -> data -> pipeline -> resume),
the cosine schedule, device-side clipping, the unanimous non-finite / loss-spike skip, the metric
dictionary of ``train_step`` and the checkpoint layout.

Two engines sit behind it:

* **library** -- ``torch`` FSDP2 / DDP / DTensor with ``torch.optim.AdamW`` (CPU, Gloo, fp32, or
  ``TrainConfig.native=False``); identical to what the reference runs.
* **native** (CUDA + bf16 on a B200) -- the model's blocks run on the sm_100a kernels, parameters
  live in a :class:`~forgeminds_b200.parallel.flat.FlatParamStore`, gradient buckets are reduced on
  a side stream while the backward is still running, and clipping + AdamW + the bf16 weight refresh
  are one fused kernel per bucket that reads its clip coefficient and skip flag from device memory.
  The optimizer is therefore enqueued *before* the single host read of the step.
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import shutil
import time
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import Dataset

from .config import ForgeConfig
from .data import BatchStream, async_loader, build_loader
from .distributed import DistContext, init_distributed, log
from .loss import logits_cross_entropy
from .offload import OffloadedAdamW, apply_activation_offload
from .parallel import native
from .parallel.ac import apply_activation_checkpointing
from .parallel.pipeline import PipelineRunner
from .perf import enable_fast_math, warn_once
from .quant import QuantState, make_optimizer_8bit, quantize_model


class _Stack:
    """Enter several context managers as one."""

    def __init__(self, *cms):
        self.cms = cms

    def __enter__(self):
        for c in self.cms:
            c.__enter__()

    def __exit__(self, *exc):
        for c in reversed(self.cms):
            c.__exit__(*exc)


def moe_kwargs(ctx: DistContext, cfg: ForgeConfig) -> dict:
    """Keyword arguments for ``GPT(cfg, moe_kwargs=...)`` that wire expert parallelism / offload."""
    return dict(ep_size=ctx.pc.ep, ep_group=ctx.ep_group, ep_rank=ctx.ep_rank, offload_experts=cfg.offload.experts)


class Trainer:
    def __init__(self, model_fn: Callable[[DistContext], nn.Module], cfg: ForgeConfig, train_ds: Dataset,
                 eval_ds: Optional[Dataset] = None, micro_batch: int = 8, callbacks=(),
                 peak_flops: Optional[float] = None):
        self.cfg = cfg
        tc, pc, oc = cfg.train, cfg.parallel, cfg.offload
        self.ctx = ctx = init_distributed(pc)
        self.micro_batch, self.callbacks, self.peak_flops = micro_batch, list(callbacks), peak_flops
        self.use_ds = pc.backend == "deepspeed"
        enable_fast_math(pc.backend == "native")
        torch.manual_seed(tc.seed)
        model = model_fn(ctx)
        self.raw = model
        mcfg = getattr(model, "cfg", None)
        self.seq = getattr(mcfg, "max_seq", None)

        if pc.ep > 1:          # every ep rank owns different experts: draw them from a rank-specific stream
            gen = torch.Generator().manual_seed(tc.seed + 1 + ctx.ep_rank)
            for name, p in model.named_parameters():
                if ".experts." in name:
                    p.data.normal_(0, 0.02, generator=gen)
        if pc.pp > 1:
            model.split_stage(ctx.pp_rank, pc.pp)
            if getattr(mcfg, "aux_coef", 0) and getattr(mcfg, "n_experts", 0):
                log(ctx, "[forgeminds_b200] WARNING: the MoE aux loss is not propagated across pipeline stages")
        model.to(ctx.device)

        self.native = self._wants_native(model)
        if mcfg is not None and hasattr(mcfg, "native") and not self.native:
            mcfg.native = False
            for blk in getattr(model, "layers", {}).values() if hasattr(model, "layers") else []:
                if hasattr(blk, "native"):
                    blk.native = False

        if pc.ep > 1 and self.native and pc.fused_comm and pc.ep <= 8 and not oc.experts:
            from .parallel import ep as fused_ep      # dispatch / combine inside the permutation kernels
            fused_ep.attach(model, ctx)
        self.quant: QuantState = quantize_model(model, cfg.quant, ctx.dp_group)
        if pc.tp > 1:
            native.apply_tp(model, ctx)
        if tc.ac != "none":
            apply_activation_checkpointing(model, tc.ac, preserve_rng_state=tc.ac_preserve_rng)
        if oc.activations and ctx.device.type == "cuda":
            apply_activation_offload(model, oc)
        self.model = model
        if tc.fused_ops:
            from .kernels import available as kernels_available
            from .kernels.apply import enable as enable_kernels
            fused = enable_kernels(model, norm=True, swiglu_mlp=True, split=tc.fused_split_mlp)._fm_fused
            warn_once(f"[forgeminds_b200] fused kernels patched {fused['norm']} norm / {fused['mlp']} MLP modules "
                      f"(native={kernels_available()})", key="fused_ops")
        self._warm(model, tc.bf16)
        if tc.compile:
            self._compile(model, tc)

        # ---- data-parallel wrapper + optimizer
        self.store = self.reducer = None
        self.off_opt = None
        dp = ctx.dp_world > 1
        trainable = [p for p in model.parameters() if p.requires_grad]
        if not trainable:
            raise RuntimeError("[forgeminds_b200] no trainable parameters -- every parameter is frozen "
                               "(int8_wo freezes the base weights: add adapters or unfreeze something)")
        if self.use_ds:
            groups = self._param_groups(trainable, tc)
            from .parallel.deepspeed_backend import init_deepspeed
            self.engine, self.opt = init_deepspeed(self.model, groups, cfg, ctx.world, micro_batch)
        elif self.native and self._flat_ok(oc, cfg) and self._fits_resident(trainable, pc):
            self._setup_native(model, tc, pc, dp)
        else:
            if dp and pc.dp_shard > 1:
                self.model = native.apply_fsdp(model, ctx, tc.bf16, pc.fsdp_cpu_offload, pc.fsdp_reshard_after_forward)
            elif dp and pc.dp_replicate > 1:
                self.model = native.apply_ddp(model, ctx)
            trainable = [p for p in self.model.parameters() if p.requires_grad]
            groups = self._param_groups(trainable, tc)
            if oc.optimizer:
                assert pc.pp == 1, "optimizer offload + pipeline parallelism is not supported"
                overlap = not self._wrapped()
                self.opt = self.off_opt = OffloadedAdamW(groups, tc.lr, tc.betas, tc.eps, oc, overlap=overlap)
                self.off_overlap = overlap
            elif cfg.quant.optimizer_8bit:
                self.opt = make_optimizer_8bit(groups, tc.lr, tc.betas, tc.eps)
            elif tc.optimizer == "muon":
                self.opt = self._muon(self.model, tc)
            else:
                kinds = {hasattr(p, "to_local") for p in trainable}
                # the fused kernel refuses a mix of DTensor and plain parameters (tensor parallel blocks
                # next to a replicated embedding): such models take the foreach implementation
                self.opt = torch.optim.AdamW(groups, lr=tc.lr, betas=tc.betas, eps=tc.eps,
                                             fused=ctx.device.type == "cuda" and len(kinds) == 1)
        self.is_ddp = isinstance(self.model, nn.parallel.DistributedDataParallel)
        self.is_fsdp = hasattr(self.model, "set_requires_gradient_sync") and not self.is_ddp
        self._trainable = [p for p in self.model.parameters() if p.requires_grad]
        self._expert_params = native.expert_params(self.model) if pc.ep > 1 else []
        self._has_dtensor = any(hasattr(p, "to_local") for p in self._trainable)

        # ---- data
        self.train_dl, self.sampler = build_loader(train_ds, micro_batch, ctx, tc.seed, workers=tc.workers)
        self.feed = BatchStream(self.train_dl, self.sampler, ctx.device, prefetch=tc.prefetch,
                                depth=tc.prefetch_depth, threaded=tc.batch_thread)
        self.eval_dl = None
        if eval_ds is not None:
            self.eval_dl = build_loader(eval_ds, micro_batch, ctx, tc.seed, workers=0, shuffle=False)[0]

        # ---- pipeline
        self.pp = None
        if pc.pp > 1:
            assert micro_batch % pc.pp_microbatches == 0, "micro_batch must be divisible by pp_microbatches"
            self.pp = PipelineRunner(self.model, ctx, logits_cross_entropy, pc.pp_microbatches, pc.pp_schedule,
                                     fwd_ctx=lambda: _Stack(self._autocast(), self.quant.autocast()))

        self.step, self.loss_ema, self.history, self.skipped = 0, None, [], 0
        n_params = sum(p.numel() for p in self.raw.parameters())
        log(ctx, f"[forgeminds_b200] world={ctx.world} mesh(pp,dp_rep,dp_shard,tp)=({pc.pp},{pc.dp_replicate},"
                 f"{pc.dp_shard},{pc.tp}) ep={pc.ep} engine={'native' if self.store is not None else 'library'} "
                 f"quant={cfg.quant.mode}/{self.quant.backend} params(local)={n_params / 1e6:.1f}M device={ctx.device}")
        if tc.resume:
            self.maybe_resume()

    # ------------------------------------------------------------------ set-up helpers
    def _wants_native(self, model) -> bool:
        tc = self.cfg.train
        if tc.native is False or not tc.bf16 or self.ctx.device.type != "cuda" or self.use_ds:
            return False
        from . import ops
        if not ops.available():
            if tc.native or torch.cuda.get_device_capability(self.ctx.device)[0] == 10:
                ops.require()
            return False
        return hasattr(model, "layers")

    def _flat_ok(self, oc, cfg) -> bool:
        tc, pc = cfg.train, cfg.parallel
        return not (oc.optimizer or cfg.quant.optimizer_8bit or pc.fsdp_cpu_offload or tc.compile) \
            and cfg.quant.mode in ("none", "fp8", "int8") and pc.tp == 1 and pc.ep == 1

    def _fits_resident(self, params, pc) -> bool:
        """The native engine keeps the bf16 working weights of the whole model on every GPU. A model
        whose weights exceed ``fsdp_resident_bytes`` and that asks for sharding goes to FSDP2 instead."""
        if pc.dp_shard in (0, 1):
            return True
        return 2 * sum(p.numel() for p in params) <= int(pc.fsdp_resident_bytes)

    def _setup_native(self, model, tc, pc, dp: bool) -> None:
        from .parallel.flat import BucketReducer, FlatAdamW, FlatParamStore
        ctx = self.ctx
        # Peer-memory step (parallel/peer.py): one data-parallel dimension inside one NVSwitch domain,
        # AdamW, no pipeline stages. Everything else reduces whole buckets with all_reduce.
        self.peer = bool(pc.fused_comm) and tc.optimizer != "muon" and pc.pp == 1 and ctx.dp_world <= 8 \
            and not (pc.dp_replicate > 1 and pc.dp_shard > 1)
        if self.peer:
            from .parallel.peer import PeerAdamW, PeerReducer
            from .parallel.symm import SymmGroup
            sg = SymmGroup(ctx.dp_group if dp else None, ctx.device, timeout_ms=pc.comm_timeout_ms)
            self.store = FlatParamStore(model, ctx.device, symm=sg)
            self.opt = PeerAdamW(self.store, lr=tc.lr, betas=tc.betas, eps=tc.eps, weight_decay=tc.weight_decay)
            self.reducer = PeerReducer(self.store)
            self._muon_opt = None
        else:
            self.store = FlatParamStore(model, ctx.device)
            self.opt = FlatAdamW(self.store, lr=tc.lr, betas=tc.betas, eps=tc.eps, weight_decay=tc.weight_decay)
            self._muon_opt = self._muon(model, tc) if tc.optimizer == "muon" else None
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=ctx.device)
        if dp and pc.ep > 1:
            raise NotImplementedError("native engine + expert parallelism: handled by parallel.ep")
        if dp and not self.peer:
            self.reducer = BucketReducer(self.store, ctx.dp_group, ctx.dp_world)
        if self.reducer is not None:
            blocks = list(model.layers.values())
            by_name = {b.name: b for b in self.store.buckets}
            for i, blk in enumerate(blocks):
                bucket = by_name.get(f"block{i}")
                if bucket is not None:
                    blk.register_full_backward_hook(self._bucket_hook(bucket))

    def _bucket_hook(self, bucket):
        def fire(module, grad_in, grad_out):
            if self._sync_now:
                self.reducer.launch(bucket)
        return fire

    def _muon(self, model, tc):
        from .muon import Muon
        mats = [p for n, p in model.named_parameters() if p.requires_grad and p.ndim >= 2 and ".layers." in f".{n}"]
        ids = {id(p) for p in mats}
        rest = [p for p in model.parameters() if p.requires_grad and id(p) not in ids]
        groups = [dict(params=mats, use_muon=True, lr=tc.muon_lr, momentum=tc.muon_momentum,
                       ns_steps=tc.muon_ns_steps, weight_decay=tc.weight_decay)]
        if rest:
            groups.append(dict(params=rest, use_muon=False, lr=tc.lr, betas=tc.betas, eps=tc.eps,
                               weight_decay=0.0))
        return Muon(groups, lr=tc.muon_lr, group=self.ctx.dp_group if self.ctx.dp_world > 1 else None)

    @staticmethod
    def _param_groups(params, tc) -> list:
        decay = [p for p in params if p.ndim >= 2]
        rest = [p for p in params if p.ndim < 2]
        groups = [{"params": decay, "weight_decay": tc.weight_decay}, {"params": rest, "weight_decay": 0.0}]
        return [g for g in groups if g["params"]]

    def _wrapped(self) -> bool:
        return isinstance(self.model, nn.parallel.DistributedDataParallel) or \
            hasattr(self.model, "set_requires_gradient_sync")

    def _warm(self, model, bf16: bool) -> None:
        prepare = getattr(model, "prepare", None)
        if prepare is None:
            return
        dtype = torch.bfloat16 if bf16 else torch.float32
        try:
            prepare(device=self.ctx.device, dtype=dtype, seq=self.seq)
        except TypeError:
            prepare()

    def _compile(self, model, tc) -> None:
        layers = getattr(model, "layers", None)
        blocks = list(layers.values()) if hasattr(layers, "values") else list(layers or [])
        kw = dict(mode=tc.compile_mode, fullgraph=tc.compile_fullgraph, backend=tc.compile_backend)
        if not blocks:
            model.compile(**kw)
            return
        for blk in blocks:
            moe = blk.ffn if getattr(blk, "is_moe", False) else None
            if moe is not None and tc.compile_fullgraph and not getattr(moe, "compile_friendly", True):
                raise RuntimeError("compile_fullgraph=True is not possible for this MoE block: its dispatch needs a "
                                   "host read on this device")
            blk.compile(**kw)

    # ------------------------------------------------------------------ small helpers
    @property
    def epoch(self):
        return self.feed.epoch

    @property
    def batches_in_epoch(self):
        return self.feed.batches

    def lr_at(self, step: int) -> float:
        tc = self.cfg.train
        if step < tc.warmup_steps:
            return tc.lr * (step + 1) / tc.warmup_steps
        span = max(1, tc.max_steps - tc.warmup_steps)
        t = min(1.0, (step - tc.warmup_steps) / span)
        return tc.lr * (tc.min_lr_ratio + (1 - tc.min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * t)))

    def _autocast(self):
        if self.cfg.train.bf16 and self.ctx.device.type in ("cuda", "cpu"):
            return torch.autocast(self.ctx.device.type, dtype=torch.bfloat16)
        return contextlib.nullcontext()

    # ------------------------------------------------------------------ gradient norm / clipping
    def _clip(self):
        """Global gradient norm as a 0-dim fp32 device tensor; clips in place (library engine) or
        stores the coefficient for the fused optimizer kernel (native engine)."""
        tc, pc, ctx = self.cfg.train, self.cfg.parallel, self.ctx
        if self.off_opt is not None:
            return self.off_opt.clip_grad_norm_(tc.grad_clip).float()
        if self.store is not None:
            sq = self.store.grad_sq_norm(self._norm_sq)[0]
            if pc.pp > 1:
                sq = ctx.sum_over_pp(sq)
            norm = sq.clamp(min=0).sqrt()
            coef = torch.clamp(tc.grad_clip / (norm + 1e-6), max=1.0) if tc.grad_clip and tc.grad_clip > 0 \
                else torch.ones_like(norm)
            self.opt.ctl[0:1].copy_(coef.reshape(1))
            return norm
        grads = [p.grad for p in self._trainable if p.grad is not None]
        if not grads:
            return torch.zeros((), device=ctx.device, dtype=torch.float32)
        if self._has_dtensor:
            sharded = [g for g in grads if hasattr(g, "to_local")]
            plain = [g for g in grads if not hasattr(g, "to_local")]
            sq = torch.zeros((), device=ctx.device, dtype=torch.float32)
            by_mesh: dict = {}
            for g in sharded:
                by_mesh.setdefault(id(g.device_mesh), []).append(g)
            for members in by_mesh.values():
                n = torch.nn.utils.get_total_norm(members)
                n = n.full_tensor() if hasattr(n, "full_tensor") else n
                sq = sq + n.float().pow(2)
            if plain:
                sq = sq + torch.nn.utils.get_total_norm(plain).float().pow(2)
            norm = sq.sqrt()
        else:
            norm = torch.nn.utils.get_total_norm(grads).float()
        tp_state = getattr(self.raw, "_fm_tp", None)
        if tp_state is not None and not isinstance(tp_state, str):
            # fused tensor parallelism keeps plain tensors: the sharded weights' share of the norm is
            # spread over the tp ranks, everything else is replicated
            mine = [p.grad for p in self._trainable if p.grad is not None and hasattr(p, "_tp_shard_dim")]
            s_sq = torch.nn.utils.get_total_norm(mine).float().pow(2) if mine else torch.zeros((), device=norm.device)
            rep_sq = norm.pow(2) - s_sq
            dist.all_reduce(s_sq, group=ctx.tp_group)
            norm = (rep_sq + s_sq).clamp(min=0).sqrt()
        if pc.ep > 1 and ctx.world > 1:      # expert gradients of the other ep ranks belong to the same model
            mine = [p.grad for p in self._expert_params if p.grad is not None]
            e_sq = torch.nn.utils.get_total_norm(mine).float().pow(2) if mine else torch.zeros((), device=norm.device)
            dense_sq = norm.pow(2) - e_sq
            dist.all_reduce(e_sq, group=ctx.ep_group)
            norm = (dense_sq + e_sq).clamp(min=0).sqrt()
        if pc.pp > 1:
            norm = ctx.sum_over_pp(norm.pow(2)).clamp(min=0).sqrt()
        if tc.grad_clip and tc.grad_clip > 0:
            coef = torch.clamp(tc.grad_clip / (norm + 1e-6), max=1.0)
            if self._has_dtensor:
                for g in grads:
                    g.mul_(coef)
            else:
                torch._foreach_mul_(grads, coef)
        return norm

    # ------------------------------------------------------------------ one micro-batch
    _sync_now = True

    def _fwd_bwd_micro(self, last: bool):
        accum = self.cfg.train.grad_accum
        ids, y = self.feed.next()
        self._sync_now = last
        if self.pp is not None:
            loss = self.pp.step(ids, y, last_sync=last)
            return loss if loss is not None else torch.zeros((), device=self.ctx.device)
        if self.is_fsdp:
            self.model.set_requires_gradient_sync(last)
        hold = self.model.no_sync() if (self.is_ddp and not last) else contextlib.nullcontext()
        with hold, self._autocast(), self.quant.autocast():
            ce, aux = self.model(ids, labels=y)
            loss = ce if aux is None else ce + aux
        if self.use_ds:
            self.engine.backward(loss)
        else:
            (loss / accum).backward()
        if self.off_opt is not None and (self.off_overlap or last):
            self.off_opt.collect()
        return ce.detach().float()

    def train_step(self) -> dict:
        tc, ctx = self.cfg.train, self.ctx
        lr = self.lr_at(self.step)
        for g in self.opt.param_groups:
            g["lr"] = lr
        self.model.train()
        if self.off_opt is not None:
            self.off_opt.begin_step()
        t0 = time.perf_counter()
        total = None
        for m in range(tc.grad_accum):
            ce = self._fwd_bwd_micro(m == tc.grad_accum - 1)
            total = ce if total is None else total + ce
        loss = total * (1.0 / tc.grad_accum)

        if self.use_ds:
            self.engine.step()
            gn_v = float(self.engine.get_global_grad_norm() or 0.0)
            lv, ok = float(loss), True
        else:
            if self.reducer is not None:
                self.reducer.finish()
            peer = getattr(self, "peer", False)
            if peer:
                # one kernel exchanges norm, loss and the finite flag with the peers and fills `ctl`
                stats = self.opt.reduce_step(self.reducer, loss, tc.grad_clip, tc.skip_nonfinite)
                gn, loss, flag = stats[0], stats[1], stats[2]
            else:
                native.sync_expert_grads(self.model, ctx, self._expert_params)
                tp_state = getattr(self.raw, "_fm_tp", None)
                if tp_state is not None and not isinstance(tp_state, str):
                    from .parallel import tp as fused_tp
                    fused_tp.sync_partial_grads(self.raw, tp_state)
                gn = self._clip().to(ctx.device)
                loss = self._reduce_loss(loss)
                if tc.skip_nonfinite:
                    finite = (torch.isfinite(gn) & torch.isfinite(loss)).to(torch.int32)
                else:
                    finite = torch.ones((), dtype=torch.int32, device=loss.device)
                flag = ctx.all_min_int(finite)
            early = self.store is not None and not (tc.skip_spike_factor > 0)
            if early:
                # the fused kernel reads the flag on the device: enqueue the update before the host read
                if not peer:
                    self.opt.ctl[1:2].copy_(flag.to(torch.float32).reshape(1))
                self._apply_update()
            # the single host synchronisation of the step
            if peer:
                gn_v, lv, flag_v, st_v = torch.cat([stats, self.store.symm.status.to(torch.float32)]).tolist()
                self.store.symm.check(int(st_v))
            else:
                flag_v, gn_v, lv = torch.stack([flag.to(torch.float32), gn.to(torch.float32), loss]).tolist()
            ok = flag_v > 0.5
            if tc.skip_spike_factor > 0 and self.loss_ema is not None and lv > tc.skip_spike_factor * self.loss_ema:
                ok = False
            if ok:
                if not early:
                    if self.store is not None:
                        self.opt.ctl[1:2].fill_(1.0)
                    self._apply_update()
                self.loss_ema = lv if self.loss_ema is None else 0.98 * self.loss_ema + 0.02 * lv
            else:
                self.skipped += 1
                if early and isinstance(getattr(self.opt, "steps", None), int):
                    self.opt.steps -= 1            # the kernel left everything untouched
            self.opt.zero_grad(set_to_none=True)

        dt = time.perf_counter() - t0
        tokens = self.micro_batch * (self.seq or 0) * tc.grad_accum * ctx.dp_world
        out = {"step": self.step + 1, "loss": lv, "lr": lr, "grad_norm": gn_v, "dt": dt, "skipped": self.skipped}
        if self.seq:
            out["tok_s"] = tokens / dt
        if self.peak_flops and hasattr(self.raw, "flops_per_token") and self.seq:
            out["mfu"] = tokens * self.raw.flops_per_token(self.seq) / dt / (self.peak_flops * ctx.world)
        if ctx.device.type == "cuda":
            out["mem_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
        self.step += 1
        return out

    def _apply_update(self) -> None:
        muon = getattr(self, "_muon_opt", None)
        if muon is not None:
            for g in muon.param_groups:
                if not g["use_muon"]:
                    g["lr"] = self.opt.param_groups[0]["lr"]
            muon.step()
        else:
            self.opt.step()

    def _reduce_loss(self, loss):
        loss = loss.to(torch.float32)
        if self.cfg.parallel.pp > 1:
            loss = self.ctx.sum_over_pp(loss)
        return self.ctx.mean_over_dp(loss)

    # ------------------------------------------------------------------ evaluation / fit
    @torch.no_grad()
    def evaluate(self):
        if self.eval_dl is None or self.cfg.parallel.pp > 1 or self.use_ds:
            return None
        self.model.eval()
        acc, n = torch.zeros((), device=self.ctx.device), 0
        loader = async_loader(self.eval_dl, self.ctx.device, depth=2) if self.cfg.train.prefetch else self.eval_dl
        try:
            for i, batch in enumerate(loader):
                if i >= self.cfg.train.eval_steps:
                    break
                with self._autocast(), self.quant.autocast():
                    ce, _ = self.model(batch["input_ids"].to(self.ctx.device), labels=batch["labels"].to(self.ctx.device))
                acc += ce.float()
                n += 1
        finally:
            if hasattr(loader, "close"):
                loader.close()
            self.model.train()
        return float(self.ctx.mean_over_dp(acc / max(n, 1)))

    def close(self) -> None:
        feed = getattr(self, "feed", None)
        if feed is not None:
            feed.close()

    def __del__(self):  # pragma: no cover
        with contextlib.suppress(Exception):
            self.close()

    def fit(self):
        tc, ctx = self.cfg.train, self.ctx
        while self.step < tc.max_steps:
            m = self.train_step()
            self.history.append(m)
            if self.step % tc.log_every == 0 or self.step == 1:
                bits = [f"step {m['step']:>6}", f"loss {m['loss']:.4f}", f"lr {m['lr']:.2e}",
                        f"gnorm {m['grad_norm']:.2f}"]
                if "tok_s" in m:
                    bits.append(f"{m['tok_s']:,.0f} tok/s")
                tail = f"{m['dt'] * 1000:.0f} ms"
                if "mfu" in m:
                    tail += f" mfu {m['mfu'] * 100:.1f}%"
                if "mem_gb" in m:
                    tail += f" mem {m['mem_gb']:.1f}G"
                bits.append(tail)
                if self.skipped:
                    bits.append(f"skipped {self.skipped}")
                log(ctx, " | ".join(bits))
            if tc.eval_every and self.step % tc.eval_every == 0:
                ev = self.evaluate()
                if ev is not None:
                    log(ctx, f"step {self.step:>6} | eval loss {ev:.4f} | ppl {math.exp(min(ev, 20)):.2f}")
            for cb in self.callbacks:
                cb(self, m)
            if tc.ckpt_every and self.step % tc.ckpt_every == 0:
                self.save()
        if tc.ckpt_every:
            self.save()
        self.sync_params()
        return self.history

    # ------------------------------------------------------------------ checkpoints
    def _paths(self, step: int):
        root = self.cfg.train.ckpt_dir
        return root, os.path.join(root, f"step_{step:07d}")

    def _dcp_state(self):
        from torch.distributed.checkpoint.state_dict import get_state_dict
        opt = () if self.off_opt is not None or self.use_ds else self.opt
        if getattr(self, "peer", False):
            # sharded optimizer: every rank presents the whole state, as a replicated run would
            self.store.sync_master()
            self.opt.gather_full()
        return get_state_dict(self.model, opt)

    def sync_params(self) -> None:
        """Make the fp32 parameters complete on every rank (they are sharded between optimizer steps
        on the peer-memory engine; the bf16 working weights are always complete)."""
        if getattr(self, "peer", False):
            self.store.sync_master()

    def save(self, keep_last: int = 3) -> None:
        import torch.distributed.checkpoint as dcp
        root, path = self._paths(self.step)
        os.makedirs(path, exist_ok=True)
        if getattr(self.raw, "_fm_tp", None) is not None and self.ctx.pc.tp > 1:
            # the fused tensor-parallel blocks hold plain, already sharded tensors under the same keys on
            # every rank, which torch.distributed.checkpoint takes for replicas and writes once
            log(self.ctx, "[forgeminds_b200] warning: a checkpoint of fused tensor-parallel blocks keeps one rank's "
                          "shards only; run with parallel.fused_comm=False (DTensor) when the run must be resumed")
        if self.use_ds:
            self.engine.save_checkpoint(root, tag=f"step_{self.step:07d}")
        else:
            msd, osd = self._dcp_state()
            state = {"model": msd}
            if self.off_opt is None:
                state["optim"] = osd
            target = os.path.join(path, "dcp")
            shutil.rmtree(target, ignore_errors=True)
            dcp.save(state, checkpoint_id=target)
            if getattr(self, "peer", False):
                self.opt.release_full()
            if self.off_opt is not None:
                torch.save(self.off_opt.state_dict(), os.path.join(path, f"offopt_rank{self.ctx.rank}.pt"))
        meta = {"step": self.step, "epoch": self.epoch, "batches_in_epoch": self.batches_in_epoch,
                "loss_ema": self.loss_ema, "micro_batch": self.micro_batch}
        with open(os.path.join(path, f"meta_rank{self.ctx.rank}.json"), "w") as f:
            json.dump(meta, f)
        self.ctx.barrier()
        if self.ctx.rank == 0:
            with open(os.path.join(root, "latest"), "w") as f:
                f.write(os.path.basename(path))
            kept = sorted(d for d in os.listdir(root) if d.startswith("step_"))
            for old in kept[:-keep_last]:
                shutil.rmtree(os.path.join(root, old), ignore_errors=True)
        self.ctx.barrier()
        log(self.ctx, f"[forgeminds_b200] saved checkpoint {path}")

    def maybe_resume(self) -> None:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import set_state_dict
        root = self.cfg.train.ckpt_dir
        marker = os.path.join(root, "latest")
        if not os.path.exists(marker):
            return
        with open(marker) as f:
            path = os.path.join(root, f.read().strip())
        if self.use_ds:
            self.engine.load_checkpoint(root, tag=os.path.basename(path))
        else:
            msd, osd = self._dcp_state()
            state = {"model": msd}
            if self.off_opt is None:
                state["optim"] = osd
            dcp.load(state, checkpoint_id=os.path.join(path, "dcp"))
            if self.off_opt is not None:
                set_state_dict(self.model, (), model_state_dict=state["model"], optim_state_dict={})
                self.off_opt.load_state_dict(torch.load(os.path.join(path, f"offopt_rank{self.ctx.rank}.pt"),
                                                        map_location="cpu", weights_only=False))
            else:
                set_state_dict(self.model, self.opt, model_state_dict=state["model"], optim_state_dict=state["optim"])
            if getattr(self, "peer", False):
                self.opt.scatter_full()
            if self.store is not None:
                self.store.refresh_shadow()
        with open(os.path.join(path, f"meta_rank{self.ctx.rank}.json")) as f:
            meta = json.load(f)
        self.step, self.loss_ema = meta["step"], meta["loss_ema"]
        self.feed.resume(meta["epoch"], meta["batches_in_epoch"])
        log(self.ctx, f"[forgeminds_b200] resumed from {path} at step {self.step}")
