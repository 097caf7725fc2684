"""Config-driven training loop with one host<->device synchronisation per optimizer step.

``Trainer`` is the façade: it builds the process groups, the model and the data stream, owns the
schedule, the skip logic, logging and checkpoints, and hands the device work to one of two engines
(:mod:`forgeminds_b200.engine`):

* **native** (CUDA + bf16 on a B200) -- blocks on the sm_100a kernels, parameters in a flat store,
  gradient buckets reduced over peer memory while the backward is still running, clipping + AdamW +
  the bf16 weight refresh in one kernel that reads its clip coefficient and apply flag from device
  memory, for every mesh of pipeline x data (sharded, replicated or both) x tensor parallelism;
* **library** -- ``torch`` FSDP2 / DDP / DTensor with ``torch.optim`` (CPU, Gloo, fp32, offloaded or
  8-bit optimizer state, ``torch.compile``, DeepSpeed).

Public behaviour follows the reference's ``forgemind/trainer.py:41-459``: the constructor, the set-up
order (quantisation -> tensor parallel -> activation checkpointing / offload -> fused ops -> cache
warm-up -> compile -> data-parallel wrapper -> optimizer -> data -> pipeline -> resume), the cosine
schedule with linear warm-up, the unanimous non-finite / loss-spike skip, the metric dictionary of
``train_step`` and the checkpoint layout.
"""
from __future__ import annotations

import contextlib
import math
import os
import shutil
import time
from typing import Callable, Optional

import torch
import torch.nn as nn
from torch.utils.data import Dataset

from .config import ForgeConfig
from .data import BatchStream, async_loader, build_loader
from .distributed import DistContext, init_distributed, log
from .engine import checkpoint as ckpt
from .engine import choose as choose_engine
from .loss import logits_cross_entropy
from .offload import apply_activation_offload
from .parallel import native as wrappers
from .parallel.ac import apply_activation_checkpointing
from .parallel.pipeline import PipelineRunner
from .perf import enable_fast_math, warn_once
from .quant import QuantState, quantize_model

EMA_KEEP = 0.98          # weight of the old value in the loss average that the spike guard compares with


def moe_kwargs(ctx: DistContext, cfg: ForgeConfig) -> dict:
    """Keyword arguments for ``GPT(cfg, moe_kwargs=...)`` that wire expert parallelism / offload."""
    return {"ep_size": ctx.pc.ep, "ep_group": ctx.ep_group, "ep_rank": ctx.ep_rank,
            "offload_experts": cfg.offload.experts}


class _Both:
    """Two context managers entered as one (autocast + the quantisation back end's context)."""

    def __init__(self, outer, inner):
        self.pair = (outer, inner)

    def __enter__(self):
        self.pair[0].__enter__()
        self.pair[1].__enter__()

    def __exit__(self, *exc):
        self.pair[1].__exit__(*exc)
        self.pair[0].__exit__(*exc)


class Trainer:
    def __init__(self, model_fn: Callable[[DistContext], nn.Module], cfg: ForgeConfig, train_ds: Dataset,
                 eval_ds: Optional[Dataset] = None, micro_batch: int = 8, callbacks=(),
                 peak_flops: Optional[float] = None):
        self.cfg, self.micro_batch = cfg, micro_batch
        self.callbacks, self.peak_flops = list(callbacks), peak_flops
        tc, pc = cfg.train, cfg.parallel
        if hasattr(cfg, "check"):          # misspelt modes and meshes that do not multiply out are named here, by field
            cfg.check(int(os.environ.get("WORLD_SIZE", "1")))
        self.ctx = ctx = init_distributed(pc)
        self.use_ds = pc.backend == "deepspeed"
        self.engine_notes: list = []
        enable_fast_math(pc.backend == "native")

        model = self._build_model(model_fn)
        self.native = self._kernels_wanted(model)
        if not self.native:
            self._pin_to_torch(model)
        model = self._prepare_model(model)

        self.eng = choose_engine(self, model)
        self.model = self.eng.model
        self._open_data(train_ds, eval_ds)
        self.pp = self._pipeline() if pc.pp > 1 else None

        self.step, self.loss_ema, self.history, self.skipped = 0, None, [], 0
        self._banner()
        if tc.resume:
            self.maybe_resume()

    # ------------------------------------------------------------------ engine attributes, as the tools know them
    store = property(lambda self: getattr(self.eng, "store", None))
    reducer = property(lambda self: getattr(self.eng, "reducer", None))
    peer = property(lambda self: bool(getattr(self.eng, "peer", False)))
    opt = property(lambda self: self.eng.opt)
    off_opt = property(lambda self: getattr(self.eng, "off_opt", None))
    engine = property(lambda self: getattr(self.eng, "ds", None))          # the DeepSpeed engine, if any

    # ------------------------------------------------------------------ construction
    def _build_model(self, model_fn):
        tc, pc, ctx = self.cfg.train, self.cfg.parallel, self.ctx
        torch.manual_seed(tc.seed)
        model = model_fn(ctx)
        self.raw = model
        mcfg = getattr(model, "cfg", None)
        self.seq = getattr(mcfg, "max_seq", None)
        if pc.ep > 1:
            # each expert-parallel rank owns different experts: draw them from a rank-specific stream
            stream = torch.Generator().manual_seed(tc.seed + 1 + ctx.ep_rank)
            with torch.no_grad():
                for name, p in model.named_parameters():
                    if ".experts." in name:
                        p.copy_(torch.empty(p.shape).normal_(0, 0.02, generator=stream))
        if pc.pp > 1:
            model.split_stage(ctx.pp_rank, pc.pp)
            if getattr(mcfg, "n_experts", 0) and getattr(mcfg, "aux_coef", 0):
                log(ctx, "[forgeminds_b200] note: the MoE auxiliary loss stays on its own pipeline stage")
        return model.to(ctx.device)

    def _kernels_wanted(self, model) -> bool:
        """Whether the blocks of this model run on the sm_100a kernels."""
        tc, ctx = self.cfg.train, self.ctx
        if tc.native is False or not tc.bf16 or ctx.device.type != "cuda" or self.use_ds:
            return False
        from . import ops
        if not ops.available():
            if tc.native or torch.cuda.get_device_capability(ctx.device)[0] == 10:
                ops.require()            # a B200 without the extension is a build problem: say so
            return False
        return hasattr(model, "layers")

    @staticmethod
    def _pin_to_torch(model) -> None:
        mcfg = getattr(model, "cfg", None)
        if mcfg is not None and hasattr(mcfg, "native"):
            mcfg.native = False
        layers = getattr(model, "layers", None)
        for blk in (layers.values() if hasattr(layers, "values") else []):
            if hasattr(blk, "native"):
                blk.native = False

    def _prepare_model(self, model):
        cfg, ctx = self.cfg, self.ctx
        tc, pc, oc = cfg.train, cfg.parallel, cfg.offload
        if pc.ep > 1 and self.native and pc.fused_comm and pc.ep <= 8 and not oc.experts:
            from .parallel import ep as fused_ep            # dispatch / combine inside the permutation kernels
            fused_ep.attach(model, ctx)
        self.quant: QuantState = quantize_model(model, cfg.quant, ctx.dp_group)
        if pc.tp > 1:
            wrappers.apply_tp(model, ctx)
        if tc.ac != "none":
            apply_activation_checkpointing(model, tc.ac, preserve_rng_state=tc.ac_preserve_rng)
        if oc.activations and ctx.device.type == "cuda":
            apply_activation_offload(model, oc)
        if tc.fused_ops:
            from .kernels import available as kernels_available
            from .kernels.apply import enable as patch_kernels
            done = patch_kernels(model, norm=True, swiglu_mlp=True, split=tc.fused_split_mlp)._fm_fused
            warn_once(f"[forgeminds_b200] fused_ops: {done['norm']} norm and {done['mlp']} MLP modules now call "
                      f"forgeminds_b200.kernels (sm_100a kernels available: {kernels_available()})", key="fused_ops")
        warm = getattr(model, "prepare", None)
        if warm is not None:
            try:
                warm(device=ctx.device, dtype=torch.bfloat16 if tc.bf16 else torch.float32, seq=self.seq)
            except TypeError:
                warm()
        if tc.compile:
            self._compile_blocks(model)
        if not any(p.requires_grad for p in model.parameters()):
            raise RuntimeError("[forgeminds_b200] no trainable parameters -- every parameter is frozen "
                               "(int8_wo freezes the base weights: add adapters or unfreeze something)")
        return model

    def _compile_blocks(self, model) -> None:
        tc = self.cfg.train
        options = {"mode": tc.compile_mode, "fullgraph": tc.compile_fullgraph, "backend": tc.compile_backend}
        layers = getattr(model, "layers", None)
        blocks = list(layers.values()) if hasattr(layers, "values") else list(layers or [])
        if not blocks:
            model.compile(**options)
            return
        for blk in blocks:
            if tc.compile_fullgraph and getattr(blk, "is_moe", False) and \
                    not getattr(blk.ffn, "compile_friendly", True):
                raise RuntimeError("compile_fullgraph=True is not possible for this MoE block: its dispatch needs a "
                                   "host read on this device")
            blk.compile(**options)

    def _open_data(self, train_ds, eval_ds) -> None:
        tc, ctx = self.cfg.train, self.ctx
        self.train_dl, self.sampler = build_loader(train_ds, self.micro_batch, ctx, tc.seed, workers=tc.workers)
        self.feed = BatchStream(self.train_dl, self.sampler, ctx.device, prefetch=tc.prefetch,
                                depth=tc.prefetch_depth, threaded=tc.batch_thread)
        self.eval_dl = None
        if eval_ds is not None:
            self.eval_dl = build_loader(eval_ds, self.micro_batch, ctx, tc.seed, workers=0, shuffle=False)[0]

    def _pipeline(self) -> PipelineRunner:
        pc = self.cfg.parallel
        if self.micro_batch % pc.pp_microbatches:
            raise AssertionError("micro_batch must be divisible by pp_microbatches")
        fused_head = self.eng.name == "native" and hasattr(self.raw, "lm_head")
        return PipelineRunner(self.model, self.ctx, logits_cross_entropy, pc.pp_microbatches, pc.pp_schedule,
                              fwd_ctx=lambda: _Both(self._autocast(), self.quant.autocast()),
                              grad_sync=self.eng.sync_scope, labels_in_model=fused_head)

    def _banner(self) -> None:
        pc, ctx = self.cfg.parallel, self.ctx
        n_local = sum(p.numel() for p in self.raw.parameters())
        log(ctx, f"[forgeminds_b200] world={ctx.world} mesh(pp,dp_rep,dp_shard,tp)=({pc.pp},{pc.dp_replicate},"
                 f"{pc.dp_shard},{pc.tp}) ep={pc.ep} engine={self.eng.name}"
                 f"{'+peer' if self.peer else ''} quant={self.cfg.quant.mode}/{self.quant.backend} "
                 f"params(local)={n_local / 1e6:.1f}M device={ctx.device}")
        for why in self.engine_notes:
            log(ctx, f"[forgeminds_b200]   library engine because: {why}")

    # ------------------------------------------------------------------ pieces the engines call back into
    def _muon(self, model, tc):
        """Muon on the 2-D weights of the blocks, AdamW on everything else."""
        from .muon import Muon
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        matrices = [p for n, p in named if p.ndim >= 2 and ".layers." in f".{n}"]
        taken = {id(p) for p in matrices}
        others = [p for _, p in named if id(p) not in taken]
        spec = [{"params": matrices, "use_muon": True, "lr": tc.muon_lr, "momentum": tc.muon_momentum,
                 "ns_steps": tc.muon_ns_steps, "weight_decay": tc.weight_decay}]
        if others:
            spec.append({"params": others, "use_muon": False, "lr": tc.lr, "betas": tc.betas, "eps": tc.eps,
                         "weight_decay": 0.0})
        return Muon(spec, lr=tc.muon_lr, group=self.ctx.dp_group if self.ctx.dp_world > 1 else None)

    def _schedule_muon(self, opt, lr: float) -> None:
        """The AdamW groups follow the schedule; the Muon groups follow its shape, scaled to ``muon_lr``."""
        tc = self.cfg.train
        shape = lr / tc.lr if tc.lr else 1.0
        for g in opt.param_groups:
            g["lr"] = tc.muon_lr * shape if g.get("use_muon") else lr

    @staticmethod
    def _param_groups(params, tc) -> list:
        """Weight decay on matrices only (``forgemind/trainer.py:103-107``)."""
        split = {True: [], False: []}
        for p in params:
            split[p.ndim >= 2].append(p)
        out = []
        if split[True]:
            out.append({"params": split[True], "weight_decay": tc.weight_decay})
        if split[False]:
            out.append({"params": split[False], "weight_decay": 0.0})
        return out

    def _autocast(self):
        if self.cfg.train.bf16 and self.ctx.device.type in ("cuda", "cpu"):
            return torch.autocast(self.ctx.device.type, dtype=torch.bfloat16)
        return contextlib.nullcontext()

    def _clip(self):
        """Global gradient norm (0-dim fp32 device tensor). The library engine scales the gradients in
        place; the native engine stores the coefficient for its optimizer kernel."""
        return self.eng.clip()

    def _reduce_loss(self, loss):
        loss = loss.to(torch.float32)
        if self.cfg.parallel.pp > 1:
            loss = self.ctx.sum_over_pp(loss)
        return self.ctx.mean_over_dp(loss)

    @property
    def epoch(self):
        return self.feed.epoch

    @property
    def batches_in_epoch(self):
        return self.feed.batches

    def lr_at(self, step: int) -> float:
        """Linear warm-up, then a cosine from ``lr`` down to ``min_lr_ratio * lr`` at ``max_steps``."""
        tc = self.cfg.train
        if step < tc.warmup_steps:
            return tc.lr * (step + 1) / tc.warmup_steps
        progress = (step - tc.warmup_steps) / max(1, tc.max_steps - tc.warmup_steps)
        cosine = 0.5 * (1.0 + math.cos(math.pi * min(1.0, progress)))
        return tc.lr * (tc.min_lr_ratio + (1.0 - tc.min_lr_ratio) * cosine)

    # ------------------------------------------------------------------ one optimizer step
    def train_step(self) -> dict:
        tc, ctx, eng = self.cfg.train, self.ctx, self.eng
        lr = self.lr_at(self.step)
        self.model.train()
        eng.begin_step(lr)
        started = time.perf_counter()
        running = None
        for k in range(tc.grad_accum):
            ids, y = self.feed.next()
            ce = eng.micro_step(ids, y, last=(k == tc.grad_accum - 1))
            running = ce if running is None else running + ce
        loss = running / tc.grad_accum

        if self.use_ds:
            norm_v, loss_v = eng.ds_step(loss)
        else:
            verdict, early = eng.settle(loss)
            values = verdict.tolist()                     # the step's only host synchronisation
            eng.check(values)
            flag_v, norm_v, loss_v = values[:3]
            go = flag_v > 0.5
            if go and tc.skip_spike_factor > 0 and self.loss_ema is not None:
                go = not (loss_v > tc.skip_spike_factor * self.loss_ema)
            if go:
                if not early:
                    eng.approve()
                self.loss_ema = loss_v if self.loss_ema is None else EMA_KEEP * self.loss_ema + (1 - EMA_KEEP) * loss_v
            else:
                self.skipped += 1
                eng.rejected(early)
            eng.zero_grad()

        elapsed = time.perf_counter() - started
        self.step += 1
        report = {"step": self.step, "loss": loss_v, "lr": lr, "grad_norm": norm_v, "dt": elapsed,
                  "skipped": self.skipped}
        if self.seq:
            n_tok = self.micro_batch * self.seq * tc.grad_accum * ctx.dp_world
            report["tok_s"] = n_tok / elapsed
            if self.peak_flops and hasattr(self.raw, "flops_per_token"):
                report["mfu"] = n_tok * self.raw.flops_per_token(self.seq) / elapsed / (self.peak_flops * ctx.world)
        if ctx.device.type == "cuda":
            report["mem_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
        return report

    # ------------------------------------------------------------------ evaluation / fit
    @torch.no_grad()
    def evaluate(self):
        if self.eval_dl is None or self.cfg.parallel.pp > 1 or self.use_ds:
            return None
        tc, dev = self.cfg.train, self.ctx.device
        self.model.eval()
        batches = async_loader(self.eval_dl, dev, depth=2) if tc.prefetch else self.eval_dl
        total, seen = torch.zeros((), device=dev), 0
        try:
            for batch in batches:
                if seen >= tc.eval_steps:
                    break
                with self._autocast(), self.quant.autocast():
                    ce, _ = self.model(batch["input_ids"].to(dev), labels=batch["labels"].to(dev))
                total += ce.float()
                seen += 1
        finally:
            if hasattr(batches, "close"):
                batches.close()
            self.model.train()
        return float(self.ctx.mean_over_dp(total / max(seen, 1)))

    def close(self) -> None:
        feed = getattr(self, "feed", None)
        if feed is not None:
            feed.close()

    def __del__(self):  # pragma: no cover
        with contextlib.suppress(Exception):
            self.close()

    def _log_step(self, m: dict) -> None:
        parts = [f"step {m['step']:>6}", f"loss {m['loss']:.4f}", f"lr {m['lr']:.2e}", f"gnorm {m['grad_norm']:.2f}"]
        if "tok_s" in m:
            parts.append(f"{m['tok_s']:,.0f} tok/s")
        parts.append(f"{m['dt'] * 1e3:.0f} ms" + (f" mfu {m['mfu'] * 100:.1f}%" if "mfu" in m else "")
                     + (f" mem {m['mem_gb']:.1f}G" if "mem_gb" in m else ""))
        if self.skipped:
            parts.append(f"skipped {self.skipped}")
        log(self.ctx, " | ".join(parts))

    def fit(self):
        tc = self.cfg.train
        while self.step < tc.max_steps:
            m = self.train_step()
            self.history.append(m)
            if self.step == 1 or self.step % tc.log_every == 0:
                self._log_step(m)
            if tc.eval_every and self.step % tc.eval_every == 0:
                held_out = self.evaluate()
                if held_out is not None:
                    log(self.ctx, f"step {self.step:>6} | eval loss {held_out:.4f} | ppl {math.exp(min(held_out, 20)):.2f}")
            for cb in self.callbacks:
                cb(self, m)
            if tc.ckpt_every and self.step % tc.ckpt_every == 0:
                self.save()
        if tc.ckpt_every:
            self.save()
        self.sync_params()
        return self.history

    # ------------------------------------------------------------------ checkpoints
    def sync_params(self) -> None:
        """Make the fp32 parameters complete on every rank (between optimizer steps the peer-memory
        engine keeps each rank's shard of them current; the bf16 working weights are always whole)."""
        self.eng.sync_params()

    def _tp_mesh(self):
        if self.cfg.parallel.tp > 1 and self.ctx.mesh is not None and ckpt.shard_dims(self.raw):
            return self.ctx.mesh["tp"]
        return None

    def _dcp_state(self):
        msd, osd = self.eng.state_for_dcp()
        if self.cfg.parallel.pp > 1:
            osd = ckpt.stage_groups(osd, f"pp{self.ctx.pp_rank}")
        return ckpt.as_sharded(self.raw, msd, osd, self._tp_mesh())

    def save(self, keep_last: int = 3) -> None:
        import torch.distributed.checkpoint as dcp
        root = self.cfg.train.ckpt_dir
        path = ckpt.step_dir(root, self.step)
        os.makedirs(path, exist_ok=True)
        if self.use_ds:
            self.engine.save_checkpoint(root, tag=os.path.basename(path))
        else:
            msd, osd = self._dcp_state()
            state = {"model": msd} if self.off_opt is not None else {"model": msd, "optim": osd}
            target = os.path.join(path, "dcp")
            shutil.rmtree(target, ignore_errors=True)      # no stale shards of an earlier layout
            dcp.save(state, checkpoint_id=target)
            self.eng.after_save()
            if self.off_opt is not None:
                torch.save(self.off_opt.state_dict(), os.path.join(path, f"offopt_rank{self.ctx.rank}.pt"))
        ckpt.write_meta(path, self.ctx.rank, {"step": self.step, "epoch": self.epoch,
                                              "batches_in_epoch": self.batches_in_epoch,
                                              "loss_ema": self.loss_ema, "micro_batch": self.micro_batch})
        self.ctx.barrier()
        if self.ctx.rank == 0:
            ckpt.publish(root, path, keep_last)
        self.ctx.barrier()
        log(self.ctx, f"[forgeminds_b200] saved checkpoint {path}")

    def maybe_resume(self) -> None:
        import torch.distributed.checkpoint as dcp
        path = ckpt.newest(self.cfg.train.ckpt_dir)
        if path is None:
            return
        if self.use_ds:
            self.engine.load_checkpoint(self.cfg.train.ckpt_dir, tag=os.path.basename(path))
        else:
            msd, osd = self._dcp_state()
            state = {"model": msd} if self.off_opt is not None else {"model": msd, "optim": osd}
            dcp.load(state, checkpoint_id=os.path.join(path, "dcp"))
            loaded_opt = ckpt.as_local(state.get("optim", {}))
            if self.cfg.parallel.pp > 1:
                loaded_opt = ckpt.stage_groups(loaded_opt, f"pp{self.ctx.pp_rank}", restore=True)
            self.eng.load_from_dcp(ckpt.as_local(state["model"]), loaded_opt)
            if self.off_opt is not None:
                self.off_opt.load_state_dict(torch.load(os.path.join(path, f"offopt_rank{self.ctx.rank}.pt"),
                                                        map_location="cpu", weights_only=False))
        meta = ckpt.read_meta(path, self.ctx.rank)
        self.step, self.loss_ema = meta["step"], meta["loss_ema"]
        self.feed.resume(meta["epoch"], meta["batches_in_epoch"])
        log(self.ctx, f"[forgeminds_b200] resumed from {path} at step {self.step}")
