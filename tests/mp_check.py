"""Multi-process checks, run under torchrun on CPU/Gloo (or NCCL when GPUs are visible):

    torchrun --standalone --local-addr 127.0.0.1 --nproc_per_node=2 tests/mp_check.py ddp
    torchrun --standalone --local-addr 127.0.0.1 --nproc_per_node=8 tests/mp_check.py 3d_full

Each scenario either trains (loss must drop, replicas must stay identical) or compares a parallel
layout against a single-process model built in the same process. Prints ``RESULT <name> ok``.
"""
import copy
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import forgeminds_b200 as fm  # noqa: E402


def _mc(**over):
    base = dict(vocab_size=256, dim=64, n_layers=4, n_heads=4, n_kv_heads=2, max_seq=32, native=False)
    base.update(over)
    return fm.GPTConfig(**base)


def _cfg(**par):
    cfg = fm.ForgeConfig()
    cfg.parallel.__dict__.update(par)
    cfg.train.__dict__.update(max_steps=25, bf16=False, log_every=1000, warmup_steps=3, lr=3e-3, resume=False,
                              prefetch=False)
    return cfg


def _train(cfg, mc, micro_batch=8, moe=False, steps=None):
    if steps:
        cfg.train.max_steps = steps
    ds = fm.SyntheticLM(mc.vocab_size, mc.max_seq, n=1024)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if moe else None), cfg, ds, micro_batch=micro_batch)
    hist = tr.fit()
    tr.close()
    return tr, hist


def _assert_drop(hist, factor=0.7):
    assert hist[-1]["loss"] < factor * hist[0]["loss"], (hist[0]["loss"], hist[-1]["loss"])


def _replicas_identical(tr, group=None):
    for p in tr.raw.parameters():
        if hasattr(p, "full_tensor"):
            continue
        ref = p.detach().clone()
        dist.broadcast(ref, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        assert torch.equal(ref, p.detach()), "replicas diverged"


def sc_ddp(world):
    tr, h = _train(_cfg(dp_replicate=world), _mc())
    _assert_drop(h)
    _replicas_identical(tr)


def sc_ddp_accum_offload(world):
    cfg = _cfg(dp_replicate=world)
    cfg.train.grad_accum = 2
    cfg.offload.optimizer, cfg.offload.smart = True, False
    tr, h = _train(cfg, _mc())
    _assert_drop(h)
    _replicas_identical(tr)


def sc_fsdp(world):
    _, h = _train(_cfg(dp_shard=world), _mc())
    _assert_drop(h)


def sc_fsdp_accum(world):
    cfg = _cfg(dp_shard=world)
    cfg.train.grad_accum = 2
    _, h = _train(cfg, _mc())
    _assert_drop(h)


def sc_hsdp(world):
    _, h = _train(_cfg(dp_replicate=2, dp_shard=world // 2), _mc())
    _assert_drop(h)


def sc_ep_ddp(world):
    tr, h = _train(_cfg(dp_replicate=world, ep=world), _mc(n_experts=4), moe=True)
    _assert_drop(h)


def sc_pp(world):
    cfg = _cfg(pp=world)
    cfg.parallel.pp_microbatches = 4
    _, h = _train(cfg, _mc())
    if dist.get_rank() == world - 1:
        _assert_drop(h)


def sc_tp(world):
    _, h = _train(_cfg(tp=world), _mc())
    _assert_drop(h)


def sc_tp_fsdp(world):
    _, h = _train(_cfg(tp=2, dp_shard=world // 2), _mc())
    _assert_drop(h)


def sc_pp_fsdp(world):
    cfg = _cfg(pp=2, dp_shard=world // 2)
    _, h = _train(cfg, _mc())
    if dist.get_rank() >= world // 2:
        _assert_drop(h)


def sc_3d_full(world):
    cfg = _cfg(pp=2, tp=2, dp_shard=world // 4)
    _, h = _train(cfg, _mc())
    if dist.get_rank() >= world // 2:
        _assert_drop(h)


# ---- equivalence against a single-process model --------------------------------------------
def sc_ep_equiv(world):
    ctx = fm.init_distributed(fm.ParallelConfig(dp_replicate=world, ep=world))
    torch.manual_seed(0)
    mc = _mc(n_experts=4, n_layers=1)
    full = fm.GPT(mc)                      # all experts on every rank
    cfg = _cfg(dp_replicate=world, ep=world)
    part = fm.GPT(mc, fm.moe_kwargs(ctx, cfg))
    sd = full.state_dict()
    n_local = 4 // world
    mine = {}
    for k, v in sd.items():
        mine[k] = v[ctx.ep_rank * n_local:(ctx.ep_rank + 1) * n_local].clone() if ".experts." in k else v.clone()
    part.load_state_dict(mine)
    g = torch.Generator().manual_seed(100 + ctx.rank)
    tok = torch.randint(0, 256, (2, 32), generator=g)
    # the single-process model sees the tokens of every rank
    gathered = [torch.empty_like(tok) for _ in range(world)]
    dist.all_gather(gathered, tok)
    loss_p, aux_p = part(tok, labels=tok)
    (loss_p + aux_p).backward()
    out_full = [full(t, labels=t) for t in gathered]
    loss_f = out_full[ctx.rank][0]
    assert torch.allclose(loss_p, loss_f, atol=1e-5), (loss_p.item(), loss_f.item())
    total = sum(l + a for l, a in out_full)
    total.backward()
    for (k, pp_), (_, pf) in zip(part.named_parameters(), full.named_parameters()):
        if ".experts." in k:
            want = pf.grad[ctx.ep_rank * n_local:(ctx.ep_rank + 1) * n_local]
            assert torch.allclose(pp_.grad, want, atol=1e-5), k


def sc_tp_equiv(world):
    ctx = fm.init_distributed(fm.ParallelConfig(tp=world))
    torch.manual_seed(0)
    mc = _mc(n_layers=2)
    single = fm.GPT(mc)
    par = copy.deepcopy(single)
    fm.parallel.native.apply_tp(par, ctx)
    tok = torch.randint(0, 256, (2, 32), generator=torch.Generator().manual_seed(5))
    ls, _ = single(tok, labels=tok)
    lp, _ = par(tok, labels=tok)
    assert torch.allclose(ls, lp, atol=1e-5)
    ls.backward()
    lp.backward()
    for (k, a), (_, b) in zip(single.named_parameters(), par.named_parameters()):
        gb = b.grad.full_tensor() if hasattr(b.grad, "full_tensor") else b.grad
        assert torch.allclose(a.grad, gb, atol=1e-5), k


def sc_pp_equiv(world):
    for schedule in ("gpipe", "1f1b"):
        pc = fm.ParallelConfig(pp=world, pp_schedule=schedule, pp_microbatches=4)
        ctx = fm.init_distributed(pc)
        torch.manual_seed(0)
        mc = _mc(n_layers=4)
        single = fm.GPT(mc)
        stage = copy.deepcopy(single).split_stage(ctx.pp_rank, world)
        from forgeminds_b200.loss import logits_cross_entropy
        runner = fm.parallel.PipelineRunner(stage, ctx, logits_cross_entropy, 4, schedule)
        tok = torch.randint(0, 256, (8, 32), generator=torch.Generator().manual_seed(7))
        loss = runner.step(tok, tok)
        ref = sum(single(t, labels=t)[0] for t in tok.chunk(4)) / 4
        ref.backward()
        if ctx.pp_rank == world - 1:
            assert torch.allclose(loss, ref.detach(), atol=1e-5), (loss.item(), ref.item())
        names = dict(single.named_parameters())
        for k, p in stage.named_parameters():
            assert torch.allclose(p.grad, names[k].grad, atol=1e-5), (schedule, k)


def sc_prefetch(world):
    """Threaded and serial batch streams hand every rank the same batches in the same order."""
    ctx = fm.init_distributed(fm.ParallelConfig(dp_replicate=world))
    ds = fm.SyntheticLM(128, 16, n=256)
    seen = {}
    for threaded in (False, True):
        dl, sampler = fm.build_loader(ds, 4, ctx, seed=9)
        s = fm.BatchStream(dl, sampler, ctx.device, threaded=threaded)
        seen[threaded] = torch.stack([s.next()[0] for _ in range(40)])
        s.close()
    assert torch.equal(seen[False], seen[True])
    mine = seen[True].reshape(-1, 16)[:, :4].contiguous()
    rows = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(rows, mine)
    assert not torch.equal(rows[0], rows[1])             # ranks read different shards


def sc_collectives(world):
    fm.init_distributed(fm.ParallelConfig(dp_replicate=world))
    r = dist.get_rank()
    t = torch.full((2,), float(r))
    assert fm.all_reduce(t.clone(), "sum")[0] == sum(range(world))
    assert fm.all_reduce(t.clone(), "max")[0] == world - 1
    assert torch.allclose(fm.all_reduce(t.clone(), "mean" if dist.get_backend() != "gloo" else "sum") /
                          (1 if dist.get_backend() != "gloo" else world), torch.full((2,), (world - 1) / 2))
    assert fm.all_gather(t).shape[0] == 2 * world
    b = torch.tensor([float(r)])
    fm.broadcast(b, src=1)
    assert b.item() == 1.0
    fm.barrier()


def sc_flat_pp_dp(world):
    """Flat-store engine under pipeline x data parallelism: every gradient bucket is reduced exactly once
    per optimizer step (from the last micro-batch's backward of the last accumulation step, never
    earlier), and the run equals the library engine's."""
    losses = {}
    for flat in (True, False):
        os.environ["FORGEMINDS_FLAT_ENGINE"] = "1" if flat else "0"
        cfg = _cfg(pp=2, **({"dp_shard": world // 2} if flat else {"dp_replicate": world // 2}))
        cfg.parallel.pp_microbatches = 4
        cfg.train.grad_accum = 2
        cfg.train.max_steps = 6
        mc = _mc()
        ds = fm.SyntheticLM(mc.vocab_size, mc.max_seq, n=1024)
        tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, ds, micro_batch=8)
        assert (tr.eng.name == "native") == flat
        launches = []
        if flat:
            real = tr.reducer.launch
            backwards = [0]
            scope = tr.eng.sync_scope

            def counted_scope(final, forward=False, _scope=scope):
                backwards[0] += 0 if forward else 1
                return _scope(final, forward)
            tr.pp.grad_sync = counted_scope

            def spy(bucket, _real=real):
                launches.append((bucket.name, backwards[0]))
                return _real(bucket)
            tr.reducer.launch = spy
        hist = []
        for _ in range(6):
            launches.clear()
            if flat:
                backwards[0] = 0
            hist.append(tr.train_step()["loss"])
            if flat:
                blocks = [b.name for b in tr.store.buckets if b.name.startswith("block")]
                assert sorted(n for n, _ in launches) == sorted(blocks), launches
                assert all(k == 2 * 4 for _, k in launches), launches       # the 8th backward of the step
        tr.close()
        losses[flat] = hist
    if dist.get_rank() >= world // 2:                 # the last stage holds the loss
        assert max(abs(a - b) for a, b in zip(losses[True], losses[False])) < 1e-4, losses


def sc_flat_ep(world):
    """Flat-store engine with expert parallelism: every rank's experts sit in buckets of their own that
    are scaled, not reduced, and the run equals the library engine's (DDP that ignores the experts +
    ``sync_expert_grads``)."""
    losses, norms = {}, {}
    for flat in (True, False):
        os.environ["FORGEMINDS_FLAT_ENGINE"] = "1" if flat else "0"
        cfg = _cfg(dp_replicate=world, ep=world)
        cfg.train.grad_accum = 2
        cfg.train.max_steps = 6
        mc = _mc(n_experts=4, n_layers=2)
        ds = fm.SyntheticLM(mc.vocab_size, mc.max_seq, n=1024)
        tr = fm.Trainer(lambda ctx: fm.GPT(mc, fm.moe_kwargs(ctx, cfg)), cfg, ds, micro_batch=8)
        assert (tr.eng.name == "native") == flat
        if flat:
            kinds = {b.name: b.local for b in tr.store.buckets}
            assert kinds == {"block0": False, "experts0": True, "block1": False, "experts1": True, "rest": False}, kinds
        hist = [tr.train_step() for _ in range(6)]
        tr.close()
        losses[flat], norms[flat] = [h["loss"] for h in hist], [h["grad_norm"] for h in hist]
    assert max(abs(a - b) for a, b in zip(losses[True], losses[False])) < 1e-4, losses
    assert max(abs(a - b) / b for a, b in zip(norms[True], norms[False])) < 1e-4, norms


def sc_pp_ckpt(world):
    """A pipeline-parallel run resumes from its checkpoint on both engines: every stage gets its own
    parameters, optimizer moments and param groups back and continues on the same trajectory."""
    import tempfile
    for flat in (True, False):
        os.environ["FORGEMINDS_FLAT_ENGINE"] = "1" if flat else "0"
        box = [tempfile.mkdtemp() if dist.is_initialized() and dist.get_rank() == 0 else None]
        if not dist.is_initialized():
            fm.init_distributed(fm.ParallelConfig(pp=world))
            box = [tempfile.mkdtemp() if dist.get_rank() == 0 else None]
        dist.broadcast_object_list(box, src=0)

        def build(resume):
            cfg = _cfg(pp=world)
            cfg.parallel.pp_microbatches = 2
            cfg.train.__dict__.update(max_steps=8, ckpt_dir=box[0], resume=resume, ckpt_every=0)
            mc = _mc()
            return fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(mc.vocab_size, mc.max_seq, n=1024), micro_batch=8)
        tr = build(False)
        for _ in range(3):
            tr.train_step()
        tr.save()
        again = build(True)
        assert again.step == 3
        assert all("weight_decay" in g for g in again.opt.param_groups)
        for _ in range(3):
            a, b = tr.train_step(), again.train_step()
            assert abs(a["loss"] - b["loss"]) < 1e-5 and abs(a["grad_norm"] - b["grad_norm"]) < 1e-4, (flat, a, b)
        tr.close()
        again.close()


def sc_tp_ckpt(world):
    """Plain tensors that hold one tensor-parallel slice per rank are stored as one sharded tensor and
    come back slice by slice (what the fused tensor-parallel blocks rely on for their checkpoints)."""
    import tempfile
    import torch.distributed.checkpoint as dcp
    from forgeminds_b200.engine import checkpoint as ckpt
    ctx = fm.init_distributed(fm.ParallelConfig(tp=world))
    rank = ctx.tp_rank
    torch.manual_seed(0)
    whole_col, whole_row, vec = torch.randn(8 * world, 6), torch.randn(5, 4 * world), torch.randn(6)

    def build(fill):
        m = torch.nn.Module()
        m.col = torch.nn.Parameter(whole_col[rank * 8:(rank + 1) * 8].clone() if fill else torch.zeros(8, 6))
        m.row = torch.nn.Parameter(whole_row[:, rank * 4:(rank + 1) * 4].clone() if fill else torch.zeros(5, 4))
        m.vec = torch.nn.Parameter(vec.clone() if fill else torch.zeros(6))
        m.col._tp_shard_dim, m.row._tp_shard_dim = 0, 1
        return m
    src = build(True)
    opt_state = {"state": {"col": {"exp_avg": src.col.detach() * 2, "step": torch.tensor(3.0)},
                           "vec": {"exp_avg": src.vec.detach() * 2, "step": torch.tensor(3.0)}}, "param_groups": []}
    msd, osd = ckpt.as_sharded(src, dict(src.named_parameters()), opt_state, ctx.mesh["tp"])
    assert tuple(msd["col"].shape) == (8 * world, 6) and tuple(msd["row"].shape) == (5, 4 * world)
    box = [tempfile.mkdtemp() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    dcp.save({"model": msd, "optim": osd}, checkpoint_id=box[0])
    dst = build(False)
    blank = {"state": {"col": {"exp_avg": torch.zeros(8, 6), "step": torch.tensor(0.0)},
                       "vec": {"exp_avg": torch.zeros(6), "step": torch.tensor(0.0)}}, "param_groups": []}
    msd2, osd2 = ckpt.as_sharded(dst, {k: v.detach() for k, v in dst.named_parameters()}, blank, ctx.mesh["tp"])
    state = {"model": msd2, "optim": osd2}
    dcp.load(state, checkpoint_id=box[0])
    local = ckpt.as_local(state)
    assert torch.equal(local["model"]["col"], src.col.detach()) and torch.equal(dst.col.detach(), src.col.detach())
    assert torch.equal(local["model"]["row"], src.row.detach())
    assert torch.equal(local["model"]["vec"], vec)
    assert torch.equal(local["optim"]["state"]["col"]["exp_avg"], src.col.detach() * 2)
    assert float(local["optim"]["state"]["col"]["step"]) == 3.0


SCENARIOS = {k[3:]: v for k, v in list(globals().items()) if k.startswith("sc_")}


def main():
    name = sys.argv[1]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    SCENARIOS[name](world)
    if dist.is_initialized():
        dist.barrier()
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"RESULT {name} ok", flush=True)
    fm.cleanup()


if __name__ == "__main__":
    main()
