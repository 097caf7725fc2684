"""Multi-GPU scenarios, one process per GPU, started by tests/test_gpu_multi.py through torchrun.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tests/mp_gpu_check.py <scenario>

Every scenario prints ``OK <scenario>`` on rank 0 when all ranks agree with the single-process
expectation. NVLink multicast stays off (plain peer loads and stores only).
"""
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import forgeminds_b200 as fm


def _init():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    return rank, world, torch.device("cuda", int(os.environ["LOCAL_RANK"]))


def _tiny(device):
    torch.manual_seed(0)
    cfg = fm.GPTConfig(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=128, ffn_hidden=384)
    return fm.GPT(cfg).to(device)


def peer_kernels():
    """reduce-scatter + norm exchange + sharded AdamW + push against all_reduce + the PyTorch AdamW."""
    from forgeminds_b200.parallel.flat import FlatParamStore, _adamw_reference
    from forgeminds_b200.parallel.peer import PeerAdamW, PeerReducer
    from forgeminds_b200.parallel.symm import SymmGroup
    rank, world, dev = _init()
    model = _tiny(dev)
    sg = SymmGroup(None, dev, timeout_ms=5000)
    store = FlatParamStore(model, dev, symm=sg)
    opt = PeerAdamW(store, lr=1e-2, weight_decay=0.1)
    red = PeerReducer(store)
    master0 = store.master.clone()
    exp_m = torch.zeros_like(master0)
    exp_v = torch.zeros_like(master0)
    exp_p = master0.clone()
    exp_sh = torch.zeros_like(store.shadow)
    for step in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        store.grad.copy_(torch.randn(store.total, device=dev, generator=g))
        want_g = store.grad.clone()
        dist.all_reduce(want_g)
        want_g /= world
        loss = torch.tensor(float(rank + step), device=dev)
        for b in store.buckets[:1]:
            red.launch(b)
        red.finish()
        stats = opt.reduce_step(red, loss, max_norm=1.0, skip_nonfinite=True)
        opt.param_groups[0]["lr"] = 1e-2
        opt.step()
        torch.cuda.synchronize()
        sg.check()
        norm = want_g.norm()
        coef = torch.clamp(1.0 / (norm + 1e-6), max=1.0)
        assert abs(stats[0].item() - norm.item()) < 1e-3 * norm.item(), (stats, norm)
        assert abs(stats[1].item() - (sum(range(world)) / world + step)) < 1e-5
        assert stats[2].item() == 1.0
        ctl = torch.stack([coef, torch.ones((), device=dev)])
        b1, b2 = 0.9, 0.95
        for b in store.buckets:
            for off, n, dec in opt._segments(b):
                lo = b.start + off
                _adamw_reference(exp_p[lo:lo + n], want_g[lo:lo + n], exp_m[lo:lo + n], exp_v[lo:lo + n],
                                 exp_sh[lo:lo + n], 1e-2, b1, b2, 1e-8, 0.1 if dec else 0.0, 1 - b1 ** (step + 1),
                                 1 - b2 ** (step + 1), ctl)
        # bf16 working weights are complete on every rank
        assert (store.shadow.float() - exp_sh.float()).abs().max() < 1e-3
        store.sync_master()
        assert (store.master - exp_p).abs().max() < 2e-5, (store.master - exp_p).abs().max()
    # the gathered optimizer state equals the replicated one
    opt.gather_full()
    full_m, full_v = opt._full
    assert (full_m - exp_m).abs().max() < 1e-5 and (full_v - exp_v).abs().max() < 1e-5
    sd = opt.state_dict()
    opt.release_full()
    opt.exp_avg.zero_()
    opt.load_state_dict(sd)
    opt.gather_full()
    for p in store.params:                     # the padding between parameters is not part of the state
        lo = store._offset[p]
        assert (opt._full[0][lo:lo + p.numel()] - exp_m[lo:lo + p.numel()]).abs().max() < 1e-5
    opt.release_full()
    dist.barrier()
    if rank == 0:
        print("OK peer_kernels", flush=True)


def peer_trainer():
    """The peer-memory engine follows the all_reduce engine step for step."""
    rank, world, dev = _init()
    losses = {}
    for fused in (True, False):
        cfg = fm.ForgeConfig()
        cfg.parallel.dp_shard = world
        cfg.parallel.fused_comm = fused
        cfg.train.__dict__.update(max_steps=12, grad_accum=2, lr=3e-3, warmup_steps=3, bf16=True, resume=False,
                                  log_every=1000, prefetch=False, ckpt_every=0)
        mc = fm.GPTConfig(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, max_seq=128, ffn_hidden=384)
        tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=512), micro_batch=4)
        assert tr.store is not None and bool(getattr(tr, "peer", False)) == fused
        hist = tr.fit()
        tr.close()
        losses[fused] = [h["loss"] for h in hist]
        norms = [h["grad_norm"] for h in hist]
        assert all(n > 0 for n in norms)
    a, b = losses[True], losses[False]
    assert a[-1] < 0.8 * a[0], a
    assert max(abs(x - y) for x, y in zip(a, b)) < 0.05, (a, b)
    if rank == 0:
        print("OK peer_trainer", flush=True)


def gemm_peer():
    """All-gather fused into the GEMM (rows pulled once into local memory by the kernel's gather warps),
    reduce-scatter fused into its epilogue (bf16 partial tiles stored into the owners' staging buffers)."""
    from forgeminds_b200 import ops
    from forgeminds_b200.parallel.symm import SymmGroup
    rank, world, dev = _init()
    C = ops.require()
    sg = SymmGroup(None, dev, timeout_ms=5000)
    slot = sg.reserve_slots(4)
    Ms, K, N = 256, 512, 384                       # per-rank rows, inner, output columns
    M = Ms * world

    def rand(shape, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        return (torch.randn(shape, device=dev, generator=g) * 0.5).to(torch.bfloat16)

    x_full = torch.cat([rand((Ms, K), 10 + r) for r in range(world)])      # every rank can rebuild every shard
    w = rand((N, K), 99 + rank)
    ready = torch.zeros(M // 128, dtype=torch.int32, device=dev)
    for trial in range(2):                                                  # twice: flags and buffers are reused
        buf = sg.alloc(M * K, torch.bfloat16)
        buf.local.view(M, K)[rank * Ms:(rank + 1) * Ms].copy_(x_full[rank * Ms:(rank + 1) * Ms])
        # 1. AG -> GEMM, gathered operand A (K-major): y = gather(x) @ w.T
        epoch = sg.next_epoch(slot)
        C.comm_signal(sg.flags.ptrs, slot, epoch, rank, sg.status)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        C.gemm_peer(buf.local.view(M, K), w, y, False, False, 1.0, False, rank, world, 1, buf.ptrs, ready, [],
                    sg.flags.local, slot, epoch, sg.timeout_ms, sg.status)
        want = x_full.float() @ w.float().T
        torch.cuda.synchronize()
        sg.check()
        assert (y.float() - want).abs().max() < 0.02 * want.abs().max(), (y.float() - want).abs().max()
        assert torch.equal(buf.local.view(M, K), x_full)                    # the rows are here now
        sg.barrier(slot + 1)
        # 2. gathered operand B (MN-major, reduction side): dw[N, K] = dy[M, N].T @ gather(x)[M, K]
        buf2 = sg.alloc(M * K, torch.bfloat16)
        buf2.local.view(M, K)[rank * Ms:(rank + 1) * Ms].copy_(x_full[rank * Ms:(rank + 1) * Ms])
        epoch = sg.next_epoch(slot)
        C.comm_signal(sg.flags.ptrs, slot, epoch, rank, sg.status)
        dy = rand((M, N), 7 + rank)
        dw = torch.empty(N, K, dtype=torch.float32, device=dev)
        C.gemm_peer(dy, buf2.local.view(M, K), dw, True, True, 1.0, False, rank, world, 2, buf2.ptrs, ready, [],
                    sg.flags.local, slot, epoch, sg.timeout_ms, sg.status)
        want = dy.float().T @ x_full.float()
        torch.cuda.synchronize()
        sg.check()
        assert (dw - want).abs().max() < 0.02 * want.abs().max()
        sg.barrier(slot + 1)
        # 3. gathered operand A, MN-major: dw2[K, N] = gather(x).T @ dy
        buf3 = sg.alloc(M * K, torch.bfloat16)
        buf3.local.view(M, K)[rank * Ms:(rank + 1) * Ms].copy_(x_full[rank * Ms:(rank + 1) * Ms])
        epoch = sg.next_epoch(slot)
        C.comm_signal(sg.flags.ptrs, slot, epoch, rank, sg.status)
        dw2 = torch.empty(K, N, dtype=torch.float32, device=dev)
        C.gemm_peer(buf3.local.view(M, K), dy, dw2, True, True, 1.0, False, rank, world, 1, buf3.ptrs, ready, [],
                    sg.flags.local, slot, epoch, sg.timeout_ms, sg.status)
        torch.cuda.synchronize()
        sg.check()
        assert (dw2 - want.T).abs().max() < 0.02 * want.abs().max()
        # 4. GEMM -> RS: the partial products of all ranks land, slice by slice, on the rank that owns the rows
        h = rand((M, K), 50 + rank)
        staging = sg.alloc(world * Ms * N, torch.bfloat16)
        sg.barrier(slot + 1)
        C.gemm_peer(h, w, staging.local.view(M, N), False, False, 1.0, False, rank, world, 0, [], None, staging.ptrs,
                    sg.flags.local, -1, 0, sg.timeout_ms, sg.status)
        sg.barrier(slot + 2)                           # all partial products have landed
        got = torch.empty(Ms, N, dtype=torch.bfloat16, device=dev)
        res = rand((Ms, N), 77)
        C.comm_sum_partials(staging.local, res, got, world)
        torch.cuda.synchronize()
        sg.check()
        want = sum(rand((M, K), 50 + r).float() @ rand((N, K), 99 + r).float().T for r in range(world))
        ref = want[rank * Ms:(rank + 1) * Ms] + res.float()
        assert (got.float() - ref).abs().max() < 0.03 * ref.abs().max(), (got.float() - ref).abs().max()
    dist.barrier()
    if rank == 0:
        print("OK gemm_peer", flush=True)


def ep_fused():
    """Expert-parallel MoE over peer memory against the same layer with all experts on one GPU."""
    import types
    from forgeminds_b200.moe import MoE
    from forgeminds_b200.parallel import ep as fused_ep
    rank, world, dev = _init()
    E, k, d, h, n = 8, 2, 256, 512, 1024
    for cap_factor, slot_factor in ((0.0, 0.0), (1.0, 0.0), (0.0, 1.5)):     # dropless, capacity, dropless in bounded buffers
        torch.manual_seed(3)
        whole = MoE(d, h, E, k, grouped_mm=True, capacity_factor=cap_factor).to(dev)
        part = MoE(d, h, E, k, grouped_mm=True, capacity_factor=cap_factor, ep_size=world, ep_rank=rank,
                   ep_group=dist.group.WORLD).to(dev)
        el = E // world
        with torch.no_grad():
            part.router.gate.weight.copy_(whole.router.gate.weight)
            for name in ("w1", "w3", "w2"):
                getattr(part.experts, name).copy_(getattr(whole.experts, name)[rank * el:(rank + 1) * el])
        ctx = types.SimpleNamespace(pc=types.SimpleNamespace(comm_timeout_ms=5000, ep_slot_factor=slot_factor),
                                    ep_group=dist.group.WORLD, device=dev)
        holder = torch.nn.ModuleList([part])
        fused_ep.attach(holder, ctx)
        for step in range(2):
            g = torch.Generator(device=dev).manual_seed(10 * step + rank)
            x = (torch.randn(n, d, device=dev, generator=g) * 0.5).to(torch.bfloat16).requires_grad_()
            xr = x.detach().clone().requires_grad_()
            go = (torch.randn(n, d, device=dev, generator=g)).to(torch.bfloat16)
            for m in (whole, part):
                m.zero_grad(set_to_none=True)
            out = part(x)
            want = whole(xr)
            torch.cuda.synchronize()
            holder._fm_ep.sg.check()
            if cap_factor == 0.0:                 # with a capacity the drop order differs between the two layouts
                assert (out.float() - want.float()).abs().max() < 0.05, (out.float() - want.float()).abs().max()
            (out.float() * go.float()).sum().backward()
            (want.float() * go.float()).sum().backward()
            torch.cuda.synchronize()
            holder._fm_ep.sg.check()
            if cap_factor > 0.0:
                continue
            assert (x.grad.float() - xr.grad.float()).norm() / xr.grad.float().norm() < 0.02
            a, b = part.router.gate.weight.grad.float(), whole.router.gate.weight.grad.float()
            assert (a - b).norm() / b.norm() < 0.02
            for name in ("w1", "w3", "w2"):
                full = getattr(whole.experts, name).grad.float().clone()
                dist.all_reduce(full)              # an expert sees the tokens of every rank
                mine = getattr(part.experts, name).grad.float()
                ref = full[rank * el:(rank + 1) * el]
                assert (mine - ref).norm() / ref.norm() < 0.02, name
    # buffers far too small for the routed rows: nothing is written out of bounds, the layer leaves its code in the
    # status word and the host learns of it where it reads the word
    from forgeminds_b200 import ops
    holder._fm_ep.slot_factor = 0.05
    x = (torch.randn(n, d, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
    out = part(x)
    out.float().sum().backward()
    torch.cuda.synchronize()
    try:
        holder._fm_ep.sg.check()
        raise AssertionError("the overflow was not reported")
    except ops.EPOverflow:
        pass
    assert torch.isfinite(out.float()).all() and torch.isfinite(x.grad.float()).all()
    holder._fm_ep.sg.check()                          # the word was cleared by the report
    dist.barrier()
    if rank == 0:
        print("OK ep_fused", flush=True)


def peer_failure():
    """Failures made on the host: a late rank is waited for; a rank that skips a launch makes the
    other rank's kernel give up after its limit, report, and leave the GPU usable."""
    import time
    from forgeminds_b200 import ops
    from forgeminds_b200.parallel.symm import SymmGroup
    rank, world, dev = _init()
    sg = SymmGroup(None, dev, timeout_ms=4000)
    slot = sg.reserve_slots(2)
    # 1. a delayed rank: the others wait (well inside the limit) and nobody reports anything
    if rank == world - 1:
        time.sleep(0.4)
    sg.barrier(slot)
    torch.cuda.synchronize()
    sg.check()
    dist.barrier()
    # 2. the last rank skips one launch: everybody else times out after 0.3 s and says so
    sg.timeout_ms = 300.0
    t0 = time.perf_counter()
    if rank != world - 1:
        sg.barrier(slot + 1)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.25 < waited < 3.0, waited
        try:
            sg.check()
        except ops.CommTimeout as e:
            assert "code 5" in str(e)
        else:
            raise AssertionError("the missing rank went unnoticed")
        assert int(ops.status_word(dev).item()) == 0                 # reading the status cleared it
        y = torch.arange(8, device=dev).float().sum()                # the context still works
        assert y.item() == 28.0
    dist.barrier()                                                   # NCCL is unaffected
    # 3. the skipped epoch is made up for and the protocol continues
    if rank == world - 1:
        sg._epochs[slot + 1] += 1
        ops.require().comm_signal(sg.flags.ptrs, slot + 1, sg._epochs[slot + 1], rank, sg.status)
    sg.timeout_ms = 4000.0
    sg.barrier(slot + 1)
    torch.cuda.synchronize()
    sg.check()
    dist.barrier()
    if rank == 0:
        print("OK peer_failure", flush=True)


def tp_grads():
    """Loss and every gradient of the sharded, sequence-parallel model equal those of the whole model."""
    import copy
    import types
    from forgeminds_b200.parallel import tp as fused_tp
    rank, world, dev = _init()
    torch.manual_seed(0)
    mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=2, n_heads=8, n_kv_heads=4, max_seq=128, ffn_hidden=512)
    whole = fm.GPT(mc).to(dev)
    part = copy.deepcopy(whole)
    ctx = types.SimpleNamespace(pc=types.SimpleNamespace(tp=world, comm_timeout_ms=5000), tp_rank=rank,
                                tp_group=dist.group.WORLD, device=dev)
    fused_tp.shard_model(part, ctx)
    g = torch.Generator(device=dev).manual_seed(5)
    tok = torch.randint(0, 512, (4, 128), device=dev, generator=g)
    lab = torch.randint(0, 512, (4, 128), device=dev, generator=g)
    for step in range(2):                       # twice: buffers and flags are reused
        for m in (whole, part):
            m.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss, _ = m(tok, labels=lab)
            loss.backward()
            m._last = loss.item()
        fused_tp.sync_partial_grads(part, part._fm_tp)
        torch.cuda.synchronize()
        part._fm_tp.sg.check()
        assert abs(whole._last - part._last) < 2e-2, (whole._last, part._last)
        full = dict(whole.named_parameters())
        for name, p in part.named_parameters():
            want = full[name].grad.float()
            dim = getattr(p, "_tp_shard_dim", None)
            if dim is not None:
                n = p.shape[dim]
                want = want.narrow(dim, rank * n, n)
            got = p.grad.float()
            rel = (got - want).norm() / want.norm().clamp(min=1e-6)
            assert rel < 2e-2, f"step {step} {name}: relative gradient error {rel.item():.3f}"
    dist.barrier()
    if rank == 0:
        print("OK tp_grads", flush=True)


def tp_fused():
    """Sequence-parallel blocks on the fused kernels follow the DTensor tensor-parallel run."""
    rank, world, dev = _init()
    losses = {}
    for fused in (True, False):
        cfg = fm.ForgeConfig()
        cfg.parallel.tp = world
        cfg.parallel.fused_comm = fused
        cfg.train.__dict__.update(max_steps=10, grad_accum=2, lr=1e-3, warmup_steps=3, bf16=True, resume=False,
                                  log_every=1000, prefetch=False, ckpt_every=0, native=None if fused else False)
        mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=2, n_heads=8, n_kv_heads=4, max_seq=128, ffn_hidden=512)
        tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=512), micro_batch=4)
        is_fused = not isinstance(getattr(tr.raw, "_fm_tp", "dtensor"), str)
        assert is_fused == fused, getattr(tr.raw, "_fm_tp", None)
        hist = tr.fit()
        tr.close()
        losses[fused] = [h["loss"] for h in hist]
    a, b = losses[True], losses[False]
    assert a[-1] < 0.85 * a[0], a
    assert max(abs(x - y) for x, y in zip(a[:4], b[:4])) < 0.03, (a, b)           # same trajectory at the start
    assert all(abs(x - y) < 0.02 + 0.02 * y for x, y in zip(a, b)), (a, b)        # two bf16 paths drift apart slowly
    if rank == 0:
        print("OK tp_fused", flush=True)


class _FixedFeed:
    """Hands the trainer the same batch at every call (each data-parallel rank has its own)."""

    def __init__(self, ids):
        self.ids = ids
        self.epoch, self.batches = 0, 0

    def next(self):
        return self.ids[:, :-1], self.ids[:, 1:]

    def close(self):
        pass

    def resume(self, *a):
        pass


def _mesh_equiv(world, rank, dev, label, check_ckpt=False, **par):
    """Gradients, global norm, losses and updates of the sm_100a engine on a mesh against a whole fp32
    PyTorch model that sees the batches of all data-parallel ranks."""
    import tempfile
    mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=4, n_heads=8, n_kv_heads=4, max_seq=128, ffn_hidden=512)
    cfg = fm.ForgeConfig()
    cfg.parallel.__dict__.update(par)
    box = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    cfg.train.__dict__.update(max_steps=8, grad_accum=1, lr=2e-3, warmup_steps=2, bf16=True, resume=False,
                              log_every=1000, prefetch=False, ckpt_every=0, ckpt_dir=box[0], grad_clip=1.0)
    if cfg.parallel.pp > 1:
        cfg.parallel.pp_microbatches = 2
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=64), micro_batch=4)
    ctx, eng, st = tr.ctx, tr.eng, tr.store
    assert eng.name == "native" and st is not None, label
    assert tr.peer, label
    # the oracle: same seed -> same initial weights, fp32 PyTorch operators, every data-parallel rank's batch
    torch.manual_seed(cfg.train.seed)
    oracle = fm.GPT(fm.GPTConfig(**{**mc.__dict__, "native": False})).to(dev)
    batches = [torch.randint(0, 512, (4, 129), device=dev, generator=torch.Generator(device=dev).manual_seed(40 + d))
               for d in range(ctx.dp_world)]
    tr.feed.close()
    tr.feed = _FixedFeed(batches[ctx.dp_rank])
    named = dict(oracle.named_parameters())
    decay = [p for p in oracle.parameters() if p.ndim >= 2]
    rest = [p for p in oracle.parameters() if p.ndim < 2]
    ref_opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}],
                                lr=2e-3, betas=cfg.train.betas, eps=cfg.train.eps)

    def oracle_step():
        ref_opt.zero_grad(set_to_none=True)
        loss = sum(oracle(b[:, :-1], labels=b[:, 1:])[0] for b in batches) / len(batches)
        loss.backward()
        return loss.item(), torch.nn.utils.get_total_norm([p.grad for p in oracle.parameters()]).item()

    # ---- one backward: every reduced gradient element that this rank owns
    want_loss, want_norm = oracle_step()
    ids, y = tr.feed.next()
    ce = eng.micro_step(ids, y, last=True)
    eng._sum_partial_grads()
    if eng.reducer is not None:
        eng.reducer.finish()
    torch.cuda.synchronize()
    expected = torch.zeros_like(st.grad)
    for name, p in tr.raw.named_parameters():
        g = named[name].grad.float()
        dim = getattr(p, "_tp_shard_dim", None)
        if dim is not None:
            g = g.narrow(dim, ctx.tp_rank * p.shape[dim], p.shape[dim])
        lo = st._offset[p]
        expected[lo:lo + p.numel()] = g.reshape(-1)
    worst = 0.0
    for b in st.buckets:
        lo, n = st.shard_range(b, st.layout.shard_rank)
        got, want = st.reduced_shard(b, st.layout.shard_rank), expected[lo:lo + n]
        if want.norm() == 0:
            continue
        rel = ((got - want).norm() / want.norm()).item()
        worst = max(worst, rel)
        assert rel < 2e-2, f"{label}: bucket {b.name}: relative gradient error {rel:.4f}"
    has_loss = cfg.parallel.pp == 1 or ctx.pp_rank == cfg.parallel.pp - 1
    if has_loss:
        mine = oracle(batches[ctx.dp_rank][:, :-1], labels=batches[ctx.dp_rank][:, 1:])[0].item()
        assert abs(ce.item() - mine) < 2e-2, (label, ce.item(), mine)
    eng.zero_grad()
    # ---- optimizer steps: global norm, mean loss and the trajectory
    for step in range(4):
        want_loss, want_norm = oracle_step()
        torch.nn.utils.clip_grad_norm_(oracle.parameters(), 1.0)
        for g in ref_opt.param_groups:
            g["lr"] = tr.lr_at(step)
        ref_opt.step()
        m = tr.train_step()
        assert m["skipped"] == 0, (label, m)
        assert abs(m["grad_norm"] - want_norm) < 2e-2 * want_norm, (label, step, m["grad_norm"], want_norm)
        assert abs(m["loss"] - want_loss) < 3e-2, (label, step, m["loss"], want_loss)
    if check_ckpt:
        tr.save()
        cfg.train.resume = True
        again = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=64), micro_batch=4)
        assert again.step == tr.step
        again.feed.close()
        again.feed = _FixedFeed(batches[ctx.dp_rank])
        a, b = tr.train_step(), again.train_step()
        assert abs(a["loss"] - b["loss"]) < 1e-3 and abs(a["grad_norm"] - b["grad_norm"]) < 1e-2 * a["grad_norm"], (a, b)
        a, b = tr.train_step(), again.train_step()         # the optimizer state came back too
        assert abs(a["loss"] - b["loss"]) < 2e-3, (label, a["loss"], b["loss"])
        again.close()
    tr.close()
    if rank == 0:
        print(f"  {label}: worst bucket gradient error {worst:.4f}", flush=True)


def mesh_equiv():
    """Every mesh the box has GPUs for, against the whole fp32 model (2 % on gradients and the norm)."""
    rank, world, dev = _init()
    if world == 2:
        _mesh_equiv(world, rank, dev, "dp_shard=2", dp_shard=2)
        _mesh_equiv(world, rank, dev, "tp=2", check_ckpt=True, tp=2)
        _mesh_equiv(world, rank, dev, "pp=2 (1f1b)", pp=2)
        _mesh_equiv(world, rank, dev, "pp=2 (gpipe)", pp=2, pp_schedule="gpipe")
    elif world == 4:
        _mesh_equiv(world, rank, dev, "dp_replicate=2 x dp_shard=2", check_ckpt=True, dp_replicate=2, dp_shard=2)
        _mesh_equiv(world, rank, dev, "tp=2 x dp_shard=2", tp=2, dp_shard=2)
        _mesh_equiv(world, rank, dev, "pp=2 x dp_shard=2", pp=2, dp_shard=2)
        _mesh_equiv(world, rank, dev, "pp=2 x tp=2", check_ckpt=True, pp=2, tp=2)
    else:
        _mesh_equiv(world, rank, dev, "pp=2 x dp_shard=2 x tp=2", check_ckpt=True, pp=2, dp_shard=world // 4, tp=2)
        _mesh_equiv(world, rank, dev, "dp_replicate=2 x dp_shard=4", dp_replicate=2, dp_shard=world // 2)
    if rank == 0:
        print("OK mesh_equiv", flush=True)


def muon_peer():
    """Owner-computes Muon over peer memory follows the replicated Muon (all_reduce of the gradients, every
    rank orthogonalising a share), and its sharded momentum survives a checkpoint."""
    import tempfile
    rank, world, dev = _init()
    box = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=2, n_heads=8, n_kv_heads=4, max_seq=128, ffn_hidden=512)
    losses = {}

    def build(fused, steps, resume=False):
        cfg = fm.ForgeConfig()
        cfg.parallel.dp_shard = world
        cfg.parallel.fused_comm = fused
        cfg.train.__dict__.update(max_steps=steps, grad_accum=2, lr=2e-3, warmup_steps=2, bf16=True, resume=resume,
                                  log_every=1000, prefetch=False, ckpt_every=0, ckpt_dir=box[0], optimizer="muon")
        return fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=512), micro_batch=4)

    for fused in (True, False):
        tr = build(fused, 10)
        assert tr.peer == fused and (type(tr.opt).__name__ == "PeerMuon") == fused, type(tr.opt).__name__
        if fused:
            owned = torch.tensor([len(tr.opt._mine)], device=dev)
            dist.all_reduce(owned)
            n_mat = sum(1 for n, p in tr.raw.named_parameters() if p.ndim >= 2 and "layers." in n)
            assert owned.item() == n_mat, (owned.item(), n_mat)          # every matrix has exactly one owner
        hist = [tr.train_step() for _ in range(6)]
        if fused:
            tr.save()
            again = build(True, 10, resume=True)
            assert again.step == 6
            a, b = tr.train_step(), again.train_step()
            assert abs(a["loss"] - b["loss"]) < 2e-3, (a["loss"], b["loss"])
            a, b = tr.train_step(), again.train_step()                  # ... and so did the momentum
            assert abs(a["loss"] - b["loss"]) < 4e-3, (a["loss"], b["loss"])
            again.close()
        tr.close()
        losses[fused] = [h["loss"] for h in hist]
        assert all(h["skipped"] == 0 for h in hist)
    a, b = losses[True], losses[False]
    assert a[-1] < 0.9 * a[0], a
    assert max(abs(x - y) for x, y in zip(a, b)) < 0.03, (a, b)
    if rank == 0:
        print("OK muon_peer", flush=True)


def ep_trainer():
    """Expert parallelism on the flat-store engine (experts in rank-local buckets, dense gradients through
    the peer reduce-scatter) follows the module engine (DDP that skips the experts + torch AdamW)."""
    rank, world, dev = _init()
    out = {}
    for flat in (True, False):
        os.environ["FORGEMINDS_FLAT_ENGINE"] = "" if flat else "0"
        cfg = fm.ForgeConfig()
        cfg.parallel.__dict__.update(dp_replicate=world, ep=world)
        cfg.train.__dict__.update(max_steps=8, grad_accum=2, lr=2e-3, warmup_steps=2, bf16=True, resume=False,
                                  log_every=1000, prefetch=False, ckpt_every=0)
        mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=2, n_heads=8, n_kv_heads=4, max_seq=128, ffn_hidden=512,
                          n_experts=2 * world, top_k=2, z_coef=0.0)
        tr = fm.Trainer(lambda ctx: fm.GPT(mc, fm.moe_kwargs(ctx, cfg)), cfg, fm.SyntheticLM(512, 128, n=512), micro_batch=4)
        assert (tr.eng.name == "native") == flat and tr.peer == flat, (tr.eng.name, tr.peer)
        assert getattr(tr.raw, "_fm_ep", None) is not None
        hist = tr.fit()
        tr.close()
        out[flat] = ([h["loss"] for h in hist], [h["grad_norm"] for h in hist])
    os.environ.pop("FORGEMINDS_FLAT_ENGINE", None)
    (la, na), (lb, nb) = out[True], out[False]
    assert la[-1] < 0.6 * la[0] and lb[-1] < 0.6 * lb[0], (la, lb)
    assert abs(na[0] - nb[0]) < 2e-2 * nb[0], (na, nb)                       # same gradient before the first update
    # the same trajectory while the routing agrees; a top-k choice that flips in one run sends the two apart
    assert max(abs(x - y) for x, y in zip(la[:3], lb[:3])) < 0.03, (la, lb)
    if rank == 0:
        print("OK ep_trainer", flush=True)


def _mesh_run(world, rank, label, steps=8, quant="none", optimizer="adamw", **par):
    cfg = fm.ForgeConfig()
    cfg.parallel.__dict__.update(par)
    cfg.quant.mode = quant
    cfg.train.__dict__.update(max_steps=steps, grad_accum=2, lr=2e-3, warmup_steps=2, bf16=True, resume=False,
                              log_every=1000, prefetch=False, ckpt_every=0, optimizer=optimizer)
    mc = fm.GPTConfig(vocab_size=512, dim=256, n_layers=4, n_heads=8, n_kv_heads=4, max_seq=128, ffn_hidden=512)
    tr = fm.Trainer(lambda ctx: fm.GPT(mc), cfg, fm.SyntheticLM(512, 128, n=1024), micro_batch=4)
    hist = tr.fit()
    tr.close()
    losses = [h["loss"] for h in hist]
    assert all(l == l for l in losses), (label, losses)
    assert losses[-1] < 0.9 * losses[0], (label, losses)
    if rank == 0:
        print(f"  {label}: engine={'native' if tr.store is not None else 'library'} "
              f"loss {losses[0]:.3f} -> {losses[-1]:.3f}", flush=True)
    return tr


def mesh_smoke():
    """Every mesh / feature combination that the box has GPUs for trains a small model for a few steps."""
    rank, world, dev = _init()
    _mesh_run(world, rank, f"dp_shard={world}", dp_shard=world)
    _mesh_run(world, rank, f"dp_replicate={world}", dp_replicate=world)
    _mesh_run(world, rank, f"dp_shard={world} + fp8", quant="fp8", dp_shard=world)
    _mesh_run(world, rank, f"dp_shard={world} + int8 + muon", quant="int8", optimizer="muon", dp_shard=world)
    _mesh_run(world, rank, f"pp=2 x dp_shard={world // 2}", pp=2, dp_shard=world // 2, pp_microbatches=2)
    _mesh_run(world, rank, f"tp=2 x dp_shard={world // 2}", tp=2, dp_shard=world // 2)
    for mode in ("int8", "fp8"):          # quantised layers under tensor parallelism run their 8-bit products
        tr = _mesh_run(world, rank, f"tp=2 x dp_shard={world // 2} + {mode}", quant=mode, tp=2, dp_shard=world // 2)
        assert tr.store is not None and tr.raw._fm_tp.quant_calls > 0, mode
    if world >= 4:
        _mesh_run(world, rank, "dp_replicate=2 x dp_shard=2 (HSDP)", dp_replicate=2, dp_shard=world // 2)
        _mesh_run(world, rank, f"tp=2 x pp=2 x dp_shard={world // 4}", tp=2, pp=2, dp_shard=world // 4, pp_microbatches=2)
    if rank == 0:
        print("OK mesh_smoke", flush=True)


if __name__ == "__main__":
    name = sys.argv[1]
    globals()[name]()
    if dist.is_initialized():
        dist.destroy_process_group()
