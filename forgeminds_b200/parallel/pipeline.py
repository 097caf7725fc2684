"""Pipeline-parallel runtime: GPipe and 1F1B schedules over point-to-point send/recv.

Each stage owns a contiguous slice of the layers (``GPT.split_stage``). Activations travel to the next
stage and gradients to the previous one with ``torch.distributed`` p2p (NCCL on GPUs, Gloo on CPU);
the loss lives on the last stage. Receives for the next micro-batch are posted before the current
one is computed (``irecv``), and sends are asynchronous and only waited for at the end of the step, so
transfers overlap compute. The first step exchanges a small header with the activation shape and
dtype; buffers are reused per micro-batch slot and re-armed when the batch shape changes. Same
contract as the reference's ``forgemind/parallel/pipeline.py:24-147``.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

_DTYPES = [torch.float32, torch.bfloat16, torch.float16]


class PipelineRunner:
    def __init__(self, model, ctx, loss_fn, n_microbatches, schedule="1f1b", fwd_ctx=contextlib.nullcontext):
        self.model, self.ctx, self.loss_fn = model, ctx, loss_fn
        self.M = int(n_microbatches)
        self.schedule, self.fwd_ctx = schedule, fwd_ctx
        self.stage, self.n_stages, self.group = ctx.pp_rank, ctx.pc.pp, ctx.pp_group
        self.is_first, self.is_last = self.stage == 0, self.stage == self.n_stages - 1
        self.prev = None if self.is_first else dist.get_global_rank(self.group, self.stage - 1)
        self.next = None if self.is_last else dist.get_global_rank(self.group, self.stage + 1)
        self.reset()
        self._seen_shape = None

    # ------------------------------------------------------------------ p2p plumbing
    def reset(self) -> None:
        """Forget the negotiated activation shape (called when the batch shape changes)."""
        self._in_meta = None          # (shape, dtype) arriving from the previous stage
        self._header_sent = False
        self._act_slots: dict = {}
        self._grad_slots: dict = {}

    def _send_header(self, t: torch.Tensor) -> None:
        h = torch.zeros(8, dtype=torch.long, device=self.ctx.device)
        h[0], h[1] = t.dim(), _DTYPES.index(t.dtype)
        h[2:2 + t.dim()] = torch.tensor(tuple(t.shape), dtype=torch.long)
        dist.send(h, self.next, group=self.group)
        self._header_sent = True

    def _recv_header(self) -> None:
        h = torch.zeros(8, dtype=torch.long, device=self.ctx.device)
        dist.recv(h, self.prev, group=self.group)
        vals = h.tolist()                      # once per (re)armed shape, not per step
        self._in_meta = (tuple(int(v) for v in vals[2:2 + int(vals[0])]), _DTYPES[int(vals[1])])

    def _slot(self, table: dict, i: int, shape, dtype) -> torch.Tensor:
        buf = table.get(i)
        if buf is None or tuple(buf.shape) != tuple(shape) or buf.dtype != dtype:
            buf = table[i] = torch.empty(tuple(shape), dtype=dtype, device=self.ctx.device)
        return buf

    def _post_act_recv(self, i: int):
        if self._in_meta is None:
            self._recv_header()
        buf = self._slot(self._act_slots, i, *self._in_meta)
        return buf, dist.irecv(buf, self.prev, group=self.group)

    # ------------------------------------------------------------------ one optimizer step
    def step(self, ids, y, last_sync: bool = True):
        M = self.M
        if ids.shape != self._seen_shape:
            self.reset()
            self._seen_shape = ids.shape
        xs, ys = ids.chunk(M), y.chunk(M)
        live = []            # (index, stage input, stage output or scaled loss), oldest first
        in_flight, keep_alive = [], []
        pending_in: dict = {}
        loss_acc = None
        has_no_sync = hasattr(self.model, "no_sync")
        is_sharded = hasattr(self.model, "set_requires_gradient_sync") and not has_no_sync

        def prefetch(i):
            if not self.is_first and i < M and i not in pending_in:
                pending_in[i] = self._post_act_recv(i)

        def forward(i):
            nonlocal loss_acc
            if self.is_first:
                inp = xs[i]
            else:
                prefetch(i)
                buf, req = pending_in.pop(i)
                req.wait()
                inp = buf.requires_grad_(True)
            prefetch(i + 1)                          # next micro-batch arrives while this one computes
            with self.fwd_ctx():
                out = self.model(inp)
            if self.is_last:
                loss = self.loss_fn(out, ys[i])
                part = loss.detach().float()
                loss_acc = part if loss_acc is None else loss_acc + part
                live.append((i, inp, loss / M))
            else:
                if not self._header_sent:
                    self._send_header(out)
                payload = out.detach().contiguous()
                keep_alive.append(payload)
                in_flight.append(dist.isend(payload, self.next, group=self.group))
                live.append((i, inp, out))

        def backward(final: bool):
            i, inp, out = live.pop(0)
            sync = final and last_sync
            if is_sharded:
                self.model.set_requires_gradient_sync(sync)
            guard = self.model.no_sync() if (has_no_sync and not sync) else contextlib.nullcontext()
            with guard:
                if self.is_last:
                    out.backward()
                else:
                    g = self._slot(self._grad_slots, i, out.shape, out.dtype)
                    dist.recv(g, self.next, group=self.group)
                    out.backward(g)
            if not self.is_first:
                gi = inp.grad.contiguous()
                keep_alive.append(gi)
                in_flight.append(dist.isend(gi, self.prev, group=self.group))
                inp.grad = None

        if self.schedule == "gpipe":
            for i in range(M):
                forward(i)
            for k in range(M):
                backward(k == M - 1)
        else:                                         # 1F1B
            warm = min(M, self.n_stages - self.stage - 1)
            for i in range(warm):
                forward(i)
            done = 0
            for i in range(warm, M):
                forward(i)
                backward(done == M - 1)
                done += 1
            while done < M:
                backward(done == M - 1)
                done += 1
        for req in in_flight:
            req.wait()
        if self.is_last and loss_acc is not None:
            return loss_acc / M
        return None
