"""Pipeline-parallel runtime: GPipe and 1F1B schedules over point-to-point send/recv.

Each stage owns a contiguous slice of the layers (``GPT.split_stage``). Activations travel to the next
stage and gradients to the previous one with ``torch.distributed`` p2p (NCCL on GPUs, Gloo on CPU);
the loss lives on the last stage. Same contract as the reference's
``forgemind/parallel/pipeline.py:24-147`` (header handshake once per batch shape, reusable buffers per
micro-batch slot, ``step`` returns the mean micro-batch loss on the last stage and ``None`` elsewhere).

Overlap. Sends are asynchronous and only waited for at the end of the step. Receives are posted ahead
of their use as early as the transport's ordering allows: a pair of ranks shares one NCCL stream for
both directions, so a receive must not be queued in front of a send that the peer needs before it can
produce the data to be received.

* activation of micro-batch ``i + 1``: posted before micro-batch ``i`` is computed (the previous stage
  sends activations in index order and needs nothing from this stage to produce them);
* gradient of micro-batch ``k``: while this stage still has activations to send, the receive is queued
  at the backward that consumes it -- queued any earlier it would sit in front of the next activation
  send on the shared stream and hold that send back until the gradient has arrived, which lengthens
  the next stage's critical path. The wait is a stream dependency, not a host block. Once this stage
  has sent its last activation (the whole backward phase of GPipe, the drain phase of 1F1B) the
  receives of all outstanding gradients are posted at once.

``grad_sync(final, forward=False)`` is a callable returning a context manager that brackets every
backward (and, with ``forward=True``, the forward of the same micro-batch); the training engine uses it
to let gradient reduction start only in the last micro-batch's backward of the last accumulation step
(DDP ``no_sync``, FSDP2 ``set_requires_gradient_sync``, or the flat-store engine's bucket hooks).
DDP decides at forward time whether the next backward reduces, which is why the forward is bracketed
too (see :func:`ddp_or_fsdp_scope`).
"""
from __future__ import annotations

import contextlib
from collections import deque

import torch
import torch.distributed as dist

_WIRE_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _no_sync_scope(model):
    """Default gradient-sync policy for torch wrappers (DDP / FSDP2) and plain modules."""
    ddp_like = hasattr(model, "no_sync")
    fsdp_like = hasattr(model, "set_requires_gradient_sync") and not ddp_like

    def scope(final: bool, forward: bool = False):
        return ddp_or_fsdp_scope(model, ddp_like, fsdp_like, final, forward)
    return scope


def ddp_or_fsdp_scope(model, ddp_like: bool, fsdp_like: bool, final: bool, forward: bool):
    """FSDP2 decides per backward. DDP arms its reducer at the end of a forward that runs outside
    ``no_sync`` and then reduces in whichever backward comes next -- under a pipeline schedule that is
    usually not the backward of the same micro-batch. So every forward runs under ``no_sync`` and the
    reducer is armed by hand right before the one backward that has to reduce."""
    if fsdp_like and not forward:
        model.set_requires_gradient_sync(final)
    if ddp_like:
        if forward or not final:
            return model.no_sync()
        model.reducer.prepare_for_backward([])
    return contextlib.nullcontext()


class PipelineRunner:
    def __init__(self, model, ctx, loss_fn, n_microbatches, schedule="1f1b", fwd_ctx=contextlib.nullcontext,
                 grad_sync=None, labels_in_model: bool = False):
        """``labels_in_model``: the last stage calls ``model(x, labels=y)`` and takes the first element of
        the result as the loss (a model whose head is fused with the cross-entropy never materialises the
        logits); otherwise ``loss_fn(model(x), y)``."""
        self.model, self.ctx, self.loss_fn = model, ctx, loss_fn
        self.labels_in_model = bool(labels_in_model)
        self.M = int(n_microbatches)
        self.schedule, self.fwd_ctx = schedule, fwd_ctx
        self.grad_sync = grad_sync or _no_sync_scope(model)
        self.stage, self.n_stages, self.group = ctx.pp_rank, ctx.pc.pp, ctx.pp_group
        self.is_first, self.is_last = self.stage == 0, self.stage == self.n_stages - 1
        self.prev = None if self.is_first else dist.get_global_rank(self.group, self.stage - 1)
        self.next = None if self.is_last else dist.get_global_rank(self.group, self.stage + 1)
        self._batch_shape = None
        self.reset()

    # ------------------------------------------------------------------ wire format
    def reset(self) -> None:
        """Forget the negotiated activation shape (called when the batch shape changes)."""
        self._arriving = None         # (shape, dtype) of what the previous stage sends
        self._announced = False
        self._act_buf: dict = {}
        self._grad_buf: dict = {}

    def _announce(self, t: torch.Tensor) -> None:
        head = [t.dim(), _WIRE_DTYPES.index(t.dtype), *t.shape]
        head += [0] * (8 - len(head))
        dist.send(torch.tensor(head, dtype=torch.long, device=self.ctx.device), self.next, group=self.group)
        self._announced = True

    def _learn_shape(self) -> None:
        head = torch.zeros(8, dtype=torch.long, device=self.ctx.device)
        dist.recv(head, self.prev, group=self.group)
        nd, code, *dims = head.tolist()                   # once per (re)armed shape, not per step
        self._arriving = (tuple(int(d) for d in dims[:int(nd)]), _WIRE_DTYPES[int(code)])

    def _buffer(self, pool: dict, i: int, shape, dtype) -> torch.Tensor:
        t = pool.get(i)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            t = pool[i] = torch.empty(tuple(shape), dtype=dtype, device=self.ctx.device)
        return t

    # ------------------------------------------------------------------ one optimizer step
    def step(self, ids, y, last_sync: bool = True):
        M = self.M
        if ids.shape != self._batch_shape:
            self.reset()
            self._batch_shape = ids.shape
        xs, ys = ids.chunk(M), y.chunk(M)
        sends, pinned = [], []                 # async sends and the tensors they read
        acts_in: dict = {}                     # micro-batch -> (buffer, request) of posted activation receives
        grads_in: dict = {}                    # micro-batch -> (buffer, request) of posted gradient receives
        open_mb: deque = deque()               # forwarded, not yet backwarded: (index, input, output-or-loss)
        awaiting_grad: deque = deque()         # micro-batches whose gradient receive is not posted yet
        loss_sum = None
        n_sent = 0

        def want_act(i):
            if self.is_first or i >= M or i in acts_in:
                return
            if self._arriving is None:
                self._learn_shape()
            buf = self._buffer(self._act_buf, i, *self._arriving)
            acts_in[i] = (buf, dist.irecv(buf, self.prev, group=self.group))

        def want_grads(upto: int):
            """Post the receives of the gradients of micro-batches <= ``upto`` (in order)."""
            while awaiting_grad and awaiting_grad[0][0] <= upto:
                k, shape, dtype = awaiting_grad.popleft()
                buf = self._buffer(self._grad_buf, k, shape, dtype)
                grads_in[k] = (buf, dist.irecv(buf, self.next, group=self.group))

        def forward(i):
            nonlocal loss_sum, n_sent
            if self.is_first:
                x = xs[i]
            else:
                want_act(i)
                buf, req = acts_in.pop(i)
                req.wait()
                x = buf.requires_grad_(True)
            want_act(i + 1)
            with self.fwd_ctx(), self.grad_sync(i == M - 1 and last_sync, forward=True):
                if self.is_last and self.labels_in_model:
                    out = self.model(x, labels=ys[i])
                else:
                    out = self.model(x)
            if self.is_last:
                loss = out[0] if self.labels_in_model else self.loss_fn(out, ys[i])
                piece = loss.detach().float()
                loss_sum = piece if loss_sum is None else loss_sum + piece
                open_mb.append((i, x, loss / M))
                return
            if not self._announced:
                self._announce(out)
            wire = out.detach().contiguous()
            pinned.append(wire)
            sends.append(dist.isend(wire, self.next, group=self.group))
            n_sent += 1
            open_mb.append((i, x, out))
            awaiting_grad.append((i, out.shape, out.dtype))
            if n_sent == M:                    # nothing of ours can queue up behind a receive any more
                want_grads(M)

        def backward(final: bool):
            i, x, out = open_mb.popleft()
            with self.grad_sync(final and last_sync):
                if self.is_last:
                    out.backward()
                else:
                    want_grads(i)
                    buf, req = grads_in.pop(i)
                    req.wait()
                    out.backward(buf)
            if not self.is_first:
                gx = x.grad.contiguous()
                pinned.append(gx)
                sends.append(dist.isend(gx, self.prev, group=self.group))
                x.grad = None

        warm = M if self.schedule == "gpipe" else min(M, self.n_stages - 1 - self.stage)
        for i in range(warm):
            forward(i)
        done = 0
        for i in range(warm, M):               # steady state of 1F1B (empty for GPipe)
            forward(i)
            backward(done == M - 1)
            done += 1
        while done < M:
            backward(done == M - 1)
            done += 1
        for req in sends:
            req.wait()
        if self.is_last and loss_sum is not None:
            return loss_sum / M
        return None
