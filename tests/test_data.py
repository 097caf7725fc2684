"""Batch pipeline: order, epoch bookkeeping, error forwarding, resume, thread hygiene."""
import threading
import time

import pytest
import torch
from torch.utils.data import Dataset

import forgeminds_b200 as fm
from forgeminds_b200.data import BatchStream, ResumableSampler, async_loader, build_loader, to_device


class Counting(Dataset):
    def __init__(self, n=40, fail_at=None, delay=0.0):
        self.n, self.fail_at, self.delay = n, fail_at, delay

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if self.fail_at is not None and i == self.fail_at:
            raise ValueError(f"bad sample {i}")
        if self.delay:
            time.sleep(self.delay)
        t = torch.full((4,), i, dtype=torch.long)
        return {"input_ids": t, "labels": t + 1}


class Ctx:
    def __init__(self, rank=0, world=1):
        self.dp_rank, self.dp_world, self.device = rank, world, torch.device("cpu")


def _stream(ds, threaded, bs=4, **kw):
    dl, sampler = build_loader(ds, bs, Ctx(), seed=3)
    return BatchStream(dl, sampler, torch.device("cpu"), threaded=threaded, **kw), dl


@pytest.mark.parametrize("threaded", [False, True])
def test_order_and_epochs_match_serial(threaded):
    s, dl = _stream(Counting(40), threaded)
    serial = []
    for epoch in range(2):
        dl.sampler.set_epoch(epoch)
        serial += [b["input_ids"][:, 0].tolist() for b in dl]
    got = [s.next()[0][:, 0].tolist() for _ in range(20)]
    assert got == serial
    assert (s.epoch, s.batches) == (2, 0)
    s.close()


def test_labels_travel_with_inputs_and_stats():
    s, _ = _stream(Counting(16), True, depth=3)
    ids, labels = next(s)
    assert torch.equal(labels, ids + 1)
    rep = s.report()
    assert rep["batches"] == 1 and rep["depth"] == 3 and rep["threaded"] is True
    s.close()
    s.close()


def test_errors_are_forwarded():
    s, _ = _stream(Counting(16, fail_at=5), True)
    with pytest.raises(ValueError, match="bad sample"):
        for _ in range(8):
            s.next()
    s.close()


def test_empty_loader_fails_at_construction():
    with pytest.raises(RuntimeError, match="no batches"):
        _stream(Counting(2), True, bs=4)


@pytest.mark.parametrize("threaded", [False, True])
def test_resume_is_exact(threaded):
    s, _ = _stream(Counting(40), threaded)
    seen = [s.next()[0][:, 0].tolist() for _ in range(14)]          # 10 batches per epoch: epoch 1, batch 4
    pos = (s.epoch, s.batches)
    s.close()
    t, _ = _stream(Counting(40), threaded)
    t.resume(*pos)
    cont = [t.next()[0][:, 0].tolist() for _ in range(8)]
    u, _ = _stream(Counting(40), threaded)
    full = [u.next()[0][:, 0].tolist() for _ in range(22)]
    assert full[:14] == seen and full[14:] == cont
    assert (t.epoch, t.batches) == (u.epoch, u.batches)
    t.close()
    u.close()


def test_no_thread_left_behind():
    before = {th.name for th in threading.enumerate()}
    s, _ = _stream(Counting(40), True)
    s.next()
    s.close()
    it = async_loader([torch.ones(2)] * 3, "cpu")
    assert len(list(it)) == 3
    time.sleep(0.05)
    after = {th.name for th in threading.enumerate() if th.name.startswith("fmb200")}
    assert not after - before


def test_overlap_hides_loader_latency():
    ds = Counting(32, delay=0.004)
    s, _ = _stream(ds, True, depth=4)
    t0 = time.perf_counter()
    for _ in range(6):
        s.next()
        time.sleep(0.02)            # the "training step"
    threaded = time.perf_counter() - t0
    s.close()
    u, _ = _stream(Counting(32, delay=0.004), False)
    t0 = time.perf_counter()
    for _ in range(6):
        u.next()
        time.sleep(0.02)
    serial = time.perf_counter() - t0
    u.close()
    assert threaded < 0.9 * serial


def test_sampler_shards_and_skips():
    a = list(ResumableSampler(10, 0, 2, seed=1))
    b = list(ResumableSampler(10, 1, 2, seed=1))
    assert len(a) == len(b) == 5 and not set(a) & set(b)
    s = ResumableSampler(10, 0, 2, seed=1)
    s.skip = 2
    assert len(s) == 3 and list(s) == a[2:] and s.skip == 0


def test_to_device_nested_and_token_file(tmp_path):
    import collections
    import numpy as np
    P = collections.namedtuple("P", "a b")
    out = to_device({"x": [torch.ones(1), (torch.zeros(1), 3)], "p": P(torch.ones(1), "s")}, torch.device("cpu"))
    assert isinstance(out["p"], P) and out["x"][1][1] == 3
    path = tmp_path / "tok.bin"
    np.arange(1000, dtype=np.uint16).tofile(path)
    tf = fm.TokenFile(str(path), seq=10)
    assert len(tf) == 99 and tf[2]["input_ids"].tolist() == list(range(20, 30)) and tf[2]["labels"][-1] == 30
    tf.close()
    syn = fm.SyntheticLM(100, 16, n=8)
    assert syn[0]["input_ids"].shape == (16,) and torch.equal(syn[0]["input_ids"][1:], syn[0]["labels"][:-1])


# ------------------------------------------------------------------ loader worker processes
def _worker_children():
    import psutil
    me = psutil.Process()
    return [c for c in me.children(recursive=True) if c.is_running() and c.status() != psutil.STATUS_ZOMBIE]


def _wait_gone(before, timeout=10.0):
    deadline = time.time() + timeout
    while time.time() < deadline:
        extra = [c for c in _worker_children() if c.pid not in before]
        if not extra:
            return []
        time.sleep(0.1)
    return extra


def test_loader_workers_are_one_persistent_pool_across_epochs():
    """``workers=2``: the same two processes serve every epoch (no respawn per epoch) and leave when the
    stream closes."""
    before = {c.pid for c in _worker_children()}
    dl, sampler = build_loader(Counting(32), 4, Ctx(), seed=1, workers=2)
    s = BatchStream(dl, sampler, torch.device("cpu"), threaded=True)
    pids = set()
    seen = []
    for _ in range(20):                                   # 8 batches per epoch: more than two epochs
        seen.append(s.next()[0][0, 0].item())
        pids |= {c.pid for c in _worker_children() if c.pid not in before}
    assert s.epoch >= 2
    assert len(pids) == 2, pids                           # one pool, reused
    s.close()
    del s, dl
    import gc
    gc.collect()
    assert _wait_gone(before) == []


def test_async_loader_over_worker_processes_releases_them_on_close():
    from torch.utils.data import DataLoader
    before = {c.pid for c in _worker_children()}
    dl = DataLoader(Counting(24), batch_size=4, num_workers=2)
    it = async_loader(dl, torch.device("cpu"), depth=2)
    first = next(iter(it))
    assert first["input_ids"].shape == (4, 4)
    it.close()                                            # stopped early: the workers must not linger
    del it, dl
    import gc
    gc.collect()
    assert _wait_gone(before) == []
