"""Host-side logic of the sharded optimizer (chunk tables, gather / scatter of the moment shards) on CPU.

The kernels need a GPU; the bookkeeping around them does not. A stand-in for the symmetric-memory
group and a patched ``all_gather_into_tensor`` let two "ranks" live in one process.
"""
import pytest
import torch

import forgeminds_b200 as fm
from forgeminds_b200.parallel import peer as P
from forgeminds_b200.parallel.flat import ALIGN, FlatParamStore
from forgeminds_b200.parallel.symm import SymmTensor


class FakeGroup:
    """What FlatParamStore / PeerAdamW read from a SymmGroup."""

    def __init__(self, rank, world):
        self.rank, self.world, self.group = rank, world, None
        self._reserved = 0
        self.device = torch.device("cpu")

    def reserve_slots(self, n):
        first = self._reserved
        self._reserved += n
        return first

    def alloc(self, numel, dtype):
        t = torch.zeros(numel, dtype=dtype)
        return SymmTensor(t, [0])


@pytest.fixture
def two_ranks(monkeypatch):
    world = 2
    opts = []
    for r in range(world):
        torch.manual_seed(0)
        model = fm.GPT(fm.GPTConfig(vocab_size=64, dim=32, n_layers=2, n_heads=2, n_kv_heads=1, max_seq=16, ffn_hidden=64))
        store = FlatParamStore(model, "cpu", symm=FakeGroup(r, world))
        opts.append(P.PeerAdamW(store))
    current = {"rank": 0}

    def all_gather(out, inp, group=None):
        me = opts[current["rank"]]
        for name in ("exp_avg", "exp_avg_sq"):
            base = getattr(me, name)
            if inp.untyped_storage().data_ptr() == base.untyped_storage().data_ptr():
                off, n = inp.storage_offset(), inp.numel()
                out.copy_(torch.cat([getattr(o, name)[off:off + n] for o in opts]))
                return
        raise AssertionError("unexpected all_gather input")

    monkeypatch.setattr(P.dist, "all_gather_into_tensor", all_gather)
    return opts, current


def test_buckets_split_evenly_and_shards_tile_the_store(two_ranks):
    opts, _ = two_ranks
    store = opts[0].store
    covered = 0
    for b in store.buckets:
        assert b.size % (ALIGN * 2) == 0
        lo0, n0 = store.shard_range(b, 0)
        lo1, n1 = store.shard_range(b, 1)
        assert lo0 == b.start and lo1 == lo0 + n0 and n0 == n1 and lo1 + n1 == b.start + b.size
        covered += n0 + n1
    assert covered == store.total
    assert opts[0].exp_avg.numel() == store.total // 2


def test_state_dict_round_trip_restores_every_shard(two_ranks):
    opts, current = two_ranks
    want = []
    for r, o in enumerate(opts):
        o.exp_avg.copy_(torch.arange(o.exp_avg.numel(), dtype=torch.float32) + 1000 * r)
        o.exp_avg_sq.copy_(torch.arange(o.exp_avg.numel(), dtype=torch.float32) * 0.5 + 7 * r)
        want.append((o.exp_avg.clone(), o.exp_avg_sq.clone()))
    dicts = []
    for r, o in enumerate(opts):
        current["rank"] = r
        o.steps = 5
        o.gather_full()
        # the gathered state has the layout of torch.optim.AdamW: one entry per parameter, full shapes
        for p in o.store.params:
            assert o.state[p]["exp_avg"].shape == p.shape
        dicts.append(o.state_dict())
        o.release_full()
        assert not o.state
    for r, o in enumerate(opts):
        current["rank"] = r
        o.exp_avg.zero_()
        o.exp_avg_sq.zero_()
        o.load_state_dict(dicts[r])
    for r, o in enumerate(opts):
        st = o.store
        for b in st.buckets:
            lo, n = st.shard_range(b, r)
            s0 = b.start // 2
            for p in b.params:                       # padding between parameters is not part of the state
                a, e = max(st._offset[p], lo), min(st._offset[p] + p.numel(), lo + n)
                if a < e:
                    sl = slice(s0 + a - lo, s0 + e - lo)
                    assert torch.equal(o.exp_avg[sl], want[r][0][sl])
                    assert torch.equal(o.exp_avg_sq[sl], want[r][1][sl])


def test_chunk_tables_cover_the_shard_once_with_the_right_decay(two_ranks, monkeypatch):
    opts, _ = two_ranks

    class FakeC:
        @staticmethod
        def comm_adam_chunk():
            return 4096

    monkeypatch.setattr(P.ops, "require", lambda: FakeC)
    for r, o in enumerate(opts):
        o._build_tables(0.1)
        assert o._tables[1][0].numel() == 0          # no rank-local buckets in a dense model
        off, soff, ln, wd = (t.tolist() for t in o._tables[0])
        seen = torch.zeros(o.store.total, dtype=torch.int32)
        for a, s, n, w in zip(off, soff, ln, wd):
            assert n % 8 == 0 and 0 < n <= 4096
            seen[a:a + n] += 1
            assert 0 <= s and s + n <= o.exp_avg.numel()
        st = o.store
        for b in st.buckets:
            lo, n = st.shard_range(b, r)
            for p, (poff, pn, dec) in zip(b.params, b.decay):
                a, e = max(b.start + poff, lo), min(b.start + poff + pn, lo + n)
                if a < e:
                    assert bool((seen[a:e] == 1).all())
                    i = next(j for j, x in enumerate(off) if x <= a < x + ln[j])
                    assert wd[i] == pytest.approx(0.1 if dec else 0.0)
        lo_all = [st.shard_range(b, r) for b in st.buckets]
        mine = sum(n for _, n in lo_all)
        assert int(seen.sum()) <= mine                # nothing outside this rank's shards


def _gather_plan(rank, world, rows_per_src, grid):
    """Python statement of the row schedule of the GEMM's gather warps (csrc/gemm_sm100.cu, gather_rows):
    the remote rows form one list, nearest rank first; CTA b takes rows b, b + grid, ... two at a time."""
    rows_total = (world - 1) * rows_per_src
    plan = []                                            # (cta, iteration, source rank, row of the full operand)
    for cta in range(grid):
        it = 0
        q = cta
        while q < rows_total:
            for qq in (q, q + grid):
                if qq < rows_total:
                    step = qq // rows_per_src + 1
                    src = (rank + step) % world
                    plan.append((cta, it, src, src * rows_per_src + (qq - (step - 1) * rows_per_src)))
            q += 2 * grid
            it += 1
    return plan


@pytest.mark.parametrize("world,rank,rows_per_src,grid", [(2, 0, 256, 148), (8, 3, 1024, 148), (4, 3, 128, 37), (8, 7, 384, 5)])
def test_gather_schedule_copies_every_remote_row_once_nearest_rank_first(world, rank, rows_per_src, grid):
    plan = _gather_plan(rank, world, rows_per_src, grid)
    rows = [r for *_, r in plan]
    own = set(range(rank * rows_per_src, (rank + 1) * rows_per_src))
    assert len(rows) == len(set(rows)) == (world - 1) * rows_per_src
    assert not own & set(rows)
    # every 128-row block of a remote shard receives exactly 128 arrivals (what the TMA producer waits for)
    per_block = {}
    for r in rows:
        per_block[r >> 7] = per_block.get(r >> 7, 0) + 1
    assert set(per_block.values()) == {128}
    # inside one CTA the sources come in the order rank+1, rank+2, ... (the order the row tiles are computed in)
    for cta in range(min(grid, 4)):
        dist = [(src - rank) % world for c, _, src, _ in plan if c == cta]
        assert dist == sorted(dist)


def test_bounded_expert_parallel_buffers_cut_the_plan_without_a_host_read():
    """Row count of bounded dispatch buffers and the clamped slot plan (device-tensor arithmetic only)."""
    from forgeminds_b200.parallel.ep import ALIGN, bounded_rows, clamp_plan
    assert bounded_rows(10240, 8192, 4, 2, 0.0) == 10240                     # 0: the worst case
    assert bounded_rows(10240, 8192, 4, 2, 100.0) == 10240                   # never more than the worst case
    rows = bounded_rows(10240, 8192, 4, 2, 2.0)
    assert rows == (2 * 8192 // 4 + 2 * ALIGN + ALIGN - 1) // ALIGN * ALIGN and rows % ALIGN == 0
    region = torch.tensor([[0, 300, 512], [512, 700, 768], [1280, 100, 256]], dtype=torch.int32)
    limit = torch.tensor([1536, 0, 0], dtype=torch.int32)
    r, l, over = clamp_plan(region, limit, 2048)
    assert torch.equal(r, region) and torch.equal(l, limit) and not bool(over)
    r, l, over = clamp_plan(region, limit, 1024)
    assert bool(over) and int(l[0]) == 1024
    assert r.tolist() == [[0, 300, 512], [512, 512, 512], [1024, 0, 0]]
    assert int((r[:, 0] + r[:, 2]).max()) <= 1024 and torch.equal(region[0], r[0])
    assert torch.equal(limit, torch.tensor([1536, 0, 0], dtype=torch.int32))   # inputs are not modified
