"""Host-side logic of the expert-parallel layer on CPU ranks (gloo, world size 2 and 4):
split sizes from the unit-1 sort, count exchange, dispatch/combine ordering and the inverse
permutation.  Device kernels are replaced by numpy/torch stand-ins behind the ``ops`` seam; the
expert computation is a stand-in function that depends on (row bytes, scale, global expert id),
so any mis-routed or mis-ordered row changes the result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flydsl_b200 import ep
from oracle import moe_oracle as orc

T, E, K, H = 37, 8, 3, 256


class FakeOps:
    def __init__(self):
        self.out = torch.zeros((T, H), dtype=torch.float32)

    def gate(self, logits):
        w, idx, _ = orc.topk_gating_softmax(logits, K)
        return w, idx

    def sort_by_expert(self, ids, w, tokens, chunk=0):
        s_ids, _, s_e, nv = orc.moe_sorting(ids.numpy(), w.numpy(), E, 1)
        return torch.from_numpy(s_ids), torch.from_numpy(s_e)

    def pack(self, xq, xs, s_ids, tokens, chunk=0):
        tok = (s_ids[: tokens * K] & 0xFFFFFF).long()
        return xq[tok].contiguous(), xs[tok].contiguous()

    def empty_rows(self, rows, like):
        return torch.empty((rows,) + tuple(like.shape[1:]), dtype=like.dtype)

    def local_experts(self, rx, rs, re_, first, rows, chunk=0):
        assert rows == 0 or (int(re_.min()) >= first and int(re_.max()) < first + E // dist.get_world_size())
        return rx.float() * rs.mean(dim=1, keepdim=True) * (re_.view(-1, 1).float() + 1.0)

    def combine(self, back, s_ids, w, lo, hi, tokens, chunk=0):
        n = hi - lo
        tok = (s_ids[: n * K] & 0xFFFFFF).long()
        slot = (s_ids[: n * K] >> 24).long()
        part = torch.zeros((n, back.shape[1]), dtype=torch.float32)
        part.index_add_(0, tok, back * w[tok, slot].view(-1, 1))
        self.out[lo:hi] = part
        return self.out


class FakeFusedOps(FakeOps):
    """Fused combine on CPU ranks: the peers' returned-rows buffers are one shared-memory tensor
    [world, T*K, H]; an "address" is rank * STRIDE + row, and a peer store is a plain write there."""
    fused_combine = True
    STRIDE = 1 << 20

    def __init__(self, shared):
        super().__init__()
        self.shared = shared

    def row_destinations(self, plan, rank):
        dst, at = [], 0
        for s, (cnt, off) in enumerate(zip(plan.recv_counts, plan.peer_offsets)):
            dst += [s * self.STRIDE + off + j for j in range(cnt)]
            at += cnt
        return torch.tensor(dst, dtype=torch.int64)

    def local_experts(self, rx, rs, re_, first, rows, chunk=0, row_dst=None):
        y = super().local_experts(rx, rs, re_, first, rows, chunk)
        if row_dst is None:
            return y
        for j in range(rows):
            d = int(row_dst[j])
            self.shared[d // self.STRIDE, d % self.STRIDE] = y[j]
        return None

    def peer_rendezvous(self):
        dist.barrier()

    def returned_rows(self, pairs):
        return self.shared[dist.get_rank(), :pairs]


class FakeDirectOps(FakeFusedOps):
    """Direct dispatch on CPU ranks: the peers' operand buffers are shared-memory tensors too, rows are
    written at the positions ``plan_direct`` assigns and read back through its segment list."""
    direct_dispatch = True
    tile_m = 4
    CAP = 256

    def __init__(self, shared, xs_shared, xsc_shared):
        super().__init__(shared)
        self.xs_shared, self.xsc_shared = xs_shared, xsc_shared

    def expert_counts(self, s_eids, pairs):
        return torch.bincount(s_eids[:pairs].long(), minlength=E).to(torch.int64)

    def check_direct_capacity(self, dp):
        assert dp.max_padded_rows <= self.CAP

    def dispatch_direct(self, xq, xs, s_ids, s_eids, dp, tokens):
        per = E // dist.get_world_size()
        for i in range(tokens * K):
            e, tok = int(s_eids[i]), int(s_ids[i]) & 0xFFFFFF
            pos = int(dp.pos_base[e]) + i
            self.xs_shared[e // per, pos] = xq[tok]
            self.xsc_shared[e // per, pos] = xs[tok]

    def local_experts_direct(self, dp):
        rank, per = dist.get_rank(), E // dist.get_world_size()
        assert dp.padded_rows == len(dp.block_expert) * self.tile_m
        pos = 0
        for n, src, row in zip(dp.seg_len.tolist(), dp.seg_src.tolist(), dp.seg_src_row.tolist()):
            for j in range(n):
                if src >= 0:
                    e = rank * per + int(dp.block_expert[(pos + j) // self.tile_m])
                    y = self.xs_shared[rank, pos + j].float() * self.xsc_shared[rank, pos + j].mean() * (e + 1.0)
                    self.shared[src, row + j] = y
            pos += n


class FakeDevicePlanOps(FakeDirectOps):
    """The step without a host round trip: the plan is ``plan_direct_tensors`` output."""
    device_plan = True

    def run_direct_on_device(self, xq, xs, s_ids, s_eids, counts, rank, tokens):
        per = E // dist.get_world_size()
        pl = ep.plan_direct_tensors(counts, rank, per, self.tile_m, self.CAP)
        for i in range(tokens * K):
            e, tok = int(s_eids[i]), int(s_ids[i]) & 0xFFFFFF
            pos = int(pl["pos_base"][e]) + i
            self.xs_shared[e // per, pos] = xq[tok]
            self.xsc_shared[e // per, pos] = xs[tok]
        dist.barrier()
        for pos in range(int(pl["padded_rows"])):
            src = int(pl["src"][pos])
            if src >= 0:
                e = rank * per + int(pl["block_expert"][pos // self.tile_m])
                y = self.xs_shared[rank, pos].float() * self.xsc_shared[rank, pos].mean() * (e + 1.0)
                self.shared[src, int(pl["src_row"][pos])] = y
        dist.barrier()


def _inputs(rank):
    g = torch.Generator().manual_seed(100 + rank)
    logits = torch.randn((T, E), generator=g)
    xq = torch.randint(0, 255, (T, H), generator=g, dtype=torch.uint8)
    xs = torch.rand((T, H // 128), generator=g) + 0.5
    return logits, xq, xs


def _worker(rank, world, port, chunks, q, shared=None, direct=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        logits, xq, xs = _inputs(rank)
        ops = (FakeOps() if shared is None else FakeFusedOps(shared) if direct is None
               else (FakeDevicePlanOps if len(direct) == 3 else FakeDirectOps)(shared, *direct[:2]))
        layer = ep.ExpertParallelMoE(ops, E, K, H, chunks=chunks)
        out = layer(logits, xq, xs)
        if shared is not None:                      # a second step reuses the peers' buffers
            dist.barrier()
            out = layer(logits, xq, xs).clone()
        w, idx, _ = orc.topk_gating_softmax(logits, K)
        want = (xq.float() * xs.mean(dim=1, keepdim=True)).unsqueeze(1) * (idx.float() + 1.0).unsqueeze(-1)
        want = (want * w.unsqueeze(-1)).sum(dim=1)
        plan = layer.last_plan
        ok = torch.allclose(out, want, rtol=1e-5, atol=1e-4)
        counts_ok = sum(plan.send_counts) == T * K and plan.rows_out == T * K
        gathered = [None] * world
        dist.all_gather_object(gathered, (plan.send_counts, plan.recv_counts))
        transposed_ok = all(gathered[r][0][rank] == plan.recv_counts[r] for r in range(world))
        if chunks == 1 and direct is None:          # block starts as the sender sees them
            offs = layer.last_plans[0].peer_offsets
            transposed_ok = transposed_ok and all(offs[r] == sum(gathered[r][0][:rank]) for r in range(world))
        q.put((rank, bool(ok), bool(counts_ok), bool(transposed_ok), float((out - want).abs().max())))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 3), (4, 2), (8, 1)])
def test_dispatch_combine_roundtrip_on_cpu_ranks(world, chunks):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, chunks, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, counts_ok, transposed_ok, err in res:
        assert ok, f"rank {rank}: combined output differs (max abs err {err})"
        assert counts_ok and transposed_ok


@pytest.mark.parametrize("world", [2, 4])
def test_fused_combine_addresses_on_cpu_ranks(world):
    """Every expert output row is written by the rank that computed it into the owner's buffer at the
    owner's send-order position; the owner's reduce then sees exactly what the all-to-all would return."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    shared = torch.full((world, T * K, H), float("nan")).share_memory_()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 1, q, shared)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, counts_ok, transposed_ok, err in res:
        assert ok, f"rank {rank}: combined output differs (max abs err {err})"
        assert counts_ok and transposed_ok


@pytest.mark.parametrize("world,device_plan", [(2, False), (4, False), (2, True), (4, True), (8, True)])
def test_direct_dispatch_layout_on_cpu_ranks(world, device_plan):
    """Rows stored by their senders at plan_direct's positions are found by the receivers' segment
    lists, grouped by expert in whole row blocks; outputs return to the owners' send-order slots."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    shared = torch.full((world, T * K, H), float("nan")).share_memory_()
    xs_sh = torch.zeros((world, FakeDirectOps.CAP, H), dtype=torch.uint8).share_memory_()
    xsc_sh = torch.zeros((world, FakeDirectOps.CAP, H // 128)).share_memory_()
    extra = (xs_sh, xsc_sh, True) if device_plan else (xs_sh, xsc_sh)
    procs = [ctx.Process(target=_worker, args=(r, world, port, 1, q, shared, extra)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, counts_ok, transposed_ok, err in res:
        assert ok, f"rank {rank}: combined output differs (max abs err {err})"
        assert counts_ok and transposed_ok


def test_plan_direct_positions_and_segments():
    """Pure bookkeeping: emulate every rank's stores and check every receiver's view of them."""
    rng = np.random.default_rng(0)
    world, experts, unit = 4, 16, 8
    per = experts // world
    lists = [np.sort(rng.integers(0, experts, size=int(rng.integers(20, 60)))) for _ in range(world)]
    lists[2] = lists[2][lists[2] != 5]                     # an expert nobody on rank 2 uses
    counts = np.stack([np.bincount(l, minlength=experts) for l in lists])
    counts[:, 9] = 0                                       # an expert with no rows at all takes no block
    lists = [l[l != 9] for l in lists]
    plans = [ep.plan_direct(counts, r, per, unit) for r in range(world)]
    bufs = [np.full((plans[d].padded_rows, 2), -1, dtype=np.int64) for d in range(world)]
    for r in range(world):
        for i, e in enumerate(lists[r]):
            pos = plans[r].pos_base[e] + i
            assert (bufs[e // per][pos] == -1).all(), "two rows at one position"
            bufs[e // per][pos] = (r, i)
    for d, p in enumerate(plans):
        pos = 0
        for n, src, row in zip(p.seg_len, p.seg_src, p.seg_src_row):
            for j in range(n):
                assert tuple(bufs[d][pos + j]) == ((-1, -1) if src < 0 else (src, row + j))
            pos += n
        assert pos == p.padded_rows == len(p.block_expert) * unit == max(pos, 0)
        assert p.rows_in == int((bufs[d][:, 0] >= 0).sum()) == sum(p.recv_counts)
        for b, el in enumerate(p.block_expert):
            for s_, i in bufs[d][b * unit:(b + 1) * unit]:
                assert s_ < 0 or lists[s_][i] == d * per + el
        assert p.max_padded_rows == max(q.padded_rows for q in plans)
        assert all(plans[s_].send_counts[d] == p.recv_counts[s_] for s_ in range(world))
        # the tensor-operation planner (what runs on the GPU without a host round trip) agrees row by row
        cap = p.max_padded_rows + 3 * unit
        t = ep.plan_direct_tensors(torch.from_numpy(counts), d, per, unit, cap)
        assert t["pos_base"].tolist() == p.pos_base.tolist()
        assert int(t["padded_rows"]) == p.padded_rows and int(t["rows_in"]) == p.rows_in
        assert int(t["max_padded_rows"]) == p.max_padded_rows
        want_src = np.concatenate([bufs[d][:, 0], np.full(cap - p.padded_rows, -1)])
        assert t["src"].tolist() == want_src.tolist()
        real = want_src >= 0
        assert t["src_row"].numpy()[real].tolist() == bufs[d][:, 1][real[:p.padded_rows]].tolist()
        assert t["block_expert"][:len(p.block_expert)].tolist() == p.block_expert.tolist()


def test_split_counts_and_checks():
    eids = torch.tensor([0, 0, 1, 3, 3, 3, 4, 7, 7], dtype=torch.int32)
    assert ep.split_counts(eids, 2, 4).tolist() == [6, 3]
    assert ep.split_counts(eids, 4, 2).tolist() == [3, 3, 1, 2]
    assert ep.split_counts(eids, 8, 1).tolist() == [2, 1, 0, 3, 1, 0, 0, 2]
    assert list(ep.expert_range(3, 4, 256)) == list(range(192, 256))
    assert ep.chunk_bounds(10, 3) == [(0, 4), (4, 7), (7, 10)] and ep.chunk_bounds(2, 4) == [(0, 1), (1, 2)]
    assert ep.chunk_bounds(5, 1) == [(0, 5)]
    with pytest.raises(ValueError):
        ep.expert_range(0, 3, 256)
    good = torch.tensor([6, 3])
    ep.check_counts(good, torch.tensor([1, 2]), 9)
    with pytest.raises(RuntimeError, match="covers"):
        ep.check_counts(torch.tensor([6, 2]), good, 9)          # a rank lost a row: caught on the host
    with pytest.raises(RuntimeError, match="negative"):
        ep.check_counts(torch.tensor([10, -1]), good, 9)
