"""Expert-parallel FP8 block-scaled MoE layer: one process per GPU, experts sharded
evenly over the ranks.

The reference has no dispatch/combine (its only expert-parallel hook is the
``expert_mask`` of the sort, kernels/moe_sorting_kernel.py:426-440); this module adds the
partitioned case on top of the same kernels.  Three transports, same arithmetic per
(token, slot) pair, bit-identical results:

``direct_dispatch`` (the fast path, needs peer-mapped buffers, ``flydsl_b200.peer``):
  1. gate the rank's own tokens over all E experts               (gating kernel)
  2. sort the (token, slot) pairs by global expert id, unit 1     (sort kernels)
  3. rows per expert, all-gathered; every rank derives every rank's receive layout
     (``plan_direct``) -- the step's single host synchronisation
  4. dispatch: each row and its scales are stored straight into the owning rank's stage-1
     operand buffer, at its final position of that rank's expert-sorted, block-padded
     layout                                                        (``flymoe_dispatch_rows``, peer stores)
  5. rendezvous; stage 1; stage 2, whose epilogue stores every output row straight into the
     token owner's buffer                                          (``flymoe_moe_gemm2_scatter_rows``)
  6. rendezvous; out[t] = sum_s w[t,s] * returned_row(t,s)        (indexed reduce kernel)
  The receiver neither sorts nor gathers, and NCCL carries only the counts and the two
  rendezvous (one-element all-reduces).  With ``device_plan`` step 3 is tensor operations on the
  GPU (``plan_direct_tensors``) and the step has no host synchronisation at all; rows that would
  not fit the receiver's buffer are then dropped and flagged in the device status word instead
  of raising.

``fused_combine``: dispatch by NCCL all-to-all (steps 2-5 of the list below), outputs return
  as in 5./6. above.

NCCL both ways (default without peer buffers; can be cut into pipelined chunks):
  2. sort by global expert id, unit 1 -- rows grouped by expert are also grouped by
     destination rank, and every rank's block arrives pre-grouped by local expert
  3. row counts per destination, exchanged for all chunks at once      (one tiny all_to_all,
     the step's single host synchronisation)
  4. pack e4m3 rows and their fp32 scales in that order           (row-gather kernel)
  5. dispatch rows, scales and expert ids                          (all_to_all_single x3, async)
  6. local experts: sort by local expert, stage 1, stage 2 into per-row bf16 outputs
  7. combine: send the rows back                                  (all_to_all_single, async)
  8. the indexed reduce.

Remote data always lands in this GPU's memory before any kernel reads it: kernels only ever
*store* to a peer, never load from one or wait on one.  The host-side bookkeeping
(``split_counts``, ``exchange_counts``, ``plan_direct``, the step order in ``forward``) is
device-agnostic so it can be exercised with gloo on CPU ranks through the ``ops`` seam.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


def expert_range(rank: int, world: int, experts: int) -> range:
    if experts % world != 0:
        raise ValueError(f"experts ({experts}) must divide evenly over {world} ranks")
    per = experts // world
    return range(rank * per, (rank + 1) * per)


def chunk_bounds(tokens: int, chunks: int) -> list:
    """Token ranges [lo, hi) of the pipeline chunks (the first chunks take the remainder)."""
    chunks = max(1, min(chunks, max(tokens, 1)))
    base, rem = divmod(tokens, chunks)
    out, lo = [], 0
    for c in range(chunks):
        hi = lo + base + (1 if c < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def split_counts(sorted_expert_ids: torch.Tensor, world: int, experts_per_rank: int) -> torch.Tensor:
    """Rows destined to each rank, from the ascending per-row expert ids of the unit-1 sort."""
    bounds = torch.arange(0, world + 1, device=sorted_expert_ids.device,
                          dtype=sorted_expert_ids.dtype) * experts_per_rank
    pos = torch.searchsorted(sorted_expert_ids.contiguous(), bounds.contiguous())
    return (pos[1:] - pos[:-1]).to(torch.int64)


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """all-to-all of equal-sized int64 blocks: block r of the result is what rank r sent here."""
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


def check_counts(send_counts, recv_counts, pairs: int, group=None) -> None:
    """Host-side consistency checks run before any payload collective is posted."""
    if int(send_counts.sum()) != pairs:
        raise RuntimeError(f"dispatch plan covers {int(send_counts.sum())} rows, expected {pairs}")
    if bool((send_counts < 0).any()) or bool((recv_counts < 0).any()):
        raise RuntimeError("negative row count in the dispatch plan")


@dataclass
class DispatchPlan:
    send_counts: list
    recv_counts: list
    rows_out: int
    rows_in: int
    # peer_offsets[s]: where this rank's block starts in rank s's send order (the row index, on rank s,
    # of the first row this rank received from s) -- the address base of the fused combine
    peer_offsets: list | None = None


@dataclass
class DirectPlan:
    """Where rows go when they are dispatched by direct stores (``plan_direct``)."""
    counts: np.ndarray          # [world, E] rows per (source rank, global expert)
    pos_base: np.ndarray        # [E] int64: row r of this rank's sorted order, expert e, lands at pos_base[e] + r
    rows_in: int                # rows this rank receives
    padded_rows: int            # its layout's extent: every local expert padded to whole row blocks
    block_expert: np.ndarray    # [blocks] int32 local expert of each row block
    seg_len: np.ndarray         # receiver layout as consecutive segments: length,
    seg_src: np.ndarray         #   source rank (-1 = padding),
    seg_src_row: np.ndarray     #   row index of the segment's first row in the source's sorted order
    send_counts: list
    recv_counts: list
    max_padded_rows: int        # largest layout over all ranks (capacity check, identical on every rank)


def plan_direct(counts: np.ndarray, rank: int, per_rank: int, unit: int) -> DirectPlan:
    """Layout of every rank's receive buffer from the all-gathered per-expert row counts.

    A rank's buffer holds its local experts in ascending order, each padded to a multiple of
    ``unit`` rows; inside an expert the rows of source 0 come first, then source 1, ...; each
    source's rows keep the order of its own expert-sorted list.  Every rank derives the same
    layouts from the same matrix, so senders know final positions and receivers know who wrote
    what, with no further exchange."""
    counts = np.asarray(counts, dtype=np.int64)
    world, E = counts.shape
    src_prefix = np.cumsum(counts, axis=0) - counts                   # rows of expert e from sources < s
    own_start = np.cumsum(counts, axis=1) - counts                    # start of expert e in source s's order
    total = counts.sum(axis=0)                                        # [E]
    padded = (total + unit - 1) // unit * unit
    start = np.zeros(E, dtype=np.int64)                               # start of expert e in its owner's layout
    extent = []
    for d in range(world):
        sl = slice(d * per_rank, (d + 1) * per_rank)
        start[sl] = np.cumsum(padded[sl]) - padded[sl]
        extent.append(int(padded[sl].sum()))
    pos_base = start + src_prefix[rank] - own_start[rank]
    lo, hi = rank * per_rank, (rank + 1) * per_rank
    # this rank's layout as segments: per local expert one segment per source, then the padding
    seg_len = np.concatenate([counts[:, lo:hi].T, (padded - total)[lo:hi, None]], axis=1).reshape(-1)
    seg_src = np.tile(np.concatenate([np.arange(world), [-1]]), per_rank)
    seg_src_row = np.concatenate([own_start[:, lo:hi].T, np.zeros((per_rank, 1), dtype=np.int64)], axis=1).reshape(-1)
    keep = seg_len > 0
    block_expert = np.repeat(np.arange(per_rank, dtype=np.int32), padded[lo:hi] // unit)
    send_counts = counts[rank].reshape(world, per_rank).sum(axis=1).tolist()
    recv_counts = counts[:, lo:hi].sum(axis=1).tolist()
    return DirectPlan(counts, pos_base.astype(np.int64), int(total[lo:hi].sum()), extent[rank], block_expert,
                      seg_len[keep].astype(np.int64), seg_src[keep].astype(np.int64),
                      seg_src_row[keep].astype(np.int64), send_counts, recv_counts, max(extent))


def plan_direct_tensors(counts: torch.Tensor, rank: int, per_rank: int, unit: int, cap_rows: int) -> dict:
    """``plan_direct`` as tensor operations on the device that holds ``counts`` -- no host round trip.

    Returns pos_base [E]; for this rank's layout the per-row arrays of length ``cap_rows``: ``src``
    (source rank, -1 = padding or beyond the layout), ``src_row`` (row in the source's sorted order);
    ``block_expert`` [cap_rows // unit] (local expert of each row block, clamped beyond the layout);
    ``padded_rows`` / ``rows_in`` / ``max_padded_rows`` as 0-dim tensors."""
    world, E = counts.shape
    dev = counts.device
    src_prefix = torch.cumsum(counts, dim=0) - counts
    own_start = torch.cumsum(counts, dim=1) - counts
    total = counts.sum(dim=0)
    padded = (total + unit - 1) // unit * unit
    pad2 = padded.view(world, per_rank)
    start = (torch.cumsum(pad2, dim=1) - pad2).reshape(-1)
    extent = pad2.sum(dim=1)                                              # [world]
    pos_base = start + src_prefix[rank] - own_start[rank]
    lo, hi = rank * per_rank, (rank + 1) * per_rank
    # segments of this rank's layout, in layout order: per local expert one per source, then the padding
    seg_len = torch.cat([counts[:, lo:hi].t(), (padded - total)[lo:hi, None]], dim=1).reshape(-1)
    seg_src = torch.cat([torch.arange(world, device=dev), torch.tensor([-1], device=dev)]).repeat(per_rank)
    seg_row = torch.cat([own_start[:, lo:hi].t(), torch.zeros((per_rank, 1), dtype=counts.dtype, device=dev)],
                        dim=1).reshape(-1)
    seg_end = torch.cumsum(seg_len, dim=0)
    pos = torch.arange(cap_rows, dtype=torch.int64, device=dev)
    which = torch.searchsorted(seg_end, pos, right=True)                  # zero-length segments are skipped
    inside = which < seg_len.numel()
    which = which.clamp(max=seg_len.numel() - 1)
    src = torch.where(inside, seg_src[which], -1)
    src_row = seg_row[which] + (pos - (seg_end - seg_len)[which])
    blk_end = torch.cumsum(padded[lo:hi] // unit, dim=0)                  # row blocks per local expert
    blocks = torch.arange(cap_rows // unit, dtype=torch.int64, device=dev)
    block_expert = torch.searchsorted(blk_end, blocks, right=True).clamp(max=per_rank - 1)
    return {"pos_base": pos_base, "src": src, "src_row": src_row, "block_expert": block_expert.to(torch.int32),
            "padded_rows": extent[rank], "rows_in": total[lo:hi].sum(), "max_padded_rows": extent.max()}


class ExpertParallelMoE:
    """Expert-parallel layer.  ``ops`` supplies the device kernels (see ``CudaOps``)."""

    def __init__(self, ops, experts: int, topk: int, model_dim: int, group=None, chunks: int = 1):
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.experts, self.topk, self.H = experts, topk, model_dim
        self.local = expert_range(self.rank, self.world, experts)
        self.per_rank = len(self.local)
        self.chunks = max(1, int(chunks))
        self.last_plans: list = []
        # a list here makes the peer-store step record one CUDA event per phase boundary: (name, event)
        self.phase_marks = None

    def _phase(self, name: str) -> None:
        if self.phase_marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream())
            self.phase_marks.append((name, ev))

    @property
    def last_plan(self) -> DispatchPlan:
        """Whole-step totals over the chunks of the last forward."""
        ps = self.last_plans
        if not ps and getattr(self, "_counts_dev", None) is not None:         # device-planned step: fetch on demand
            dp = plan_direct(self._counts_dev.cpu().numpy(), self.rank, self.per_rank, self.ops.tile_m)
            ps = [DispatchPlan(dp.send_counts, dp.recv_counts, sum(dp.send_counts), dp.rows_in)]
        send = [sum(p.send_counts[r] for p in ps) for r in range(self.world)]
        recv = [sum(p.recv_counts[r] for p in ps) for r in range(self.world)]
        return DispatchPlan(send, recv, sum(send), sum(recv))

    def plan(self, eids_per_chunk: list, pairs_per_chunk: list) -> list:
        """Per-chunk send/receive row counts; one count exchange and ONE host sync for the step."""
        n, C = self.world, len(eids_per_chunk)
        send = torch.stack([split_counts(e, n, self.per_rank) for e in eids_per_chunk])   # [C, n]
        start = torch.cumsum(send, dim=1) - send                                           # block starts, [C, n]
        send_by_rank = torch.stack([send.t(), start.t()], dim=2).contiguous().view(-1)     # [n * C * 2]
        recv_by_rank = exchange_counts(send_by_rank, self.group)
        both = torch.stack([send_by_rank, recv_by_rank]).cpu().view(2, n, C, 2)
        plans = []
        for c in range(C):
            s, r = both[0, :, c, 0], both[1, :, c, 0]
            check_counts(s, r, pairs_per_chunk[c])
            plans.append(DispatchPlan(s.tolist(), r.tolist(), int(s.sum()), int(r.sum()),
                                      both[1, :, c, 1].tolist()))
        self.last_plans = plans
        return plans

    def forward(self, logits, xq, x_scale):
        """logits [T,E]; xq e4m3 [T,H]; x_scale f32 row-major [T,H/128] -> out [T,H]."""
        ops, k, g = self.ops, self.topk, self.group
        T = logits.shape[0]
        bounds = chunk_bounds(T, self.chunks)
        C = len(bounds)
        self._phase("start")
        topk_w, topk_ids = ops.gate(logits)
        if getattr(ops, "direct_dispatch", False):
            return self._forward_direct(topk_w, topk_ids, xq, x_scale, T)
        sorted_c = []
        for c, (lo, hi) in enumerate(bounds):
            sorted_c.append(ops.sort_by_expert(topk_ids[lo:hi], topk_w[lo:hi], hi - lo, c))
        pairs = [(hi - lo) * k for lo, hi in bounds]
        plans = self.plan([e[:p] for (_, e), p in zip(sorted_c, pairs)], pairs)

        # dispatch of every chunk is posted up front; NCCL runs them in order on its own stream
        recv, works = [], []
        for c, (lo, hi) in enumerate(bounds):
            s_ids, s_eids = sorted_c[c]
            p, pl = pairs[c], plans[c]
            send_x, send_s = ops.pack(xq[lo:hi], x_scale[lo:hi], s_ids, hi - lo, c)
            rx, rs, re_ = (ops.empty_rows(pl.rows_in, t) for t in (send_x, send_s, s_eids))
            w = [dist.all_to_all_single(rx, send_x[:p], pl.recv_counts, pl.send_counts, group=g, async_op=True),
                 dist.all_to_all_single(rs, send_s[:p], pl.recv_counts, pl.send_counts, group=g, async_op=True),
                 dist.all_to_all_single(re_, s_eids[:p], pl.recv_counts, pl.send_counts, group=g, async_op=True)]
            recv.append((rx, rs, re_))
            works.append(w)

        # experts on chunk c while chunk c+1 is still arriving and chunk c-1 is already going back
        if getattr(ops, "fused_combine", False):
            # Stage 2 stores every expert output row straight into the buffer of the rank that owns the
            # token (peer stores from the GEMM epilogue): no combine all-to-all, only a rendezvous.
            if C != 1:
                raise ValueError("the fused combine runs the step as one chunk")
            for w in works[0]:
                w.wait()
            rx, rs, re_ = recv[0]
            ops.local_experts(rx, rs, re_, self.local.start, plans[0].rows_in, 0,
                              row_dst=ops.row_destinations(plans[0], self.rank))
            ops.peer_rendezvous()
            lo, hi = bounds[0]
            return ops.combine(ops.returned_rows(pairs[0]), sorted_c[0][0], topk_w[lo:hi], lo, hi, T, 0)

        back, back_works = [], []
        for c in range(C):
            for w in works[c]:
                w.wait()
            rx, rs, re_ = recv[c]
            y = ops.local_experts(rx, rs, re_, self.local.start, plans[c].rows_in, c)
            b = ops.empty_rows(pairs[c], y)
            back_works.append(dist.all_to_all_single(b, y[:plans[c].rows_in], plans[c].send_counts,
                                                     plans[c].recv_counts, group=g, async_op=True))
            back.append(b)

        out = None
        for c, (lo, hi) in enumerate(bounds):
            back_works[c].wait()
            out = ops.combine(back[c], sorted_c[c][0], topk_w[lo:hi], lo, hi, T, c)
        return out

    def _forward_direct(self, topk_w, topk_ids, xq, x_scale, T):
        """Dispatch and combine as peer stores from this library's own kernels: rows travel straight
        into the owners' GEMM operand buffers at their final sorted positions, expert outputs travel
        straight back from stage 2's epilogue.  NCCL carries only the per-expert row counts and the
        two rendezvous of the step."""
        ops, k, g = self.ops, self.topk, self.group
        P = T * k
        s_ids, s_eids = ops.sort_by_expert(topk_ids, topk_w, T, 0)
        mine = ops.expert_counts(s_eids, P)                                   # int64 [E]
        matrix = ops.counts_matrix(self.world) if hasattr(ops, "counts_matrix") else None
        gathered = (list(matrix.unbind(0)) if matrix is not None
                    else [torch.empty_like(mine) for _ in range(self.world)])
        self._phase("gate_sort_count")
        dist.all_gather(gathered, mine, group=g)
        self._phase("count_exchange")
        if getattr(ops, "device_plan", False):
            # the whole plan stays on the device: no host synchronisation in the step
            self._counts_dev = matrix if matrix is not None else torch.stack(gathered)
            self.last_plans = []
            extra = {} if self.phase_marks is None else {"phase": self._phase}
            ops.run_direct_on_device(xq, x_scale, s_ids, s_eids, self._counts_dev, self.rank, T, **extra)
            out = ops.combine(ops.returned_rows(P), s_ids, topk_w, 0, T, T, 0)
            self._phase("reduce")
            return out
        counts = torch.stack(gathered).cpu().numpy()                          # the step's host synchronisation
        if int(counts[self.rank].sum()) != P:
            raise RuntimeError(f"dispatch plan covers {int(counts[self.rank].sum())} rows, expected {P}")
        dp = plan_direct(counts, self.rank, self.per_rank, ops.tile_m)
        self.last_plans = [DispatchPlan(dp.send_counts, dp.recv_counts, P, dp.rows_in)]
        ops.check_direct_capacity(dp)
        ops.dispatch_direct(xq, x_scale, s_ids, s_eids, dp, T)
        ops.peer_rendezvous()                                                 # every rank's rows have landed
        ops.local_experts_direct(dp)
        ops.peer_rendezvous()                                                 # every rank's outputs are back
        return ops.combine(ops.returned_rows(P), s_ids, topk_w, 0, T, T, 0)

    __call__ = forward


class CudaOps:
    """The device side of ``ExpertParallelMoE`` on one B200: the library's own kernels."""

    def __init__(self, w1q, w1_scale, w2q, w2_scale, experts: int, topk: int, tokens: int,
                 tile_m: int = 128, headroom: float = 1.3, impl: str = "tcgen05", chunks: int = 1,
                 comm_sms: int = 0, fused_combine: bool = False, direct_dispatch: bool = False,
                 device_plan: bool = False, group=None):
        from . import _lib
        self._lib = _lib
        self.lib = _lib.load()
        # With a pipelined step the all-to-all kernels run beside the persistent GEMMs: leave them SMs.
        if comm_sms > 0:
            sms = torch.cuda.get_device_properties(w1q.device).multi_processor_count
            _lib.check(self.lib.flymoe_set_gemm_cta_limit(max(1, sms - comm_sms)), "set_gemm_cta_limit")
        self.E, self.k, self.T = experts, topk, tokens
        self.E_local, _, self.H = w1q.shape
        self.I = w2q.shape[2]
        self.tile_m, self.impl = tile_m, impl
        self.w = (w1q, w1_scale, w2q, w2_scale)
        dev = w1q.device
        self.dev = dev
        i32, f32 = torch.int32, torch.float32
        self.topk_w = torch.empty((tokens, topk), dtype=f32, device=dev)
        self.topk_ids = torch.empty((tokens, topk), dtype=i32, device=dev)
        self.tei = torch.empty((tokens, topk), dtype=i32, device=dev)
        self.out = torch.empty((tokens, self.H), dtype=torch.bfloat16, device=dev)
        bounds = chunk_bounds(tokens, chunks)
        tc = max(hi - lo for lo, hi in bounds)            # tokens of the largest chunk
        pc = tc * topk
        cap = pc + experts - topk                         # unit-1 sort: no padding rows
        ws = int(self.lib.flymoe_moe_sorting_workspace_elems(tc, experts, topk, 1))
        self.ws = torch.empty(max(ws, 1), dtype=i32, device=dev)
        self.chunk_bufs = []
        packed = 0 if direct_dispatch else pc              # direct dispatch stores rows at the receiver: no send buffers
        for _ in bounds:                                   # buffers that must outlive their chunk's collectives
            self.chunk_bufs.append({
                "s_ids": torch.empty(cap, dtype=i32, device=dev), "s_w": torch.empty(cap, dtype=f32, device=dev),
                "s_eids": torch.empty(cap, dtype=i32, device=dev), "nvalid": torch.empty(2, dtype=i32, device=dev),
                "send_x": torch.empty((packed, self.H), dtype=torch.uint8, device=dev),
                "send_s": torch.empty((packed, self.H // 128), dtype=f32, device=dev),
                "inverse": torch.empty(pc, dtype=i32, device=dev), "y": None})
        self.headroom = headroom
        # set by a caller that copies ``out`` away on another stream: the reduce of the next step waits
        # for this event before it overwrites ``out`` (the rest of that step runs without waiting)
        self.out_free_event = None
        self.inner = None
        self._ensure_inner(int(pc * headroom))
        # Fused combine: a [tokens * topk, H] bf16 buffer per rank that all ranks can store into.
        # Direct dispatch: in front of it, the stage-1 operand rows and their scales of this rank.
        self.direct_dispatch = bool(direct_dispatch)
        self.device_plan = bool(device_plan) and self.direct_dispatch
        self.fused_combine = bool(fused_combine) or self.direct_dispatch
        self.peers = None
        if self.fused_combine:
            from .peer import PeerBuffers
            if chunks != 1:
                raise ValueError("fused_combine / direct_dispatch need chunks == 1")
            al = lambda n: (n + 255) // 256 * 256
            rows = self.inner.cap_rows if self.direct_dispatch else 0
            self._off_xs = 0
            self._off_xsc = al(rows * self.H)
            self._off_back = self._off_xsc + al(rows * (self.H // 128) * 4)
            self.peers = PeerBuffers(self._off_back + tokens * topk * self.H * 2, dev, group)
            self._rendezvous_flag = torch.zeros(1, dtype=i32, device=dev)
            if self.direct_dispatch:
                # everything the device-side planner writes, allocated once
                world = len(self.peers.ptrs)
                i64 = torch.int64
                self._counts_mine = torch.zeros(experts, dtype=i64, device=dev)
                self._counts_all = torch.zeros((world, experts), dtype=i64, device=dev)
                self._peer_ptrs = torch.tensor(self.peers.ptrs, dtype=i64, device=dev)
                self._plan_tables = torch.zeros((3, experts), dtype=i64, device=dev)      # dst_x, dst_scale, pos_base
                self._plan_row_dst = torch.zeros(self.inner.cap_rows, dtype=i64, device=dev)
                ws = int(self.lib.flymoe_ep_plan_workspace_elems(world, experts))
                self._plan_ws = torch.zeros(max(ws, 1), dtype=i32, device=dev)

    def _ensure_inner(self, rows: int) -> None:
        from .layer import FusedMoEBlockscale
        if self.inner is not None and self.inner.max_tokens >= rows:
            return
        self.inner = None
        w1q, w1s, w2q, w2s = self.w
        self.inner = FusedMoEBlockscale(w1q, w1s, w2q, w2s, 1, max_tokens=rows, tile_m=self.tile_m,
                                        stage2_mode="rows", impl=self.impl)
        self.ones = torch.ones((rows, 1), dtype=torch.float32, device=self.dev)

    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def gate(self, logits):
        L = self._lib
        T = logits.shape[0]
        L.check(self.lib.flymoe_topk_gating_softmax(logits.data_ptr(), L.DTYPE_CODE[logits.dtype],
                                                    self.topk_w.data_ptr(), self.topk_ids.data_ptr(),
                                                    self.tei.data_ptr(), T, self.E, self.k, 1, self._stream()),
                "topk_gating_softmax")
        return self.topk_w, self.topk_ids

    def sort_by_expert(self, topk_ids, topk_w, T, chunk: int = 0):
        L, b = self._lib, self.chunk_bufs[chunk]
        L.check(self.lib.flymoe_moe_sorting(topk_ids.data_ptr(), topk_w.data_ptr(), b["s_ids"].data_ptr(),
                                            b["s_w"].data_ptr(), b["s_eids"].data_ptr(), b["nvalid"].data_ptr(),
                                            None, 0, None, self.ws.data_ptr(), self.ws.numel(), T, self.E, self.k, 1,
                                            self._stream()), "moe_sorting")
        return b["s_ids"], b["s_eids"]

    def pack(self, xq, x_scale, s_ids, T, chunk: int = 0):
        L, b = self._lib, self.chunk_bufs[chunk]
        P = T * self.k
        L.check(self.lib.flymoe_gather_rows(xq.data_ptr(), b["send_x"].data_ptr(), s_ids.data_ptr(),
                                            b["nvalid"].data_ptr(), T, self.k, self.H, L.ROWS_BY_TOKEN, P,
                                            self._stream()), "gather_rows")
        L.check(self.lib.flymoe_gather_rows(x_scale.data_ptr(), b["send_s"].data_ptr(), s_ids.data_ptr(),
                                            b["nvalid"].data_ptr(), T, self.k, (self.H // 128) * 4, L.ROWS_BY_TOKEN, P,
                                            self._stream()), "gather_rows")
        return b["send_x"], b["send_s"]

    def empty_rows(self, rows: int, like: torch.Tensor) -> torch.Tensor:
        return torch.empty((rows,) + tuple(like.shape[1:]), dtype=like.dtype, device=like.device)

    def row_destinations(self, plan: DispatchPlan, rank: int) -> torch.Tensor:
        """Byte address, in the owning rank's returned-rows buffer, of every received row."""
        row_bytes = self.H * 2
        base, at = [], 0
        for s, (cnt, off) in enumerate(zip(plan.recv_counts, plan.peer_offsets)):
            base.append(self.peers.ptrs[s] + self._off_back + (off - at) * row_bytes)   # + j * row_bytes for row j
            at += cnt
        base_d = torch.tensor(base, dtype=torch.int64, device=self.dev)
        cnt_d = torch.tensor(plan.recv_counts, dtype=torch.int64, device=self.dev)
        rows = plan.rows_in
        return (torch.repeat_interleave(base_d, cnt_d, output_size=rows)
                + torch.arange(rows, dtype=torch.int64, device=self.dev) * row_bytes)

    def peer_rendezvous(self) -> None:
        self.peers.barrier(self._rendezvous_flag)

    def returned_rows(self, pairs: int) -> torch.Tensor:
        back = self.peers.local[self._off_back:self._off_back + pairs * self.H * 2]
        return back.view(torch.bfloat16).view(pairs, self.H)

    # ---- direct dispatch --------------------------------------------------------------------
    def expert_counts(self, s_eids: torch.Tensor, pairs: int) -> torch.Tensor:
        """Rows per global expert from the ascending per-row expert ids of the unit-1 sort (one kernel)."""
        b = self.chunk_bufs[0]
        self._lib.check(self.lib.flymoe_expert_counts(s_eids.data_ptr(), b["nvalid"].data_ptr(),
                                                      self._counts_mine.data_ptr(), self.E, pairs, self._stream()),
                        "expert_counts")
        return self._counts_mine

    def counts_matrix(self, world: int) -> torch.Tensor:
        """The [world, E] buffer the per-expert row counts of all ranks are gathered into."""
        return self._counts_all

    def check_direct_capacity(self, dp: DirectPlan) -> None:
        if dp.max_padded_rows > self.inner.cap_rows:       # same verdict on every rank: all hold the same matrix
            raise RuntimeError(f"a rank would receive {dp.max_padded_rows} padded rows, buffers hold "
                               f"{self.inner.cap_rows}; raise headroom")

    def dispatch_direct(self, xq, x_scale, s_ids, s_eids, dp: DirectPlan, T: int) -> None:
        L, b = self._lib, self.chunk_bufs[0]
        per = self.E_local
        owner = np.arange(self.E) // per
        ptrs = np.asarray(self.peers.ptrs, dtype=np.int64)[owner]
        kb4 = (self.H // 128) * 4
        tables = np.stack([ptrs + self._off_xs + dp.pos_base * self.H, ptrs + self._off_xsc + dp.pos_base * kb4])
        tab = torch.from_numpy(tables).to(self.dev)
        self._tables = tab                                   # alive until the kernel has run
        L.check(self.lib.flymoe_dispatch_rows(xq.data_ptr(), x_scale.data_ptr(), s_ids.data_ptr(), s_eids.data_ptr(),
                                              b["nvalid"].data_ptr(), tab[0].data_ptr(), tab[1].data_ptr(), None, 0,
                                              T, self.k, self.H, self.E, T * self.k, self._stream()), "dispatch_rows")

    def run_direct_on_device(self, xq, x_scale, s_ids, s_eids, counts, rank: int, T: int, phase=None) -> None:
        """Dispatch, local experts and the two rendezvous with the plan computed on the GPU
        (``flymoe_ep_plan_direct``: two small kernels, the arithmetic of ``plan_direct``).  Launch sizes use
        the buffers' capacity; the kernels read the real extents from device memory.  A step that does not
        fit the capacity drops the rows that would fall outside and raises the device status word
        (``flymoe_device_status``) instead of an exception."""
        L, b, inner = self._lib, self.chunk_bufs[0], self.inner
        cap, U, H = inner.cap_rows, self.tile_m, self.H
        tab = self._plan_tables
        L.check(self.lib.flymoe_ep_plan_direct(
            counts.data_ptr(), self._peer_ptrs.data_ptr(), self._off_xs, self._off_xsc, self._off_back,
            tab[0].data_ptr(), tab[1].data_ptr(), tab[2].data_ptr(), inner.sorted_ids.data_ptr(),
            inner.sorted_expert_ids.data_ptr(), inner.num_valid_ids.data_ptr(), self._plan_row_dst.data_ptr(),
            self._plan_ws.data_ptr(), self._plan_ws.numel(), counts.shape[0], rank, self.E, U, H, cap,
            self._stream()), "ep_plan_direct")
        phase = phase or (lambda name: None)
        phase("plan")
        L.check(self.lib.flymoe_dispatch_rows(xq.data_ptr(), x_scale.data_ptr(), s_ids.data_ptr(), s_eids.data_ptr(),
                                              b["nvalid"].data_ptr(), tab[0].data_ptr(), tab[1].data_ptr(),
                                              tab[2].data_ptr(), cap, T, self.k, H, self.E, T * self.k,
                                              self._stream()), "dispatch_rows")
        phase("dispatch")
        self.peer_rendezvous()
        phase("wait_for_peers_rows")
        base_ptr = self.peers.local.data_ptr()
        inner.experts_forward_sorted(base_ptr + self._off_xs, base_ptr + self._off_xsc, cap, cap // U,
                                     self._stream(), self._plan_row_dst)
        phase("stage1_stage2_combine")
        self.peer_rendezvous()
        phase("wait_for_peers_outputs")

    def local_experts_direct(self, dp: DirectPlan) -> None:
        inner, dev = self.inner, self.dev
        rows, blocks = dp.padded_rows, int(dp.block_expert.shape[0])
        if rows == 0:
            return
        row_bytes = self.H * 2
        seg_pos = np.cumsum(dp.seg_len) - dp.seg_len
        src = np.maximum(dp.seg_src, 0)
        base = np.asarray(self.peers.ptrs, dtype=np.int64)[src] + self._off_back + (dp.seg_src_row - seg_pos) * row_bytes
        seg = torch.from_numpy(np.stack([dp.seg_len, (dp.seg_src >= 0).astype(np.int64), base])).to(dev)
        which = torch.repeat_interleave(torch.arange(seg.shape[1], device=dev), seg[0], output_size=rows)
        pos = torch.arange(rows, dtype=torch.int64, device=dev)
        pad_id = (1 << 24) | rows
        inner.sorted_ids[:rows] = torch.where(seg[1][which] != 0, pos, pad_id).to(torch.int32)
        inner.sorted_expert_ids[:blocks] = torch.from_numpy(dp.block_expert).to(dev)
        inner.num_valid_ids.fill_(rows)
        row_dst = seg[2][which] + pos * row_bytes
        base_ptr = self.peers.local.data_ptr()
        inner.experts_forward_sorted(base_ptr + self._off_xs, base_ptr + self._off_xsc, rows, blocks,
                                     self._stream(), row_dst)

    def local_experts(self, recv_x, recv_s, recv_e, first_expert: int, rows: int, chunk: int = 0, row_dst=None):
        self._ensure_inner(rows)
        b = self.chunk_bufs[chunk]
        if row_dst is not None:
            if rows == 0:
                return None
            local_ids = (recv_e - first_expert).view(rows, 1)
            return self.inner.experts_forward(local_ids, self.ones, recv_x, recv_s, rows, self._stream(),
                                              x_scale_row_major=True, row_dst=row_dst)
        if b["y"] is None or b["y"].shape[0] < max(rows, 1):
            b["y"] = torch.empty((max(int(rows * self.headroom), 1), self.H), dtype=torch.bfloat16, device=self.dev)
        if rows == 0:
            return b["y"]
        local_ids = (recv_e - first_expert).view(rows, 1)
        return self.inner.experts_forward(local_ids, self.ones, recv_x, recv_s, rows, self._stream(),
                                          out=b["y"], x_scale_row_major=True)

    def combine(self, back, s_ids, topk_w, lo: int, hi: int, T: int, chunk: int = 0):
        L, b = self._lib, self.chunk_bufs[chunk]
        n = hi - lo
        P = n * self.k
        if self.out_free_event is not None:
            torch.cuda.current_stream().wait_event(self.out_free_event)
        L.check(self.lib.flymoe_sorted_inverse(s_ids.data_ptr(), b["nvalid"].data_ptr(), b["inverse"].data_ptr(),
                                               n, self.k, P, self._stream()), "sorted_inverse")
        L.check(self.lib.flymoe_moe_reduce(back.data_ptr(), self.out[lo:hi].data_ptr(), None, topk_w.data_ptr(),
                                           b["inverse"].data_ptr(), n, self.k, self.H, L.BF16, self._stream()),
                "moe_reduce")
        return self.out
