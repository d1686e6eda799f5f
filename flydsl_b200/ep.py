"""Expert-parallel FP8 block-scaled MoE layer: one process per GPU, experts sharded
evenly over the ranks, tokens dispatched and results combined with NCCL all-to-all.

The reference has no dispatch/combine (its only expert-parallel hook is the
``expert_mask`` of the sort, kernels/moe_sorting_kernel.py:426-440); this module adds the
partitioned case on top of the same kernels:

  1. gate the rank's own tokens over all E experts               (gating kernel)
  2. sort the (token, slot) pairs by global expert id, unit 1     (sort kernels) — rows
     grouped by expert are also grouped by destination rank, and every rank's block
     arrives pre-grouped by local expert
  3. exchange per-rank row counts                                 (all_to_all_single, tiny)
  4. pack e4m3 rows and their fp32 scales in that order           (row-gather kernel)
  5. dispatch rows, scales and expert ids                          (all_to_all_single x3)
  6. local experts: sort by local expert, stage 1, stage 2 into per-row bf16 outputs
  7. combine: send the rows back                                  (all_to_all_single)
  8. out[t] = sum_s w[t,s] * returned_row(t,s)                    (indexed reduce kernel)

Remote data always lands in this GPU's memory before any kernel reads it.  The host-side
bookkeeping (``split_counts``, ``exchange_counts``, the step order in ``forward``) is
device-agnostic so it can be exercised with gloo on CPU ranks through the ``ops`` seam.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def expert_range(rank: int, world: int, experts: int) -> range:
    if experts % world != 0:
        raise ValueError(f"experts ({experts}) must divide evenly over {world} ranks")
    per = experts // world
    return range(rank * per, (rank + 1) * per)


def split_counts(sorted_expert_ids: torch.Tensor, world: int, experts_per_rank: int) -> torch.Tensor:
    """Rows destined to each rank, from the ascending per-row expert ids of the unit-1 sort."""
    bounds = torch.arange(0, world + 1, device=sorted_expert_ids.device,
                          dtype=sorted_expert_ids.dtype) * experts_per_rank
    pos = torch.searchsorted(sorted_expert_ids.contiguous(), bounds.contiguous())
    return (pos[1:] - pos[:-1]).to(torch.int64)


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """all-to-all of one int64 per peer: recv_counts[r] = rows rank r sends to this rank."""
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


class ExpertParallelMoE:
    """Expert-parallel layer.  ``ops`` supplies the device kernels (see ``CudaOps``)."""

    def __init__(self, ops, experts: int, topk: int, model_dim: int, group=None):
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.experts, self.topk, self.H = experts, topk, model_dim
        self.local = expert_range(self.rank, self.world, experts)
        self.per_rank = len(self.local)
        self.last_plan: DispatchPlan | None = None

    def plan(self, sorted_expert_ids_rows: torch.Tensor, pairs: int) -> DispatchPlan:
        send = split_counts(sorted_expert_ids_rows, self.world, self.per_rank)
        recv = exchange_counts(send, self.group)
        both = torch.stack([send, recv]).cpu()          # the one host synchronisation of a step
        check_counts(both[0], both[1], pairs)
        plan = DispatchPlan(both[0].tolist(), both[1].tolist(), int(both[0].sum()), int(both[1].sum()))
        self.last_plan = plan
        return plan

    def forward(self, logits, xq, x_scale):
        """logits [T,E]; xq e4m3 [T,H]; x_scale f32 row-major [T,H/128] -> out [T,H]."""
        ops, k = self.ops, self.topk
        T = logits.shape[0]
        pairs = T * k
        topk_w, topk_ids = ops.gate(logits)
        s_ids, s_eids = ops.sort_by_expert(topk_ids, topk_w, T)          # unit 1: one expert id per row
        plan = self.plan(s_eids[:pairs], pairs)
        send_x, send_s = ops.pack(xq, x_scale, s_ids, T)
        recv_x = ops.empty_rows(plan.rows_in, send_x)
        recv_s = ops.empty_rows(plan.rows_in, send_s)
        recv_e = ops.empty_rows(plan.rows_in, s_eids)
        dist.all_to_all_single(recv_x, send_x[:pairs], plan.recv_counts, plan.send_counts, group=self.group)
        dist.all_to_all_single(recv_s, send_s[:pairs], plan.recv_counts, plan.send_counts, group=self.group)
        dist.all_to_all_single(recv_e, s_eids[:pairs], plan.recv_counts, plan.send_counts, group=self.group)
        y = ops.local_experts(recv_x, recv_s, recv_e, self.local.start, plan.rows_in)
        back = ops.empty_rows(pairs, y)
        dist.all_to_all_single(back, y[:plan.rows_in], plan.send_counts, plan.recv_counts, group=self.group)
        return ops.combine(back, s_ids, topk_w, T)

    __call__ = forward


class CudaOps:
    """The device side of ``ExpertParallelMoE`` on one B200: the library's own kernels."""

    def __init__(self, w1q, w1_scale, w2q, w2_scale, experts: int, topk: int, tokens: int,
                 tile_m: int = 128, headroom: float = 1.3, impl: str = "tcgen05"):
        from . import _lib
        from .layer import FusedMoEBlockscale
        self._lib = _lib
        self.lib = _lib.load()
        self.E, self.k, self.T = experts, topk, tokens
        self.E_local, _, self.H = w1q.shape
        self.I = w2q.shape[2]
        self.tile_m, self.impl = tile_m, impl
        self.w = (w1q, w1_scale, w2q, w2_scale)
        dev = w1q.device
        self.dev = dev
        P = tokens * topk
        i32, f32 = torch.int32, torch.float32
        self.topk_w = torch.empty((tokens, topk), dtype=f32, device=dev)
        self.topk_ids = torch.empty((tokens, topk), dtype=i32, device=dev)
        self.tei = torch.empty((tokens, topk), dtype=i32, device=dev)
        cap = P + experts - topk                        # unit-1 sort: no padding rows
        self.s_ids = torch.empty(cap, dtype=i32, device=dev)
        self.s_w = torch.empty(cap, dtype=f32, device=dev)
        self.s_eids = torch.empty(cap, dtype=i32, device=dev)
        self.nvalid = torch.empty(2, dtype=i32, device=dev)
        ws = int(self.lib.flymoe_moe_sorting_workspace_elems(tokens, experts, topk, 1))
        self.ws = torch.empty(max(ws, 1), dtype=i32, device=dev)
        self.send_x = torch.empty((P, self.H), dtype=torch.uint8, device=dev)
        self.send_s = torch.empty((P, self.H // 128), dtype=f32, device=dev)
        self.inverse = torch.empty(P, dtype=i32, device=dev)
        self.out = torch.empty((tokens, self.H), dtype=torch.bfloat16, device=dev)
        self.headroom = headroom
        self.inner = None
        self._ensure_inner(int(P * headroom))

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

    def sort_by_expert(self, topk_ids, topk_w, T):
        L = self._lib
        L.check(self.lib.flymoe_moe_sorting(topk_ids.data_ptr(), topk_w.data_ptr(), self.s_ids.data_ptr(),
                                            self.s_w.data_ptr(), self.s_eids.data_ptr(), self.nvalid.data_ptr(),
                                            None, 0, None, self.ws.data_ptr(), self.ws.numel(), T, self.E, self.k, 1,
                                            self._stream()), "moe_sorting")
        return self.s_ids, self.s_eids

    def pack(self, xq, x_scale, s_ids, T):
        L = self._lib
        P = T * self.k
        L.check(self.lib.flymoe_gather_rows(xq.data_ptr(), self.send_x.data_ptr(), s_ids.data_ptr(),
                                            self.nvalid.data_ptr(), T, self.k, self.H, L.ROWS_BY_TOKEN, P,
                                            self._stream()), "gather_rows")
        L.check(self.lib.flymoe_gather_rows(x_scale.data_ptr(), self.send_s.data_ptr(), s_ids.data_ptr(),
                                            self.nvalid.data_ptr(), T, self.k, (self.H // 128) * 4, L.ROWS_BY_TOKEN, P,
                                            self._stream()), "gather_rows")
        return self.send_x, self.send_s

    def empty_rows(self, rows: int, like: torch.Tensor) -> torch.Tensor:
        return torch.empty((rows,) + tuple(like.shape[1:]), dtype=like.dtype, device=like.device)

    def local_experts(self, recv_x, recv_s, recv_e, first_expert: int, rows: int):
        self._ensure_inner(rows)
        if rows == 0:
            return torch.empty((0, self.H), dtype=torch.bfloat16, device=self.dev)
        local_ids = (recv_e - first_expert).view(rows, 1)
        return self.inner.experts_forward(local_ids, self.ones, recv_x, recv_s, rows, self._stream(),
                                          x_scale_row_major=True)

    def combine(self, back, s_ids, topk_w, T):
        L = self._lib
        P = T * self.k
        L.check(self.lib.flymoe_sorted_inverse(s_ids.data_ptr(), self.nvalid.data_ptr(), self.inverse.data_ptr(),
                                               T, self.k, P, self._stream()), "sorted_inverse")
        L.check(self.lib.flymoe_moe_reduce(back.data_ptr(), self.out.data_ptr(), None, topk_w.data_ptr(),
                                           self.inverse.data_ptr(), T, self.k, self.H, L.BF16, self._stream()),
                "moe_reduce")
        return self.out
