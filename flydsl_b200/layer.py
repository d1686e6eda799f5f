"""Fused FP8 block-scaled MoE layer: gating -> sort -> stage 1 -> stage 2 on one GPU.

The same five kernels that back ``flydsl_b200.kernels.*``, chained without the
reference's intermediate round trips: stage 1 writes the e4m3 intermediate and its
1x128 scales directly in sorted-row order, so stage 2 reads contiguous rows by TMA and
no separate requantisation or second gather runs.  All buffers are allocated once at
construction for ``max_tokens``; ``forward`` only enqueues kernels on the current
stream (no allocation, no host synchronisation).
"""

from __future__ import annotations

import torch

from . import _lib

_FP8 = (torch.float8_e4m3fn, torch.uint8)


class FusedMoEBlockscale:
    """One MoE layer with e4m3 weights in plain row-major order.

    w1q [E, 2I, H] (gate rows first), w1_scale f32 [E, 2I/128, H/128],
    w2q [E, H, I], w2_scale f32 [E, H/128, I/128].  ``tile_m`` is both the sort
    unit and the GEMM row-block (16/32/64/128).
    """

    def __init__(self, w1q, w1_scale, w2q, w2_scale, topk: int, *, max_tokens: int, tile_m: int = 128,
                 out_dtype=torch.bfloat16, renormalize: bool = True, stage2_mode: str = "atomic",
                 impl: str = "tcgen05", num_router_experts: int | None = None):
        E, two_i, H = w1q.shape
        I = two_i // 2
        if tuple(w2q.shape) != (E, H, I):
            raise ValueError(f"w2q must be [E, H, I] = {(E, H, I)}, got {tuple(w2q.shape)}")
        if H % 128 or I % 128:
            raise ValueError("model_dim and inter_dim must be multiples of 128")
        if stage2_mode not in ("atomic", "reduce", "rows"):
            raise ValueError("stage2_mode must be 'atomic', 'reduce' or 'rows'")
        if stage2_mode == "rows" and int(topk) != 1:
            raise ValueError("stage2_mode='rows' (one unweighted output row per input row) needs topk == 1")
        if out_dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("out_dtype must be torch.bfloat16 or torch.float16")
        for name, t, dts in (("w1q", w1q, _FP8), ("w2q", w2q, _FP8), ("w1_scale", w1_scale, (torch.float32,)),
                             ("w2_scale", w2_scale, (torch.float32,))):
            _lib.require_cuda(name, t, dts)
        self.lib = _lib.load()
        self.w1q, self.w1_scale, self.w2q, self.w2_scale = w1q, w1_scale, w2q, w2_scale
        self.E, self.H, self.I, self.topk = E, H, I, int(topk)
        self.router_experts = int(num_router_experts) if num_router_experts is not None else E
        self.tile_m, self.max_tokens = int(tile_m), int(max_tokens)
        self.out_dtype, self.renormalize = out_dtype, bool(renormalize)
        self.stage2_mode = stage2_mode
        self.impl = {"tcgen05": _lib.IMPL_TCGEN05, "simt": _lib.IMPL_SIMT}[impl]
        dev = w1q.device
        self.device = dev
        T, k, U = self.max_tokens, self.topk, self.tile_m
        self.capacity = T * k + E * U - k
        self.blocks = (self.capacity + U - 1) // U
        self.cap_rows = self.blocks * U
        i32, f32 = torch.int32, torch.float32
        self.topk_weights = torch.empty((T, k), dtype=f32, device=dev)
        self.topk_ids = torch.empty((T, k), dtype=i32, device=dev)
        self.tei = torch.empty((T, k), dtype=i32, device=dev)
        self.sorted_ids = torch.empty(self.cap_rows, dtype=i32, device=dev)
        self.sorted_weights = torch.empty(self.cap_rows, dtype=f32, device=dev)
        self.sorted_expert_ids = torch.empty(self.blocks, dtype=i32, device=dev)
        self.num_valid_ids = torch.zeros(2, dtype=i32, device=dev)
        ws = int(self.lib.flymoe_moe_sorting_workspace_elems(T, E, k, U))
        self.workspace = torch.empty(max(ws, 1), dtype=i32, device=dev)
        # Row blocks of 16 or 32 rows: stage 1 fetches each sorted row's activations by token id inside
        # the kernel.  Larger blocks: a gather kernel copies them into sorted order first (faster there).
        self.gather_in_kernel = self.tile_m <= 32
        self.xs = None if self.gather_in_kernel else torch.empty((self.cap_rows, H), dtype=torch.uint8, device=dev)
        self.a2q = torch.empty((self.cap_rows, I), dtype=torch.uint8, device=dev)
        self.a2_scale = torch.empty((I // 128, self.cap_rows), dtype=f32, device=dev)
        self.out = torch.empty((T, H), dtype=out_dtype, device=dev)
        self.pair_out = (torch.empty((T * k, H), dtype=out_dtype, device=dev)
                         if stage2_mode == "reduce" else None)
        self.out_code = _lib.DTYPE_CODE[out_dtype]
        # When set to a list, forward() appends ("gemm1"|"gemm2", start, end) CUDA events recorded
        # on torch's current stream around the two GEMM launches (used by the benchmark).
        self.timing_events = None

    def _mark(self):
        if self.timing_events is None:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream())
        return ev

    # ---------------------------------------------------------------- pieces
    def gate(self, logits: torch.Tensor, tokens: int, stream: int) -> None:
        _lib.require_cuda("logits", logits, (torch.float32, torch.float16, torch.bfloat16),
                          tokens * self.router_experts)
        _lib.check(self.lib.flymoe_topk_gating_softmax(
            logits.data_ptr(), _lib.DTYPE_CODE[logits.dtype], self.topk_weights.data_ptr(),
            self.topk_ids.data_ptr(), self.tei.data_ptr(), tokens, self.router_experts, self.topk,
            1 if self.renormalize else 0, stream), "topk_gating_softmax")

    def experts_forward(self, topk_ids, topk_weights, xq, x_scale_t, tokens: int, stream: int,
                        out: torch.Tensor | None = None, x_scale_row_major: bool = False,
                        row_dst: torch.Tensor | None = None) -> torch.Tensor:
        """sort -> (gather, for row blocks of 64 or 128 rows) -> stage 1 -> stage 2 for already-routed tokens.

        topk_ids i32 [tokens, k] (ids in [0, E) of this layer's experts; ids outside
        that range are ignored), topk_weights f32 [tokens, k], xq e4m3 [tokens, H],
        x_scale_t f32 [H/128, tokens] (or row-major [tokens, H/128] with
        ``x_scale_row_major``).  stage2_mode "atomic": weighted atomic accumulation into the
        zeroed ``out``; "reduce": per-pair rows then a weighted top-k reduce (deterministic);
        "rows" (topk == 1): the unweighted expert output of every input row; with ``row_dst``
        (int64 [tokens], byte addresses, 0 = drop) each row is stored to its own address --
        possibly in a peer GPU's mapped memory -- instead of ``out``.
        """
        T, k, U, E, H, I = tokens, self.topk, self.tile_m, self.E, self.H, self.I
        if T > self.max_tokens:
            raise ValueError(f"tokens={T} exceeds max_tokens={self.max_tokens}")
        _lib.require_cuda("xq", xq, _FP8, T * H)
        _lib.require_cuda("x_scale_t", x_scale_t, (torch.float32,), (H // 128) * T)
        out = self.out if out is None else out
        _lib.require_cuda("out", out, (self.out_dtype,), T * H)
        lib = self.lib
        capacity = T * k + E * U - k
        blocks = (capacity + U - 1) // U
        cap_rows = blocks * U
        _lib.check(lib.flymoe_moe_sorting(
            topk_ids.data_ptr(), topk_weights.data_ptr(), self.sorted_ids.data_ptr(),
            self.sorted_weights.data_ptr(), self.sorted_expert_ids.data_ptr(), self.num_valid_ids.data_ptr(),
            out.data_ptr() if self.stage2_mode == "atomic" else None,
            T * H * out.element_size() if self.stage2_mode == "atomic" else 0, None, self.workspace.data_ptr(),
            self.workspace.numel(), T, E, k, U, stream), "moe_sorting")
        if not self.gather_in_kernel:
            _lib.check(lib.flymoe_gather_rows(
                xq.data_ptr(), self.xs.data_ptr(), self.sorted_ids.data_ptr(), self.num_valid_ids.data_ptr(),
                T, k, H, _lib.ROWS_BY_TOKEN, cap_rows, stream), "gather_rows")
        sx_stride, sx_row_stride = (1, H // 128) if x_scale_row_major else (x_scale_t.numel() // (H // 128), 1)
        t0 = self._mark()
        _lib.check(lib.flymoe_moe_gemm1(
            self.a2q.data_ptr(), self.a2_scale.data_ptr(), self.cap_rows,
            xq.data_ptr() if self.gather_in_kernel else self.xs.data_ptr(),
            x_scale_t.data_ptr(), sx_stride, sx_row_stride, self.w1q.data_ptr(), self.w1_scale.data_ptr(),
            self.sorted_ids.data_ptr(), self.sorted_expert_ids.data_ptr(), self.sorted_weights.data_ptr(),
            self.num_valid_ids.data_ptr(), T, I, H, blocks, E, k, U, 0, _lib.E4M3,
            _lib.ROWS_BY_TOKEN if self.gather_in_kernel else _lib.ROWS_SORTED,
            _lib.ROWS_BY_TOKEN, _lib.ROWS_SORTED, self.impl, stream), "moe_gemm1")
        t1 = self._mark()
        accumulate = self.stage2_mode == "atomic"
        target = self.pair_out if self.stage2_mode == "reduce" else out
        if row_dst is not None:
            if self.stage2_mode != "rows":
                raise ValueError("row_dst needs stage2_mode='rows'")
            _lib.require_cuda("row_dst", row_dst, (torch.int64,), T)
            _lib.check(lib.flymoe_moe_gemm2_scatter_rows(
                row_dst.data_ptr(), self.a2q.data_ptr(), self.a2_scale.data_ptr(), self.cap_rows,
                self.w2q.data_ptr(), self.w2_scale.data_ptr(), self.sorted_ids.data_ptr(),
                self.sorted_expert_ids.data_ptr(), self.sorted_weights.data_ptr(), self.num_valid_ids.data_ptr(),
                T, H, I, blocks, E, k, U, 0, self.out_code, _lib.ROWS_SORTED, _lib.ROWS_SORTED, stream),
                "moe_gemm2_scatter_rows")
            if self.timing_events is not None:
                self.timing_events.append(("gemm1", t0, t1))
                self.timing_events.append(("gemm2", t1, self._mark()))
            return out
        _lib.check(lib.flymoe_moe_gemm2(
            target.data_ptr(), self.a2q.data_ptr(), self.a2_scale.data_ptr(), self.cap_rows,
            self.w2q.data_ptr(), self.w2_scale.data_ptr(), self.sorted_ids.data_ptr(),
            self.sorted_expert_ids.data_ptr(), self.sorted_weights.data_ptr(), self.num_valid_ids.data_ptr(),
            T, H, I, blocks, E, k, U, 1 if accumulate else 0, self.out_code, 1 if accumulate else 0,
            _lib.ROWS_SORTED, _lib.ROWS_SORTED, self.impl, stream), "moe_gemm2")
        if self.timing_events is not None:
            self.timing_events.append(("gemm1", t0, t1))
            self.timing_events.append(("gemm2", t1, self._mark()))
        if self.stage2_mode == "reduce":
            # per-pair rows hold the unweighted expert outputs; weight and sum them here
            _lib.check(lib.flymoe_moe_reduce(
                self.pair_out.data_ptr(), out.data_ptr(), None, topk_weights.data_ptr(), None, T, k, H,
                self.out_code, stream), "moe_reduce")
        return out

    def experts_forward_sorted(self, xs_ptr: int, x_scale_ptr: int, rows: int, blocks: int, stream: int,
                               row_dst: torch.Tensor) -> None:
        """Stage 1 and stage 2 over rows that already sit in sorted, block-padded order.

        ``xs_ptr``: e4m3 [rows, H]; ``x_scale_ptr``: f32 row-major [rows, H/128]; the caller has
        filled ``self.sorted_ids[:rows]`` (row index, or a pad id), ``self.sorted_expert_ids[:blocks]``
        and ``self.num_valid_ids[0] = rows``.  Every valid row's output goes to ``row_dst[row]``
        (int64 byte addresses).  Used by the expert-parallel layer, whose dispatch kernel writes
        the rows into this layout on the receiving GPU."""
        if self.stage2_mode != "rows":
            raise ValueError("experts_forward_sorted needs stage2_mode='rows'")
        if rows > self.cap_rows or blocks > self.blocks or blocks * self.tile_m != rows:
            raise ValueError(f"rows={rows} / blocks={blocks} do not fit this layer (cap_rows={self.cap_rows})")
        if rows == 0:
            return
        _lib.require_cuda("row_dst", row_dst, (torch.int64,), rows)
        lib, E, H, I, U = self.lib, self.E, self.H, self.I, self.tile_m
        t0 = self._mark()
        _lib.check(lib.flymoe_moe_gemm1(
            self.a2q.data_ptr(), self.a2_scale.data_ptr(), self.cap_rows, xs_ptr, x_scale_ptr, 1, H // 128,
            self.w1q.data_ptr(), self.w1_scale.data_ptr(), self.sorted_ids.data_ptr(),
            self.sorted_expert_ids.data_ptr(), self.sorted_weights.data_ptr(), self.num_valid_ids.data_ptr(),
            rows, I, H, blocks, E, 1, U, 0, _lib.E4M3, _lib.ROWS_SORTED, _lib.ROWS_SORTED, _lib.ROWS_SORTED,
            self.impl, stream), "moe_gemm1")
        t1 = self._mark()
        _lib.check(lib.flymoe_moe_gemm2_scatter_rows(
            row_dst.data_ptr(), self.a2q.data_ptr(), self.a2_scale.data_ptr(), self.cap_rows,
            self.w2q.data_ptr(), self.w2_scale.data_ptr(), self.sorted_ids.data_ptr(),
            self.sorted_expert_ids.data_ptr(), self.sorted_weights.data_ptr(), self.num_valid_ids.data_ptr(),
            rows, H, I, blocks, E, 1, U, 0, self.out_code, _lib.ROWS_SORTED, _lib.ROWS_SORTED, stream),
            "moe_gemm2_scatter_rows")
        if self.timing_events is not None:
            self.timing_events.append(("gemm1", t0, t1))
            self.timing_events.append(("gemm2", t1, self._mark()))

    # ---------------------------------------------------------------- whole layer
    def forward(self, logits: torch.Tensor, xq: torch.Tensor, x_scale_t: torch.Tensor,
                out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """logits [T, E] (f32/f16/bf16), xq e4m3 [T, H], x_scale_t f32 [H/128, T] -> out [T, H]."""
        tokens = logits.shape[0]
        h = _lib.stream_handle(stream)
        self.gate(logits, tokens, h)
        res = self.experts_forward(self.topk_ids, self.topk_weights, xq, x_scale_t, tokens, h, out)
        return res[:tokens] if res.shape[0] != tokens else res

    __call__ = forward

    def kernel_launches(self, tokens: int) -> int:
        """Kernels this layer enqueues per forward (memset of the output not counted)."""
        sort = 1 if tokens * self.topk <= 8192 else 3
        return 1 + sort + (0 if self.gather_in_kernel else 1) + 1 + 1 + (1 if self.stage2_mode == "reduce" else 0)

    def experts_kernel_launches(self, rows: int) -> int:
        """Kernels experts_forward enqueues for ``rows`` input rows."""
        return self.kernel_launches(rows) - 1


def quant_act_1x128(x: torch.Tensor, stream=None):
    """bf16/f16/f32 [R, K] -> (q e4m3 [R, K], scale f32 transposed [K/128, R]) on the GPU."""
    _lib.require_cuda("x", x, (torch.bfloat16, torch.float16, torch.float32))
    R, K = x.shape
    if K % 128:
        raise ValueError("K must be a multiple of 128")
    q = torch.empty((R, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((K // 128, R), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().flymoe_quant_act_1x128(x.data_ptr(), _lib.DTYPE_CODE[x.dtype], q.data_ptr(),
                                                  s.data_ptr(), R, R, K, _lib.stream_handle(stream)),
               "quant_act_1x128")
    return q, s
