"""Two-stage MoE GEMMs with per-token / per-channel scales for B200.

Mirrors ``kernels/moe_gemm_2stage.py`` of the reference for its 8-bit and 16-bit variants:

* ``compile_moe_gemm1`` (:90-108) -> launcher with the positional order of :1730-1745
  ``(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
  max_token_ids, tokens, inter, k, size_expert_ids, stream)``
* ``compile_moe_gemm2`` (:1780-1796) -> launcher of :3151-3166
* ``compile_moe_reduction`` (:3202), ``MoeGemm2Mode`` (:3405), ``compile_moe_gemm2_ex`` (:3517)

Data contract (the reference's, tests/kernels/test_moe_gemm.py:446-450, :548-579):
``in_dtype="fp8"``: x e4m3 [tokens, K] with ONE fp32 scale per token ([tokens]); weights e4m3
[E, N, K] with ONE fp32 scale per weight row ([E*N]).  ``"int8"``: the same with signed 8-bit
operands (exact int32 accumulation).  ``"int8smooth"``: x and its scales are given per (token,
slot) pair in slot-major order ([topk*tokens, K], [topk*tokens]: row ``slot*tokens + token``, :546-555).  Stage 1 writes ``silu(gate)*up`` to row
``t*topk + s`` of a [tokens, topk, inter] f16/bf16 tensor; stage 2 reads that layout (e4m3/int8
plus one scale per row) and accumulates ``sorted_weight * (a2 . W2^T)`` into ``out[t]``
(pre-zeroed; f16/bf16/f32) or, with ``accumulate=False``, stores per-pair rows.
``"fp16"`` / ``"bf16"``: x, the weights and the stage-2 input are 16-bit floats and there are no
scales (the scale arguments are ignored; the reference passes empty tensors, :569-579 of its test).

With one scale per row and column the whole K range is accumulated inside the tensor cores'
accumulator memory and every tile is scaled once, ``(sum_k a*w) * scale_a[row] * scale_w[col]``.

``"int4"`` (W4A8) / ``"int4_bf16"`` (W4A16): the weights arrive as the reference's packed int4 bytes
(its test's ``_pack_shuffled_int8_to_packed_int4_no_perm`` over the preshuffled values, ``N*K/2`` bytes)
with one fp32 scale per weight row; x is int8 with per-token scales, or bf16 without.  The packed
tensor is unpacked once per weight tensor (like the preshuffle conversion) to int8 or bf16 and the
int8 / bf16 kernels run on the copy: same results, without the memory saving of 4-bit weights.

``"int4_bf16"`` with ``group_size=32``: ``arg_scale_w`` holds group-wise scales in the reference's kernel
layout (f32 ``[E, K/32, N]``, or with ``scale_is_bf16`` bf16 ``[E, K/64, N, 2]``) instead of one per weight
row; they are multiplied in while unpacking (``bf16(value * scale)``), after which the scale-less bf16 kernel
runs.

``k_batch > 1`` (stage 1): the reference's split-K launches add the scaled gate and up sums, without
activation and routing weight, to a caller-zeroed fp32 ``[tokens*topk, 2*inter]`` buffer and the caller
finishes ``silu(gate)*up`` (:121-122; its test :582-587, :708-713).  The launcher built here keeps that
output contract; K is not actually split (one CTA sums the whole K range and adds once per element).

Not built here: ``k_batch > 1`` with bf16 activations (bf16 partial sums) and group-wise scales with int8
activations (``in_dtype="int4"`` with ``group_size > 0``) raise ``ValueError`` at build time; ``group_size`` other than 32 is rejected as in
the reference and ignored for the variants without packed weights.
Additions (keyword-only): ``w_layout`` ("preshuffle16x16" default, or "plain") and ``impl``
("tcgen05" default, "simt" cross-check) as in ``moe_blockscale_2stage``.
"""

from __future__ import annotations

import functools

import torch

from .. import _lib
from .moe_blockscale_2stage import (MoeGemm2Mode, _GATHER_IN_KERNEL_MAX, _IMPL, _LauncherScratch, _MoeGemm2ReduceWrapper, _OUT16,
                                    _plain_weight, _resolve_scratch, compile_moe_reduction, logger)

_VALID_IN = ("fp8", "fp16", "bf16", "int8", "int8smooth", "int4", "int4_bf16")
_BUILT_IN = _VALID_IN
# activation dtypes; the weights have the same type except for the packed-int4 variants (int8/uint8 bytes)
_IN_TORCH = {"fp8": (torch.float8_e4m3fn, torch.uint8), "int8": (torch.int8,), "int8smooth": (torch.int8,),
             "fp16": (torch.float16,), "bf16": (torch.bfloat16,), "int4": (torch.int8,), "int4_bf16": (torch.bfloat16,)}
_IN_CODE = {"fp8": _lib.E4M3, "int8": _lib.I8, "int8smooth": _lib.I8, "fp16": _lib.F16, "bf16": _lib.BF16,
            "int4": _lib.I8, "int4_bf16": _lib.BF16}
_INT4_TO = {"int4": torch.int8, "int4_bf16": torch.bfloat16}          # what the packed weights are unpacked to
_PACKED_W = (torch.int8, torch.uint8)
_TILE_M = (16, 32, 64, 128)


def _check(in_dtype, group_size, k_batch, tile_m, tile_k, model_dim, inter_dim, experts, topk, w_layout, impl):
    if in_dtype not in _VALID_IN:
        raise ValueError(f"in_dtype must be one of {_VALID_IN}, got {in_dtype!r}")
    if in_dtype not in _BUILT_IN:
        raise ValueError(f"in_dtype={in_dtype!r} is not built on this implementation (built: {_BUILT_IN})")
    # group_size only means something with packed int4 weights (the reference ignores it otherwise)
    if group_size > 0 and in_dtype == "int4":
        raise ValueError("group-wise weight scales are built for in_dtype='int4_bf16' only: with int8 activations "
                         "the scales cannot be folded into the unpacked weights")
    if group_size > 0 and in_dtype == "int4_bf16" and group_size != 32:
        raise ValueError(f"FlyDSL groupwise scale only supports group_size=32, got {group_size}. "
                         "This is due to int4 preshuffle layout constraints.")
    if in_dtype in _INT4_TO and w_layout != "preshuffle16x16":
        raise ValueError("packed int4 weights are defined on the preshuffled order: w_layout must be 'preshuffle16x16'")
    if k_batch < 1:
        raise ValueError(f"k_batch must be >= 1, got {k_batch}")
    if k_batch > 1:
        # split-K launches keep the reference's OUTPUT contract (raw fp32 gate|up sums added to a zeroed
        # [tokens*topk, 2*inter] buffer); K itself is not split here, one CTA owns the whole K range of a tile
        if in_dtype in ("bf16", "int4_bf16"):
            raise ValueError("k_batch > 1 with bf16 activations accumulates bf16 partial sums in the reference; "
                             "that output format is not built here")
        if model_dim % k_batch:
            raise ValueError(f"model_dim={model_dim} not divisible by k_batch={k_batch}")
        if (model_dim // k_batch) % tile_k:
            raise ValueError(f"K_per_batch={model_dim // k_batch} not divisible by tile_k={tile_k}")
        if impl != "tcgen05":
            raise ValueError("k_batch > 1 is built for the tensor-core path only (impl='tcgen05')")
    if tile_k % 64 != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got tile_k_bytes={tile_k} (tile_k={tile_k}, elem_bytes=1)")
    if (tile_m * tile_k) % 256 != 0:
        raise ValueError(f"tile_m*tile_k*elem_bytes must be divisible by 256: tile_m={tile_m}, tile_k={tile_k}, elem_bytes=1")
    if model_dim % 128 or inter_dim % 128:
        raise ValueError(f"model_dim ({model_dim}) and inter_dim ({inter_dim}) must be multiples of 128 on this implementation")
    if experts < 1 or topk < 1 or topk > 255:
        raise ValueError(f"experts/topk out of range: experts={experts}, topk={topk}")
    if w_layout not in ("preshuffle16x16", "plain"):
        raise ValueError(f"w_layout must be 'preshuffle16x16' or 'plain', got {w_layout!r}")
    if impl not in _IMPL:
        raise ValueError(f"impl must be one of {sorted(_IMPL)}, got {impl!r}")
    if impl != "tcgen05" and in_dtype in ("fp16", "bf16", "int4_bf16"):
        raise ValueError("16-bit operands are built for the tensor-core path only (impl='tcgen05')")
    if impl == "tcgen05" and tile_m not in _TILE_M:
        raise ValueError(f"tile_m must be one of {_TILE_M} for the tensor-core path, got {tile_m}")


@functools.lru_cache(maxsize=1024)
def compile_moe_gemm1(*, model_dim: int, inter_dim: int, experts: int, topk: int, tile_m: int, tile_n: int,
                      tile_k: int, doweight_stage1: bool, in_dtype: str = "fp8", group_size: int = -1,
                      out_dtype: str = "f16", use_cshuffle_epilog: bool | None = None, scale_is_bf16: bool = False,
                      k_batch: int = 1, w_layout: str = "preshuffle16x16", impl: str = "tcgen05"):
    """Build the stage-1 launcher (gate/up grouped GEMM + SiLU(gate)*up, per-token scales)."""
    if out_dtype not in ("f16", "bf16"):
        raise ValueError(f"out_dtype must be 'f16' or 'bf16', got {out_dtype!r}")
    _check(in_dtype, group_size, k_batch, tile_m, tile_k, model_dim, inter_dim, experts, topk, w_layout, impl)
    if use_cshuffle_epilog is not None:
        logger.debug("stage 1: use_cshuffle_epilog does not apply here and is ignored")
    impl_code = _IMPL[impl]
    in_code = _IN_CODE[in_dtype]
    in_torch = _IN_TORCH[in_dtype]
    grouped = group_size > 0 and in_dtype == "int4_bf16"     # group-wise weight scales, folded in while unpacking
    no_x_scale = in_dtype in ("fp16", "bf16", "int4_bf16")
    no_w_scale = in_dtype in ("fp16", "bf16") or grouped
    ebytes = 2 if no_x_scale else 1
    int4_to = _INT4_TO.get(in_dtype)
    w_torch = _PACKED_W if int4_to is not None else in_torch
    gs_torch = (torch.bfloat16,) if scale_is_bf16 else (torch.float32,)
    raw_sums = k_batch > 1                     # the split-K output contract: fp32 gate|up sums, [tokens*topk, 2*inter]
    out_torch = torch.float32 if raw_sums else _OUT16[out_dtype]
    out_code = _lib.DTYPE_CODE[out_torch]
    by_pair = in_dtype == "int8smooth"          # x and scale_x per (token, slot), slot-major: row s*tokens + t
    wrows = experts * 2 * inter_dim
    scratch = _LauncherScratch(torch.uint8)

    def launch_moe_gemm1(arg_out, arg_x, arg_w, arg_scale_x, arg_scale_w, arg_sorted_token_ids, arg_expert_ids,
                         arg_sorted_weights, arg_max_token_ids, tokens_in, inter_in, k_in, size_expert_ids_in,
                         stream=None, *, gather_buffer=None):
        tokens, blocks = int(tokens_in), int(size_expert_ids_in)
        if int(inter_in) != inter_dim or int(k_in) != model_dim:
            raise ValueError(f"launcher built for inter_dim={inter_dim}, model_dim={model_dim}; "
                             f"called with inter={inter_in}, k={k_in}")
        cap_rows = blocks * tile_m
        pairs = tokens * topk
        x_rows = pairs if by_pair else tokens
        _lib.require_cuda("arg_out", arg_out, (out_torch,), pairs * inter_dim * (2 if raw_sums else 1))
        _lib.require_cuda("arg_x", arg_x, in_torch, x_rows * model_dim)
        _lib.require_cuda("arg_w", arg_w, w_torch, wrows * model_dim // (2 if int4_to is not None else 1))
        if not no_x_scale:
            _lib.require_cuda("arg_scale_x", arg_scale_x, (torch.float32,), x_rows)
        if not no_w_scale:
            _lib.require_cuda("arg_scale_w", arg_scale_w, (torch.float32,), wrows)
        sx_ptr = 0 if no_x_scale else _lib.ptr(arg_scale_x)
        sw_ptr = 0 if no_w_scale else _lib.ptr(arg_scale_w)
        _lib.require_cuda("arg_sorted_token_ids", arg_sorted_token_ids, (torch.int32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_expert_ids", arg_expert_ids, (torch.int32,), blocks)
        _lib.require_cuda("arg_sorted_weights", arg_sorted_weights, (torch.float32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_max_token_ids", arg_max_token_ids, (torch.int32,), 1)
        h = _lib.stream_handle(stream)
        lib = _lib.load()
        if grouped:
            _lib.require_cuda("arg_scale_w", arg_scale_w, gs_torch, wrows * (model_dim // 32))
        w_plain = _plain_weight(arg_w, wrows, model_dim, w_layout, h, int4_to, arg_scale_w if grouped else None,
                                2 * inter_dim)
        row_layout = _lib.ROWS_BY_SLOT if by_pair else _lib.ROWS_BY_TOKEN
        x_ptr, x_layout = _lib.ptr(arg_x), row_layout
        if impl_code == _lib.IMPL_TCGEN05 and tile_m > _GATHER_IN_KERNEL_MAX:
            gbuf = _resolve_scratch(scratch, gather_buffer, "gather_buffer", arg_x.device, h,
                                    cap_rows * model_dim * ebytes)
            _lib.check(lib.flymoe_gather_rows(x_ptr, _lib.ptr(gbuf), _lib.ptr(arg_sorted_token_ids),
                                              _lib.ptr(arg_max_token_ids), tokens, topk, model_dim * ebytes, row_layout,
                                              cap_rows, h), "gather_rows")
            x_ptr, x_layout = _lib.ptr(gbuf), _lib.ROWS_SORTED
        _lib.check(lib.flymoe_moe_gemm1_pertoken(
            _lib.ptr(arg_out), x_ptr, sx_ptr, _lib.ptr(w_plain), sw_ptr,
            _lib.ptr(arg_sorted_token_ids), _lib.ptr(arg_expert_ids), _lib.ptr(arg_sorted_weights),
            _lib.ptr(arg_max_token_ids), tokens, inter_dim, model_dim, blocks, experts, topk, tile_m,
            1 if doweight_stage1 else 0, in_code, out_code, x_layout, row_layout, _lib.ROWS_BY_PAIR, impl_code, h),
            "moe_gemm1_pertoken")

    return launch_moe_gemm1


@functools.lru_cache(maxsize=1024)
def compile_moe_gemm2(*, model_dim: int, inter_dim: int, experts: int, topk: int, tile_m: int, tile_n: int,
                      tile_k: int, doweight_stage2: bool, in_dtype: str = "fp8", group_size: int = -1,
                      out_dtype: str = "f16", use_cshuffle_epilog: bool | None = None, accumulate: bool = True,
                      scale_is_bf16: bool = False, w_layout: str = "preshuffle16x16", impl: str = "tcgen05"):
    """Build the stage-2 launcher (down grouped GEMM + weighted scatter-reduce, per-token scales)."""
    out_s = str(out_dtype).strip().lower()
    if out_s not in ("f16", "fp16", "half", "bf16", "bfloat16", "f32", "fp32", "float"):
        raise ValueError(f"out_dtype must be 'f16', 'bf16', or 'f32', got {out_dtype!r}")
    out_is_f32 = out_s in ("f32", "fp32", "float")
    out_is_bf16 = out_s in ("bf16", "bfloat16")
    if (not bool(accumulate)) and out_is_f32:
        raise ValueError("compile_moe_gemm2(accumulate=False) only supports out_dtype in {'f16','bf16'}")
    _check(in_dtype, group_size, 1, tile_m, tile_k, model_dim, inter_dim, experts, topk, w_layout, impl)
    if use_cshuffle_epilog is not None:
        logger.debug("stage 2: use_cshuffle_epilog does not apply here and is ignored")
    impl_code = _IMPL[impl]
    in_code = _IN_CODE[in_dtype]
    in_torch = _IN_TORCH[in_dtype]
    grouped = group_size > 0 and in_dtype == "int4_bf16"
    no_x_scale = in_dtype in ("fp16", "bf16", "int4_bf16")
    no_w_scale = in_dtype in ("fp16", "bf16") or grouped
    ebytes = 2 if no_x_scale else 1
    int4_to = _INT4_TO.get(in_dtype)
    w_torch = _PACKED_W if int4_to is not None else in_torch
    gs_torch = (torch.bfloat16,) if scale_is_bf16 else (torch.float32,)
    out_torch = torch.float32 if out_is_f32 else (torch.bfloat16 if out_is_bf16 else torch.float16)
    out_code = _lib.DTYPE_CODE[out_torch]
    wrows = experts * model_dim
    acc = 1 if accumulate else 0
    scratch = _LauncherScratch(torch.uint8)

    def launch_moe_gemm2(arg_out, arg_x, arg_w, arg_scale_x, arg_scale_w, arg_sorted_token_ids, arg_expert_ids,
                         arg_sorted_weights, arg_num_valid_ids, tokens_in, n_in, k_in, size_expert_ids_in,
                         stream=None, *, gather_buffer=None):
        tokens, blocks = int(tokens_in), int(size_expert_ids_in)
        if int(n_in) != model_dim or int(k_in) != inter_dim:
            raise ValueError(f"launcher built for model_dim={model_dim}, inter_dim={inter_dim}; "
                             f"called with n={n_in}, k={k_in}")
        cap_rows = blocks * tile_m
        pairs = tokens * topk
        out_rows = tokens if accumulate else pairs
        _lib.require_cuda("arg_out", arg_out, (out_torch,), out_rows * model_dim)
        _lib.require_cuda("arg_x", arg_x, in_torch, pairs * inter_dim)
        _lib.require_cuda("arg_w", arg_w, w_torch, wrows * inter_dim // (2 if int4_to is not None else 1))
        if not no_x_scale:
            _lib.require_cuda("arg_scale_x", arg_scale_x, (torch.float32,), pairs)
        if not no_w_scale:
            _lib.require_cuda("arg_scale_w", arg_scale_w, (torch.float32,), wrows)
        sx_ptr = 0 if no_x_scale else _lib.ptr(arg_scale_x)
        sw_ptr = 0 if no_w_scale else _lib.ptr(arg_scale_w)
        _lib.require_cuda("arg_sorted_token_ids", arg_sorted_token_ids, (torch.int32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_expert_ids", arg_expert_ids, (torch.int32,), blocks)
        _lib.require_cuda("arg_sorted_weights", arg_sorted_weights, (torch.float32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_num_valid_ids", arg_num_valid_ids, (torch.int32,), 1)
        h = _lib.stream_handle(stream)
        lib = _lib.load()
        if grouped:
            _lib.require_cuda("arg_scale_w", arg_scale_w, gs_torch, wrows * (inter_dim // 32))
        w_plain = _plain_weight(arg_w, wrows, inter_dim, w_layout, h, int4_to, arg_scale_w if grouped else None,
                                model_dim)
        a_ptr, a_layout = _lib.ptr(arg_x), _lib.ROWS_BY_PAIR
        if impl_code == _lib.IMPL_TCGEN05 and tile_m > _GATHER_IN_KERNEL_MAX:
            gbuf = _resolve_scratch(scratch, gather_buffer, "gather_buffer", arg_x.device, h,
                                    cap_rows * inter_dim * ebytes)
            _lib.check(lib.flymoe_gather_rows(a_ptr, _lib.ptr(gbuf), _lib.ptr(arg_sorted_token_ids),
                                              _lib.ptr(arg_num_valid_ids), tokens, topk, inter_dim * ebytes,
                                              _lib.ROWS_BY_PAIR, cap_rows, h), "gather_rows")
            a_ptr, a_layout = _lib.ptr(gbuf), _lib.ROWS_SORTED
        _lib.check(lib.flymoe_moe_gemm2_pertoken(
            _lib.ptr(arg_out), a_ptr, sx_ptr, _lib.ptr(w_plain), sw_ptr,
            _lib.ptr(arg_sorted_token_ids), _lib.ptr(arg_expert_ids), _lib.ptr(arg_sorted_weights),
            _lib.ptr(arg_num_valid_ids), tokens, model_dim, inter_dim, blocks, experts, topk, tile_m,
            1 if doweight_stage2 else 0, in_code, out_code, acc, a_layout, _lib.ROWS_BY_PAIR, impl_code, h),
            "moe_gemm2_pertoken")

    return launch_moe_gemm2


def compile_moe_gemm2_ex(*, model_dim: int, inter_dim: int, experts: int, topk: int, tile_m: int, tile_n: int,
                         tile_k: int, doweight_stage2: bool, in_dtype: str = "fp8", group_size: int = -1,
                         out_dtype: str = "f16", use_cshuffle_epilog: bool | None = None,
                         mode: str = MoeGemm2Mode.ATOMIC, valid_mask=None, zero_intermediate: bool = True,
                         scale_is_bf16: bool = False, **extra):
    """Stage 2 with explicit mode control: "atomic" or "reduce" (no atomics + reduce kernel).
    ``zero_intermediate=False`` skips clearing the per-pair rows, as in the reference (valid when
    every pair is routed to one of this launcher's experts)."""
    common = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m,
                  tile_n=tile_n, tile_k=tile_k, doweight_stage2=doweight_stage2, in_dtype=in_dtype,
                  group_size=group_size, out_dtype=out_dtype, use_cshuffle_epilog=use_cshuffle_epilog,
                  scale_is_bf16=scale_is_bf16, **extra)
    if mode == MoeGemm2Mode.REDUCE:
        use_mask = valid_mask is not None
        out_s = str(out_dtype).strip().lower()
        if out_s in ("f32", "fp32", "float"):
            raise ValueError("mode='reduce' supports out_dtype 'f16' or 'bf16'")
        gemm2_exe = compile_moe_gemm2(accumulate=False, **common)
        dtype_str = "f16" if out_s in ("f16", "fp16", "half") else "bf16"
        reduce_exe = compile_moe_reduction(topk=topk, model_dim=model_dim, dtype_str=dtype_str, use_mask=use_mask)
        return _MoeGemm2ReduceWrapper(gemm2_exe=gemm2_exe, reduce_exe=reduce_exe, topk=topk, model_dim=model_dim,
                                      out_dtype_str=dtype_str, use_mask=use_mask, zero_rows=zero_intermediate)
    return compile_moe_gemm2(accumulate=True, **common)
