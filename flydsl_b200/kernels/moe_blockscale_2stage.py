"""FP8 (e4m3) block-scaled two-stage MoE GEMMs for B200.

Mirrors ``kernels/moe_blockscale_2stage.py`` of the reference:

* ``compile_moe_blockscale_gemm1`` (:70-84) -> launcher with the positional order of
  :1142-1157 ``(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids,
  sorted_weights, max_token_ids, tokens, inter, k, size_expert_ids, stream)``
* ``compile_moe_blockscale_gemm2`` (:1189-1207) -> launcher of :2335-2350
* ``compile_moe_reduction`` (:2383-2589), ``MoeGemm2Mode`` (:2593-2597),
  ``compile_moe_blockscale_gemm2_ex`` (:2700-2786)

Data contract (same as the reference): x e4m3 [tokens, K]; activation scales fp32
stored transposed [K/128, rows]; weights e4m3 [E, N, K] with fp32 scales
[E, N/128, K/128]; stage 1 writes row ``t*topk + s``; stage 2 reads that row and
accumulates ``sorted_weight * (a2 . W2^T)`` into ``out[t]`` (pre-zeroed) or, with
``accumulate=False``, stores per-pair rows for ``compile_moe_reduction``.

Additions, all keyword-only and off by default:

* ``out_dtype="fp8"`` on stage 1 fuses the per-row, per-128-column requantisation the
  reference performs between the stages (tests/kernels/test_moe_blockscale.py:447-452):
  the launcher then takes ``arg_out_scale=`` (fp32 [inter/128, rows]).
* ``w_layout``: ``"preshuffle16x16"`` (default, the reference's weight order,
  tests/utils.py:76-96; converted once per weight tensor and cached) or ``"plain"``
  (row-major [E, N, K]).
* ``row_layout="sorted"``: the activation/intermediate rows are already in sorted
  order (the fused layer uses this to skip the row gather).
* ``impl``: ``"tcgen05"`` (default) or ``"simt"`` (CUDA-core cross-check kernel).

AMD-only tuning knobs (``waves_per_eu``, ``use_cshuffle_epilog``) are accepted and ignored.
"""

from __future__ import annotations

import functools
import logging
import weakref

import torch

from .. import _lib

logger = logging.getLogger("flydsl_b200")

_FP8_DTYPES = (torch.float8_e4m3fn, torch.uint8)
_BYTE_DTYPES = _FP8_DTYPES + (torch.int8,)     # anything the one-byte weight re-layout can move
_OUT16 = {"f16": torch.float16, "bf16": torch.bfloat16}
_IMPL = {"tcgen05": _lib.IMPL_TCGEN05, "simt": _lib.IMPL_SIMT}
_TILE_M = (16, 32, 64, 128)
# Row blocks of up to this many rows have their rows fetched by index inside the GEMM kernel (one warp
# keeps up with them); larger ones are gathered into sorted order ahead of the launch, which is faster.
_GATHER_IN_KERNEL_MAX = 32


# ------------------------------------------------------------------------- weight layout
# Row-major copies of preshuffled weights, one per live weight tensor.  An entry lives exactly as
# long as the storage it was converted from (a finalizer on the storage object removes it), so a
# model with any number of layers converts every weight once, at its first launch or ahead of time
# with ``prepare_weight``.  The default layout therefore doubles the memory of every weight that
# is launched with it; ``w_layout="plain"`` (or converting at load time and dropping the
# preshuffled tensor) avoids the second copy.
_plain_cache: dict = {}


_WEIGHT_DTYPES = _BYTE_DTYPES + (torch.float16, torch.bfloat16)


def _reorder_weight(w: torch.Tensor, rows: int, cols: int, to_plain: int, stream) -> torch.Tensor:
    _lib.require_cuda("w", w, _WEIGHT_DTYPES, rows * cols)
    out = torch.empty(rows * cols, dtype=w.dtype, device=w.device)
    _order_after_current_stream(stream, w.device)
    _lib.check(_lib.load().flymoe_shuffle_weight_elems(_lib.ptr(w), _lib.ptr(out), rows, cols, w.element_size(),
                                                       to_plain, _lib.stream_handle(stream)), "shuffle_weight")
    return out


def unshuffle_weight(w: torch.Tensor, rows: int, cols: int, stream=None) -> torch.Tensor:
    """Return a row-major copy of a 16x16-preshuffled weight ([rows, cols] one- or two-byte elements)."""
    return _reorder_weight(w, rows, cols, 1, stream)


def shuffle_weight(w: torch.Tensor, rows: int, cols: int, stream=None) -> torch.Tensor:
    """Row-major weight (one- or two-byte elements) -> the reference's 16x16 preshuffle order."""
    return _reorder_weight(w, rows, cols, 0, stream)


def _order_after_current_stream(stream, device) -> None:
    """A tensor that torch has just allocated is only safe to touch in the order of torch's current
    stream; when the caller launches on another stream, make that stream wait for the current one."""
    if stream is None:
        return
    cur = torch.cuda.current_stream(device)
    h = _lib.stream_handle(stream)
    if h == cur.cuda_stream:
        return
    ev = torch.cuda.Event()
    ev.record(cur)
    torch.cuda.ExternalStream(h, device=device).wait_event(ev)


def prepare_weight(w: torch.Tensor, rows: int, cols: int, stream=None) -> torch.Tensor:
    """Convert a 16x16-preshuffled weight to row-major now (e.g. at model load) and remember the
    copy for the lifetime of ``w``: launchers built with ``w_layout="preshuffle16x16"`` then find
    it and only enqueue kernels.  Returns the row-major tensor, which may also be passed to
    launchers built with ``w_layout="plain"`` in place of ``w``."""
    return _plain_weight(w, rows, cols, "preshuffle16x16", stream)


def unpack_int4_weight(w: torch.Tensor, rows: int, cols: int, dtype=torch.int8, stream=None, *,
                       group_scale: torch.Tensor | None = None, rows_per_expert: int = 0) -> torch.Tensor:
    """The reference's packed-int4 weights (signed 4-bit values of the 16x16-preshuffled one-byte layout,
    eight per four bytes; ``rows*cols/2`` bytes) -> row-major ``[rows*cols]`` int8 or bfloat16.
    ``group_scale`` (bfloat16 output only): group-wise scales of 32-wide K groups in the reference's kernel
    layout (f32 ``[E, cols/32, rows_per_expert]`` or bf16 ``[E, cols/64, rows_per_expert, 2]``), multiplied
    in before the value is rounded to bfloat16."""
    if dtype not in (torch.int8, torch.bfloat16):
        raise ValueError(f"unpack_int4_weight: dtype must be torch.int8 or torch.bfloat16, got {dtype}")
    _lib.require_cuda("w", w, (torch.int8, torch.uint8), rows * cols // 2)
    gs_ptr, gs_code = None, 0
    if group_scale is not None:
        if rows_per_expert <= 0 or rows % rows_per_expert:
            raise ValueError("unpack_int4_weight: rows must be a multiple of rows_per_expert")
        _lib.require_cuda("group_scale", group_scale, (torch.float32, torch.bfloat16), rows * (cols // 32))
        gs_ptr, gs_code = _lib.ptr(group_scale), _lib.DTYPE_CODE[group_scale.dtype]
    out = torch.empty(rows * cols, dtype=dtype, device=w.device)
    _order_after_current_stream(stream, w.device)
    _lib.check(_lib.load().flymoe_unpack_int4_weight_grouped(
        _lib.ptr(w), _lib.ptr(out), rows, cols, _lib.DTYPE_CODE[dtype], gs_ptr, gs_code, 32 if gs_ptr else 0,
        rows_per_expert, _lib.stream_handle(stream)), "unpack_int4_weight")
    return out


def _plain_weight(w: torch.Tensor, rows: int, cols: int, layout: str, stream, int4_to=None,
                  group_scale: torch.Tensor | None = None, rows_per_expert: int = 0) -> torch.Tensor:
    """Row-major operand of a weight tensor, converted once per tensor.  ``int4_to`` (torch.int8 or
    torch.bfloat16): ``w`` holds packed int4 values and is unpacked to that type instead, with the
    group-wise scales folded in when given (the copy is then tied to that scale tensor as well)."""
    if layout == "plain":
        return w
    # An entry is only valid for the allocation it was made from: a freed weight's address is reused
    # by the allocator, so the storage object itself (weakly referenced) is part of the check.
    storage = w.untyped_storage()
    gkey = None if group_scale is None else (group_scale.data_ptr(), group_scale._version, group_scale.dtype)
    key = (w.data_ptr(), w.numel(), w.element_size(), w.device.index, rows, cols, int4_to, gkey)
    gstorage = None if group_scale is None else group_scale.untyped_storage()
    hit = _plain_cache.get(key)
    if (hit is not None and hit[0] == w._version and hit[2]() is storage
            and (gstorage is None or (hit[3] is not None and hit[3]() is gstorage))):
        return hit[1]
    if int4_to is None:
        plain = unshuffle_weight(w, rows, cols, stream)
    else:
        plain = unpack_int4_weight(w, rows, cols, int4_to, stream, group_scale=group_scale, rows_per_expert=rows_per_expert)
    _plain_cache[key] = (w._version, plain, weakref.ref(storage), None if gstorage is None else weakref.ref(gstorage))
    weakref.finalize(storage, _drop_plain, key, id(plain))
    return plain


def _drop_plain(key, plain_id) -> None:
    hit = _plain_cache.get(key)
    if hit is not None and id(hit[1]) == plain_id:
        del _plain_cache[key]


def clear_weight_cache() -> None:
    _plain_cache.clear()


# ------------------------------------------------------------------------- scratch
class _LauncherScratch:
    """Device scratch owned by ONE compiled launcher: one buffer per (device, stream), so two
    launchers -- or one launcher used on two streams -- never share it.  A buffer is created at the
    first call on that stream (or ahead of time with ``reserve``) and replaced only by a larger one;
    replaced buffers stay referenced, because kernels already enqueued on a stream torch does not
    track may still read them.  Callers that must not allocate on the call path (graph capture,
    a fixed memory budget) pass their own buffer to the launcher instead.  Launchers built for row
    blocks of 16 or 32 rows need no gather buffer at all."""

    def __init__(self, dtype):
        self.dtype = dtype
        self.bufs: dict = {}
        self.retired: list = []

    def get(self, device, stream_handle: int, numel: int) -> torch.Tensor:
        key = (device.index, stream_handle)
        buf = self.bufs.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self.retired.append(buf)
            buf = torch.empty(max(numel, 1), dtype=self.dtype, device=device)
            self.bufs[key] = buf
        return buf


def _resolve_scratch(scratch: _LauncherScratch, given, name: str, device, stream_handle: int, numel: int):
    if given is None:
        return scratch.get(device, stream_handle, numel)
    _lib.require_cuda(name, given, (scratch.dtype,), numel)
    return given


def _check_common(model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, scale_block_k, w_layout,
                  row_layout, impl):
    if scale_block_k != 128:
        raise ValueError(f"scale_block_k must be 128, got {scale_block_k}")
    if tile_k % 64 != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got tile_k_bytes={tile_k} (tile_k={tile_k}, elem_bytes=1)")
    if (tile_m * tile_k) % 256 != 0:
        raise ValueError(f"tile_m*tile_k*elem_bytes must be divisible by 256: tile_m={tile_m}, tile_k={tile_k}, elem_bytes=1")
    if w_layout not in ("preshuffle16x16", "plain"):
        raise ValueError(f"w_layout must be 'preshuffle16x16' or 'plain', got {w_layout!r}")
    if row_layout not in ("token", "sorted"):
        raise ValueError(f"row_layout must be 'token' or 'sorted', got {row_layout!r}")
    if impl not in _IMPL:
        raise ValueError(f"impl must be one of {sorted(_IMPL)}, got {impl!r}")
    if impl == "tcgen05" and tile_m not in _TILE_M:
        raise ValueError(f"tile_m must be one of {_TILE_M} for the tensor-core path, got {tile_m}")
    if experts < 1 or topk < 1 or topk > 255:
        raise ValueError(f"experts/topk out of range: experts={experts}, topk={topk}")
    if tile_n <= 0:
        raise ValueError(f"tile_n must be positive, got {tile_n}")


# ------------------------------------------------------------------------- stage 1
@functools.lru_cache(maxsize=1024)
def compile_moe_blockscale_gemm1(*, model_dim: int, inter_dim: int, experts: int, topk: int, tile_m: int,
                                 tile_n: int, tile_k: int, doweight_stage1: bool, scale_block_k: int = 128,
                                 out_dtype: str = "f16", use_cshuffle_epilog: bool | None = None,
                                 waves_per_eu: int | None = None, w_layout: str = "preshuffle16x16",
                                 row_layout: str = "token", impl: str = "tcgen05"):
    """Build the stage-1 launcher (gate/up grouped FP8 GEMM + SiLU(gate)*up)."""
    if out_dtype not in ("f16", "bf16", "fp8"):
        raise ValueError(f"out_dtype must be 'f16' or 'bf16', got {out_dtype!r}")
    if model_dim % scale_block_k != 0:
        raise ValueError(f"model_dim ({model_dim}) must be divisible by scale_block_k ({scale_block_k})")
    if (2 * inter_dim) % 128 != 0:
        raise ValueError(f"2*inter_dim ({2 * inter_dim}) must be divisible by 128 (ScaleBlockN)")
    if inter_dim % 128 != 0:
        raise ValueError(f"inter_dim ({inter_dim}) must be divisible by 128 (one output quantisation group per tile)")
    _check_common(model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, scale_block_k, w_layout,
                  row_layout, impl)
    if waves_per_eu is not None or use_cshuffle_epilog is not None:
        logger.debug("stage 1: waves_per_eu / use_cshuffle_epilog are AMD tuning knobs and are ignored")
    impl_code = _IMPL[impl]
    fp8_out = out_dtype == "fp8"
    out_code = _lib.E4M3 if fp8_out else _lib.DTYPE_CODE[_OUT16[out_dtype]]
    out_torch = _FP8_DTYPES if fp8_out else (_OUT16[out_dtype],)
    sorted_rows = row_layout == "sorted"
    wrows = experts * 2 * inter_dim
    scratch = _LauncherScratch(torch.uint8)

    def launch_moe_blockscale_gemm1(arg_out, arg_x, arg_w, arg_scale_x, arg_scale_w, arg_sorted_token_ids,
                                    arg_expert_ids, arg_sorted_weights, arg_max_token_ids, tokens_in,
                                    inter_in, k_in, size_expert_ids_in, stream=None, *, arg_out_scale=None,
                                    gather_buffer=None):
        tokens, blocks = int(tokens_in), int(size_expert_ids_in)
        if int(inter_in) != inter_dim or int(k_in) != model_dim:
            raise ValueError(f"launcher built for inter_dim={inter_dim}, model_dim={model_dim}; "
                             f"called with inter={inter_in}, k={k_in}")
        cap_rows = blocks * tile_m
        pairs = tokens * topk
        x_rows = cap_rows if sorted_rows else tokens
        out_rows = cap_rows if sorted_rows else pairs
        kb = model_dim // 128
        _lib.require_cuda("arg_out", arg_out, out_torch, out_rows * inter_dim)
        _lib.require_cuda("arg_x", arg_x, _FP8_DTYPES, x_rows * model_dim)
        _lib.require_cuda("arg_w", arg_w, _FP8_DTYPES, wrows * model_dim)
        _lib.require_cuda("arg_scale_x", arg_scale_x, (torch.float32,), kb * x_rows)
        _lib.require_cuda("arg_scale_w", arg_scale_w, (torch.float32,), experts * (2 * inter_dim // 128) * kb)
        _lib.require_cuda("arg_sorted_token_ids", arg_sorted_token_ids, (torch.int32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_expert_ids", arg_expert_ids, (torch.int32,), blocks)
        _lib.require_cuda("arg_sorted_weights", arg_sorted_weights, (torch.float32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_max_token_ids", arg_max_token_ids, (torch.int32,), 1)
        out_scale_stride = 0
        if fp8_out:
            if arg_out_scale is None:
                raise ValueError("out_dtype='fp8' needs arg_out_scale (fp32 [inter_dim/128, rows])")
            _lib.require_cuda("arg_out_scale", arg_out_scale, (torch.float32,), (inter_dim // 128) * out_rows)
            out_scale_stride = arg_out_scale.numel() // (inter_dim // 128)
        sx_stride = arg_scale_x.numel() // kb
        h = _lib.stream_handle(stream)
        lib = _lib.load()
        w_plain = _plain_weight(arg_w, wrows, model_dim, w_layout, h)
        x_layout = _lib.ROWS_SORTED if sorted_rows else _lib.ROWS_BY_TOKEN
        x_ptr = _lib.ptr(arg_x)
        if impl_code == _lib.IMPL_TCGEN05 and not sorted_rows and tile_m > _GATHER_IN_KERNEL_MAX:
            gbuf = _resolve_scratch(scratch, gather_buffer, "gather_buffer", arg_x.device, h, cap_rows * model_dim)
            _lib.check(lib.flymoe_gather_rows(x_ptr, _lib.ptr(gbuf), _lib.ptr(arg_sorted_token_ids),
                                              _lib.ptr(arg_max_token_ids), tokens, topk, model_dim,
                                              _lib.ROWS_BY_TOKEN, cap_rows, h), "gather_rows")
            x_ptr = _lib.ptr(gbuf)
            x_layout = _lib.ROWS_SORTED
        _lib.check(lib.flymoe_moe_gemm1(
            _lib.ptr(arg_out), _lib.ptr(arg_out_scale), out_scale_stride, x_ptr, _lib.ptr(arg_scale_x),
            sx_stride, 1, _lib.ptr(w_plain), _lib.ptr(arg_scale_w), _lib.ptr(arg_sorted_token_ids),
            _lib.ptr(arg_expert_ids), _lib.ptr(arg_sorted_weights), _lib.ptr(arg_max_token_ids),
            tokens, inter_dim, model_dim, blocks, experts, topk, tile_m, 1 if doweight_stage1 else 0,
            out_code, x_layout, _lib.ROWS_SORTED if sorted_rows else _lib.ROWS_BY_TOKEN,
            _lib.ROWS_SORTED if sorted_rows else _lib.ROWS_BY_PAIR, impl_code, h), "moe_gemm1")

    launch_moe_blockscale_gemm1.reserve = lambda tokens, blocks, device, stream=None: scratch.get(
        torch.device(device), _lib.stream_handle(stream), int(blocks) * tile_m * model_dim)
    return launch_moe_blockscale_gemm1


# ------------------------------------------------------------------------- stage 2
@functools.lru_cache(maxsize=1024)
def compile_moe_blockscale_gemm2(*, model_dim: int, inter_dim: int, experts: int, topk: int, tile_m: int,
                                 tile_n: int, tile_k: int, doweight_stage2: bool, scale_block_k: int = 128,
                                 out_dtype: str = "f16", use_cshuffle_epilog: bool | None = None,
                                 accumulate: bool = True, waves_per_eu: int | None = None,
                                 w_layout: str = "preshuffle16x16", row_layout: str = "token",
                                 impl: str = "tcgen05"):
    """Build the stage-2 launcher (down grouped FP8 GEMM + weighted scatter-reduce)."""
    out_s = str(out_dtype).strip().lower()
    if out_s not in ("f16", "fp16", "half", "bf16", "bfloat16", "f32", "fp32", "float"):
        raise ValueError(f"out_dtype must be 'f16', 'bf16', or 'f32', got {out_dtype!r}")
    out_is_f32 = out_s in ("f32", "fp32", "float")
    out_is_bf16 = out_s in ("bf16", "bfloat16")
    if (not bool(accumulate)) and out_is_f32:
        raise ValueError("compile_moe_blockscale_gemm2(accumulate=False) only supports out_dtype in {'f16','bf16'}")
    if inter_dim % scale_block_k != 0:
        raise ValueError(f"inter_dim ({inter_dim}) must be divisible by scale_block_k ({scale_block_k})")
    if model_dim % 128 != 0:
        raise ValueError(f"model_dim ({model_dim}) must be divisible by 128 (ScaleBlockN)")
    _check_common(model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, scale_block_k, w_layout,
                  row_layout, impl)
    if waves_per_eu is not None or use_cshuffle_epilog is not None:
        logger.debug("stage 2: waves_per_eu / use_cshuffle_epilog are AMD tuning knobs and are ignored")
    impl_code = _IMPL[impl]
    out_torch = torch.float32 if out_is_f32 else (torch.bfloat16 if out_is_bf16 else torch.float16)
    out_code = _lib.DTYPE_CODE[out_torch]
    sorted_rows = row_layout == "sorted"
    wrows = experts * model_dim
    acc = 1 if accumulate else 0
    scratch = _LauncherScratch(torch.uint8)

    def launch_moe_blockscale_gemm2(arg_out, arg_x, arg_w, arg_scale_x, arg_scale_w, arg_sorted_token_ids,
                                    arg_expert_ids, arg_sorted_weights, arg_num_valid_ids, tokens_in, n_in,
                                    k_in, size_expert_ids_in, stream=None, *, gather_buffer=None):
        tokens, blocks = int(tokens_in), int(size_expert_ids_in)
        if int(n_in) != model_dim or int(k_in) != inter_dim:
            raise ValueError(f"launcher built for model_dim={model_dim}, inter_dim={inter_dim}; "
                             f"called with n={n_in}, k={k_in}")
        cap_rows = blocks * tile_m
        pairs = tokens * topk
        a_rows = cap_rows if sorted_rows else pairs
        kb = inter_dim // 128
        out_rows = tokens if accumulate else pairs
        _lib.require_cuda("arg_out", arg_out, (out_torch,), out_rows * model_dim)
        _lib.require_cuda("arg_x", arg_x, _FP8_DTYPES, a_rows * inter_dim)
        _lib.require_cuda("arg_w", arg_w, _FP8_DTYPES, wrows * inter_dim)
        _lib.require_cuda("arg_scale_x", arg_scale_x, (torch.float32,), kb * a_rows)
        _lib.require_cuda("arg_scale_w", arg_scale_w, (torch.float32,), experts * (model_dim // 128) * kb)
        _lib.require_cuda("arg_sorted_token_ids", arg_sorted_token_ids, (torch.int32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_expert_ids", arg_expert_ids, (torch.int32,), blocks)
        _lib.require_cuda("arg_sorted_weights", arg_sorted_weights, (torch.float32,), max(0, cap_rows - tile_m + 1))
        _lib.require_cuda("arg_num_valid_ids", arg_num_valid_ids, (torch.int32,), 1)
        sa_stride = arg_scale_x.numel() // kb
        h = _lib.stream_handle(stream)
        lib = _lib.load()
        w_plain = _plain_weight(arg_w, wrows, inter_dim, w_layout, h)
        a_layout = _lib.ROWS_SORTED if sorted_rows else _lib.ROWS_BY_PAIR
        a_ptr = _lib.ptr(arg_x)
        if impl_code == _lib.IMPL_TCGEN05 and not sorted_rows and tile_m > _GATHER_IN_KERNEL_MAX:
            gbuf = _resolve_scratch(scratch, gather_buffer, "gather_buffer", arg_x.device, h, cap_rows * inter_dim)
            _lib.check(lib.flymoe_gather_rows(a_ptr, _lib.ptr(gbuf), _lib.ptr(arg_sorted_token_ids),
                                              _lib.ptr(arg_num_valid_ids), tokens, topk, inter_dim,
                                              _lib.ROWS_BY_PAIR, cap_rows, h), "gather_rows")
            a_ptr = _lib.ptr(gbuf)
            a_layout = _lib.ROWS_SORTED
        _lib.check(lib.flymoe_moe_gemm2(
            _lib.ptr(arg_out), a_ptr, _lib.ptr(arg_scale_x), sa_stride, _lib.ptr(w_plain),
            _lib.ptr(arg_scale_w), _lib.ptr(arg_sorted_token_ids), _lib.ptr(arg_expert_ids),
            _lib.ptr(arg_sorted_weights), _lib.ptr(arg_num_valid_ids), tokens, model_dim, inter_dim, blocks,
            experts, topk, tile_m, 1 if doweight_stage2 else 0, out_code, acc, a_layout,
            _lib.ROWS_SORTED if sorted_rows else _lib.ROWS_BY_PAIR, impl_code, h), "moe_gemm2")

    launch_moe_blockscale_gemm2.reserve = lambda tokens, blocks, device, stream=None: scratch.get(
        torch.device(device), _lib.stream_handle(stream), int(blocks) * tile_m * inter_dim)
    return launch_moe_blockscale_gemm2


# ------------------------------------------------------------------------- top-k reduce
@functools.lru_cache(maxsize=1024)
def compile_moe_reduction(*, topk: int, model_dim: int, dtype_str: str = "f16", use_mask: bool = False):
    """Y[t, d] = sum_k X[t, k, d] (fp32 accumulate); optional uint8 valid_mask [tokens, topk].

    Launcher: ``launch(X, Y, valid_mask, m_tokens, stream)`` as in the reference (:2571-2587).
    """
    dts = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
    if dtype_str not in dts:
        raise ValueError(f"Unsupported dtype: {dtype_str}")
    if model_dim % 8 != 0:
        raise ValueError(f"model_dim ({model_dim}) must be divisible by 8")
    dt = dts[dtype_str]
    code = _lib.DTYPE_CODE[dt]

    def launch_moe_reduction(X, Y, valid_mask, m_tokens, stream=None, *, weights=None):
        m = int(m_tokens)
        _lib.require_cuda("X", X, (dt,), m * topk * model_dim)
        _lib.require_cuda("Y", Y, (dt,), m * model_dim)
        mask_ptr = None
        if use_mask:
            _lib.require_cuda("valid_mask", valid_mask, (torch.uint8,), m * topk)
            mask_ptr = _lib.ptr(valid_mask)
        if weights is not None:
            _lib.require_cuda("weights", weights, (torch.float32,), m * topk)
        _lib.check(_lib.load().flymoe_moe_reduce(_lib.ptr(X), _lib.ptr(Y), mask_ptr, _lib.ptr(weights), None, m,
                                                 topk, model_dim, code, _lib.stream_handle(stream)), "moe_reduce")

    return launch_moe_reduction


class MoeGemm2Mode:
    """Execution mode for MoE GEMM2."""

    ATOMIC = "atomic"  # atomic accumulation into [tokens, model_dim]
    REDUCE = "reduce"  # per-pair rows + top-k reduce kernel (deterministic)


class _MoeGemm2ReduceWrapper:
    """Deterministic stage 2: per-(token, slot) rows without atomics, then the top-k reduce.

    Called with stage 2's own positional arguments (plus ``valid_mask``).  The [tokens*topk,
    model_dim] rows between the two kernels live in a buffer the wrapper keeps per (device,
    stream, row count): a call with a shape it has seen before allocates nothing.  Stage 2 writes
    the row of every (token, slot) pair routed to one of its experts.  With a mask the reduce skips
    the other rows; without one they are cleared first (``zero_rows``, one memset on the stream), so
    pairs routed elsewhere add zero -- switch that off when every pair is routed to an expert this
    launcher holds.
    """

    def __init__(self, gemm2_exe, reduce_exe, topk: int, model_dim: int, out_dtype_str: str = "f16",
                 use_mask: bool = False, zero_rows: bool = True):
        self._gemm2_exe = gemm2_exe
        self._reduce_exe = reduce_exe
        self._topk = int(topk)
        self._model_dim = int(model_dim)
        self._row_dtype = torch.bfloat16 if out_dtype_str == "bf16" else torch.float16
        self._use_mask = bool(use_mask)
        self._rows = _LauncherScratch(self._row_dtype)
        self._zero_rows = bool(zero_rows) and not self._use_mask
        self._warned = False

    def __call__(self, arg_out, arg_x, arg_w, arg_scale_x, arg_scale_w, arg_sorted_token_ids, arg_expert_ids,
                 arg_sorted_weights, arg_num_valid_ids, tokens_in, n_in, k_in, size_expert_ids_in,
                 valid_mask=None, stream=None):
        tokens = int(tokens_in)
        h = _lib.stream_handle(stream)
        pair_rows = self._rows.get(arg_out.device, h, tokens * self._topk * self._model_dim)
        if self._zero_rows:
            with torch.cuda.stream(torch.cuda.ExternalStream(h, device=arg_out.device)):
                pair_rows[: tokens * self._topk * self._model_dim].zero_()
        self._gemm2_exe(pair_rows, arg_x, arg_w, arg_scale_x, arg_scale_w, arg_sorted_token_ids, arg_expert_ids,
                        arg_sorted_weights, arg_num_valid_ids, tokens, n_in, k_in, size_expert_ids_in, h)
        if valid_mask is not None and not self._use_mask and not self._warned:
            logger.warning("this launcher was built without a mask: the valid_mask argument is ignored")
            self._warned = True
        self._reduce_exe(pair_rows, arg_out, valid_mask if self._use_mask else None, tokens, h)

    @property
    def mode(self) -> str:
        return MoeGemm2Mode.REDUCE


def compile_moe_blockscale_gemm2_ex(*, model_dim: int, inter_dim: int, experts: int, topk: int, tile_m: int,
                                    tile_n: int, tile_k: int, doweight_stage2: bool, in_dtype: str = "fp8",
                                    out_dtype: str = "f16", use_cshuffle_epilog: bool | None = None,
                                    mode: str = MoeGemm2Mode.ATOMIC, valid_mask=None,
                                    zero_intermediate: bool = True, **extra):
    """Stage 2 with explicit mode control: "atomic" or "reduce" (no atomics + reduce kernel).
    ``zero_intermediate=False`` skips clearing the per-pair rows (valid when every pair is routed to
    one of this launcher's experts)."""
    if in_dtype != "fp8":
        raise ValueError(f"the block-scaled path is FP8-only, got in_dtype={in_dtype!r}")
    common = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk, tile_m=tile_m,
                  tile_n=tile_n, tile_k=tile_k, doweight_stage2=doweight_stage2, out_dtype=out_dtype,
                  use_cshuffle_epilog=use_cshuffle_epilog, **extra)
    if mode == MoeGemm2Mode.REDUCE:
        use_mask = valid_mask is not None
        out_s = str(out_dtype).strip().lower()
        if out_s in ("f32", "fp32", "float"):
            raise ValueError("mode='reduce' supports out_dtype 'f16' or 'bf16'")
        gemm2_exe = compile_moe_blockscale_gemm2(accumulate=False, **common)
        dtype_str = "f16" if out_s in ("f16", "fp16", "half") else "bf16"
        reduce_exe = compile_moe_reduction(topk=topk, model_dim=model_dim, dtype_str=dtype_str, use_mask=use_mask)
        return _MoeGemm2ReduceWrapper(gemm2_exe=gemm2_exe, reduce_exe=reduce_exe, topk=topk, model_dim=model_dim,
                                      out_dtype_str=dtype_str, use_mask=use_mask, zero_rows=zero_intermediate)
    return compile_moe_blockscale_gemm2(accumulate=True, **common)
