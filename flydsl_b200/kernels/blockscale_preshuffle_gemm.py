"""Dense FP8 (e4m3) block-scaled GEMM for B200.

Mirrors ``kernels/blockscale_preshuffle_gemm.py`` of the reference:
``compile_blockscale_preshuffle_gemm`` (:32-45) returns a launcher with the positional order of
:866-875 ``(c, a, b, scale_a, scale_b, M, N, stream)``.

Data contract (the reference's): ``a`` e4m3 [M, K]; ``scale_a`` fp32 stored transposed
[K/128, M]; ``b`` e4m3 [N, K] in the 16x16 preshuffle order (tests/utils.py:76-96; converted to
row-major once per weight tensor and cached) or row-major with ``w_layout="plain"``; ``scale_b``
fp32 [ceil(N/128), K/128]; ``c`` [M, N] bf16/fp16.  ``c = sum_kb (a_kb . b_kb^T) * scale_a[kb, m] *
scale_b[n/128, kb]`` -- the arithmetic of MoE stage 2 without grouping, and it runs on the same
tcgen05 kernel (one expert, identity routing).

Differences: N must be a multiple of 64 (covers the reference's 2112-column case); ``tile_m`` must be 16/32/64/128 and is the only tile parameter that changes anything --
``tile_n`` / ``tile_k`` are checked like the reference does and otherwise ignored, as are the AMD
knobs ``use_cshuffle_epilog``, ``waves_per_eu`` and ``use_async_copy``.
"""

from __future__ import annotations

import functools

import torch

from .. import _lib
from .moe_blockscale_2stage import _FP8_DTYPES, _LauncherScratch, _plain_weight, _resolve_scratch

_OUT = {"bf16": torch.bfloat16, "fp16": torch.float16}


@functools.lru_cache(maxsize=1024)
def compile_blockscale_preshuffle_gemm(*, M: int, N: int, K: int, tile_m: int, tile_n: int, tile_k: int,
                                       scale_block_k: int = 128, out_dtype: str = "bf16",
                                       use_cshuffle_epilog: bool = False, waves_per_eu: int | None = None,
                                       use_async_copy: bool = False, w_layout: str = "preshuffle16x16"):
    """Build the launcher.  FP8 inputs, per-block scales, bf16/fp16 output."""
    if out_dtype not in ("fp16", "bf16"):
        raise ValueError(f"out_dtype must be 'fp16' or 'bf16', got {out_dtype!r}")
    if tile_k % scale_block_k != 0:
        raise ValueError(f"tile_k ({tile_k}) must be divisible by scale_block_k ({scale_block_k})")
    if K % tile_k != 0:
        raise ValueError(f"K ({K}) must be divisible by tile_k ({tile_k})")
    if K % scale_block_k != 0:
        raise ValueError(f"K ({K}) must be divisible by scale_block_k ({scale_block_k})")
    if tile_k % 64 != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got {tile_k}")
    if scale_block_k != 128:
        raise ValueError(f"scale_block_k must be 128, got {scale_block_k}")
    if N % 64 != 0:
        raise ValueError(f"N ({N}) must be a multiple of 64 on this implementation")
    if tile_m not in (16, 32, 64, 128):
        raise ValueError(f"tile_m must be one of (16, 32, 64, 128), got {tile_m}")
    if w_layout not in ("preshuffle16x16", "plain"):
        raise ValueError(f"w_layout must be 'preshuffle16x16' or 'plain', got {w_layout!r}")
    out_torch = _OUT[out_dtype]
    out_code = _lib.DTYPE_CODE[out_torch]
    # routing tables of the grouped kernel (identity routing): one buffer per (device, stream) of this
    # launcher, sized for M at its first call on that stream; ``workspace=`` takes the caller's own
    scratch = _LauncherScratch(torch.int32)
    ws_elems = int(_lib.load().flymoe_blockscale_gemm_workspace_elems(M, tile_m)) if M > 0 else 1

    def launch_gemm(arg_c, arg_a, arg_b, arg_scale_a, arg_scale_b, i32_m, i32_n, stream=None, *, workspace=None):
        m, n = int(i32_m), int(i32_n)
        if n != N:
            raise ValueError(f"launcher built for N={N}; called with N={n}")
        if m > M:
            raise ValueError(f"launcher built for M<={M}; called with M={m}")
        lib = _lib.load()
        _lib.require_cuda("arg_c", arg_c, (out_torch,), m * N)
        _lib.require_cuda("arg_a", arg_a, _FP8_DTYPES, m * K)
        _lib.require_cuda("arg_b", arg_b, _FP8_DTYPES, N * K)
        _lib.require_cuda("arg_scale_a", arg_scale_a, (torch.float32,), (K // 128) * m)
        _lib.require_cuda("arg_scale_b", arg_scale_b, (torch.float32,), ((N + 127) // 128) * (K // 128))
        s = _lib.stream_handle(stream)
        b_plain = _plain_weight(arg_b, N, K, w_layout, stream)
        ws = _resolve_scratch(scratch, workspace, "workspace", arg_a.device, s, ws_elems)
        sa_stride = arg_scale_a.numel() // (K // 128)          # the transposed layout's row length (>= m)
        _lib.check(lib.flymoe_blockscale_gemm(_lib.ptr(arg_c), _lib.ptr(arg_a), _lib.ptr(arg_scale_a), sa_stride,
                                              _lib.ptr(b_plain), _lib.ptr(arg_scale_b), _lib.ptr(ws), ws.numel(),
                                              m, N, K, tile_m, out_code, s), "blockscale_gemm")

    return launch_gemm
