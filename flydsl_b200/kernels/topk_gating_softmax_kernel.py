"""Fused softmax + top-k expert selection for MoE gating (B200).

Mirrors ``kernels/topk_gating_softmax_kernel.py`` of the reference:
``build_topk_gating_softmax_module(num_experts, topk, dtype_str, renormalize)``
(:54-59) returns a launcher called as
``launch(GatingOutput, TopkWeights, TopkIndices, TokenExpertIndices, num_tokens, stream=...)``
(:336-344).  Outputs: weights f32 [T,k], indices i32 [T,k] in descending order of
logit with ties resolved to the lower expert id, and
token_expert_indices[t,k] = k*T + t (:331-333).
"""

from __future__ import annotations

import functools

import torch

from .. import _lib

KERNEL_NAME = "topk_gating_softmax_kernel"
WARP_SIZE = 32
WARPS_PER_BLOCK = 4
BLOCK_THREADS = WARPS_PER_BLOCK * WARP_SIZE

_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


@functools.lru_cache(maxsize=256)
def build_topk_gating_softmax_module(num_experts: int, topk: int, dtype_str: str = "bf16",
                                     renormalize: bool = True):
    """Return the launcher for one (num_experts, topk, dtype, renormalize) combination."""
    if dtype_str not in _DTYPES:
        raise ValueError(f"dtype_str must be one of {sorted(_DTYPES)}, got {dtype_str!r}")
    if not (1 <= num_experts <= 1024):
        raise ValueError(f"num_experts must be in [1, 1024], got {num_experts}")
    if not (1 <= topk <= min(32, num_experts)):
        raise ValueError(f"topk must be in [1, min(32, num_experts)], got {topk}")
    torch_dtype = _DTYPES[dtype_str]
    code = _lib.DTYPE_CODE[torch_dtype]
    renorm = 1 if renormalize else 0

    def launch_topk_gating_softmax(GatingOutput, TopkWeights, TopkIndices, TokenExpertIndices,
                                   num_tokens, stream=None):
        n = int(num_tokens)
        _lib.require_cuda("GatingOutput", GatingOutput, (torch_dtype,), n * num_experts)
        _lib.require_cuda("TopkWeights", TopkWeights, (torch.float32,), n * topk)
        _lib.require_cuda("TopkIndices", TopkIndices, (torch.int32,), n * topk)
        _lib.require_cuda("TokenExpertIndices", TokenExpertIndices, (torch.int32,), n * topk)
        lib = _lib.load()
        _lib.check(lib.flymoe_topk_gating_softmax(
            _lib.ptr(GatingOutput), code, _lib.ptr(TopkWeights), _lib.ptr(TopkIndices),
            _lib.ptr(TokenExpertIndices), n, num_experts, topk, renorm,
            _lib.stream_handle(stream)), "topk_gating_softmax")

    return launch_topk_gating_softmax
