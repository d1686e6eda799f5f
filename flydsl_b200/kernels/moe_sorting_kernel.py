"""MoE token sorting (counting sort by expert with block-aligned padding) for B200.

Mirrors ``kernels/moe_sorting_kernel.py`` of the reference: ``moe_sorting_flydsl``
(:1628-1772) with the same argument order and the same caller-allocated outputs,
``moe_sorting_get_workspace_size`` (:1588-1598), ``compile_moe_sorting``
(:1601-1613), ``_compute_sub_tokens`` (:1560-1585) and the ``BLOCK_SIZE`` /
``UNIT_SIZE`` constants (:41-42).

Packed id format: ``(topk_slot << 24) | token``; padding rows carry
``(topk << 24) | num_tokens`` and weight 0.  Rows at or beyond
``num_valid_ids[0]`` are unspecified, as in the reference kernel.
"""

from __future__ import annotations

import torch

from .. import _lib

BLOCK_SIZE = 256
UNIT_SIZE = 32
WARP_SIZE = 32


def _compute_sub_tokens(num_experts, arch=None):
    """Largest token count the single-block shared-memory path accepts.

    The CUDA sort keeps only per-warp histograms in shared memory, so the limit is
    on (token, slot) pairs rather than on a per-token mesh; this helper keeps the
    reference's name and meaning (tokens below it need no workspace) for callers
    that size buffers with it.
    """
    return 1024  # 8192 pairs at 8 slots per token


def _native_workspace(M, num_experts, topk, unit_size):
    return int(_lib.load().flymoe_moe_sorting_workspace_elems(int(M), int(num_experts), int(topk),
                                                             int(unit_size)))


def moe_sorting_get_workspace_size(M, num_experts, topk, unit_size=UNIT_SIZE):
    """Workspace size (int32 elements) for the multi-block path; 0 for the single-block path.

    Never smaller than what the CUDA sort needs; for the multi-block path it is the
    larger of that and the reference's own formula, so buffers sized for the reference
    keep working.
    """
    need = _native_workspace(M, num_experts, topk, unit_size)
    if need == 0:
        return 0
    mesh_stride = ((M + unit_size - 1) // unit_size) * unit_size
    ref = (num_experts * mesh_stride + 3) // 4 + (num_experts + 1)
    return max(need, ref)


def compile_moe_sorting(*, num_experts, topk, max_tokens=128, unit_size=UNIT_SIZE, has_mask=False):
    """Kept for callers that pre-compile: the CUDA kernels are ahead-of-time compiled,
    so this only validates the configuration and returns three equivalent launchers."""
    if not (1 <= num_experts <= 1024):
        raise ValueError(f"num_experts must be in [1, 1024], got {num_experts}")
    if not (1 <= topk <= 255):
        raise ValueError(f"topk must be in [1, 255], got {topk}")

    def launch(topk_ids, topk_weights, sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids,
               moe_buf, expert_mask=None, workspace=None):
        return moe_sorting_flydsl(topk_ids, topk_weights, sorted_ids, sorted_weights, sorted_expert_ids,
                                  num_valid_ids, moe_buf, num_experts, unit_size,
                                  expert_mask if has_mask else None, None, workspace)

    return launch, launch, launch


def moe_sorting_flydsl(topk_ids, topk_weights, sorted_ids, sorted_weights, sorted_expert_ids,
                       num_valid_ids, moe_buf, num_experts, unit_size=UNIT_SIZE, expert_mask=None,
                       num_local_tokens=None, workspace=None):
    """Sort (token, slot) pairs by expert; see the module docstring for the formats.

    All outputs are pre-allocated by the caller and returned in the reference's order:
    ``sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids, moe_buf``.  ``moe_buf``
    (the stage-2 accumulation target) is zeroed.  Work is enqueued on the current stream.
    """
    _lib.require_cuda("topk_ids", topk_ids, (torch.int32,))
    if topk_ids.dim() != 2:
        raise ValueError("topk_ids must be [tokens, topk]")
    topk = topk_ids.shape[1]
    if num_local_tokens is not None:
        M = int(num_local_tokens.item()) if isinstance(num_local_tokens, torch.Tensor) else int(num_local_tokens)
    else:
        M = topk_ids.shape[0]
    if M > topk_ids.shape[0]:
        raise ValueError("num_local_tokens exceeds topk_ids.shape[0]")
    capacity = M * topk + num_experts * unit_size - topk
    nblocks = (capacity + unit_size - 1) // unit_size
    _lib.require_cuda("topk_weights", topk_weights, (torch.float32,), M * topk)
    _lib.require_cuda("sorted_ids", sorted_ids, (torch.int32,), capacity)
    _lib.require_cuda("sorted_weights", sorted_weights, (torch.float32,), capacity)
    _lib.require_cuda("sorted_expert_ids", sorted_expert_ids, (torch.int32,), nblocks)
    _lib.require_cuda("num_valid_ids", num_valid_ids, (torch.int32,), 2)
    if expert_mask is not None:
        _lib.require_cuda("expert_mask", expert_mask, (torch.int32,), num_experts)
    moe_buf_bytes = 0
    if moe_buf is not None:
        _lib.require_cuda("moe_buf", moe_buf)
        moe_buf_bytes = moe_buf.numel() * moe_buf.element_size()

    need = _native_workspace(M, num_experts, topk, unit_size)
    ws_elems = 0
    if need > 0:
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.int32, device=topk_ids.device)
        _lib.require_cuda("workspace", workspace, (torch.int32,), need)
        ws_elems = workspace.numel()
    lib = _lib.load()
    _lib.check(lib.flymoe_moe_sorting(
        _lib.ptr(topk_ids), _lib.ptr(topk_weights), _lib.ptr(sorted_ids), _lib.ptr(sorted_weights),
        _lib.ptr(sorted_expert_ids), _lib.ptr(num_valid_ids), _lib.ptr(moe_buf), moe_buf_bytes,
        _lib.ptr(expert_mask), _lib.ptr(workspace) if need > 0 else None, ws_elems,
        M, int(num_experts), int(topk), int(unit_size), _lib.stream_handle(None)), "moe_sorting")
    return sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids, moe_buf
