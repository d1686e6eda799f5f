"""CPU oracle for the FP8 block-scaled fused-MoE path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch/numpy on the CPU, the algorithm that the
reference project uses as its own correctness oracle for this path.  It is the
checker for the CUDA kernels: only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may import it.  Nothing in the shipped package
imports it, and the shipped package has no CPU fallback.

Parity pin: every function below is compared, on seeded inputs, against the
reference's own torch functions executed from the reference checkout (see
``tests/golden/make_golden.py``, which lifts those functions at generation
time and stores their outputs as fixtures).

Reference locations each function follows (paths inside the reference project):

* gating          tests/kernels/test_topk_gating_softmax.py:84-94 (softmax ->
                  top-k -> renormalise), tie rule (lower expert id wins) from
                  kernels/topk_gating_softmax_kernel.py:156-174, eps :315-317,
                  token_expert_indices convention :331-333
* sorting         tests/kernels/test_moe_sorting.py:69-105
* quantisers      tests/utils.py:29-73 (pertoken_quant),
                  tests/kernels/test_moe_blockscale.py:269-276 (128x128 blocks)
* weight shuffle  tests/utils.py:76-96
* stage 1         tests/kernels/test_moe_blockscale.py:76-112
* requant         tests/kernels/test_moe_blockscale.py:447-452
* stage 2         tests/kernels/test_moe_blockscale.py:115-150
* top-k reduce    tests/kernels/test_moe_reduce.py:88-93
* dense GEMM      tests/kernels/test_blockscale_preshuffle_gemm.py:101-125
* per-token-scale family (one scale per activation row / weight row)
                  tests/kernels/test_ref.py:91-165 (stage 1), :168-239 (stage 2),
                  quantisation of its inputs tests/kernels/test_moe_gemm.py:446-450,
                  :463-488 (fp8, int8, per-(token, slot) "int8smooth"), :451-462 (fp16 / bf16:
                  cast, no scales), :489-499 (int4 weights: int8 values quantised to +-7, packed by
                  :49-65 after the preshuffle; activations int8 or bf16)

Differences from the reference text, all value-preserving: weights are
dequantised one expert at a time (the reference expands every expert to fp32
at once), and the top-k selection is made on the raw fp32 logits with a stable
sort so that ties and probability collapses resolve to the lower expert id on
every machine.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
BLK = 128


# --------------------------------------------------------------------------- gating
def topk_gating_softmax(logits: torch.Tensor, topk: int, renormalize: bool = True):
    """softmax over experts, pick the k largest (ties -> lower id), renormalise.

    Returns (weights f32 [T,k], indices i32 [T,k], token_expert_indices i32 [T,k]).
    """
    x = logits.to(torch.float32)
    T, _E = x.shape
    probs = torch.softmax(x, dim=1)
    order = torch.sort(x, dim=1, descending=True, stable=True).indices
    idx = order[:, :topk].contiguous()
    w = torch.gather(probs, 1, idx)
    if renormalize:
        w = w / w.sum(dim=1, keepdim=True).clamp(min=1e-20)
    tei = (torch.arange(topk, dtype=torch.int32).view(1, topk) * T
           + torch.arange(T, dtype=torch.int32).view(T, 1))
    return w.to(torch.float32), idx.to(torch.int32), tei.to(torch.int32)


def gating_prob_rule_differs(logits: torch.Tensor, topk: int) -> int:
    """Number of rows where 'top-k on fp32 probabilities' selects a different set."""
    x = logits.to(torch.float32)
    probs = torch.softmax(x, dim=1)
    a = torch.sort(x, dim=1, descending=True, stable=True).indices[:, :topk]
    b = torch.sort(probs, dim=1, descending=True, stable=True).indices[:, :topk]
    return int((a.sort(dim=1).values != b.sort(dim=1).values).any(dim=1).sum())


# --------------------------------------------------------------------------- sorting
def moe_sorting(topk_ids, topk_weights, num_experts: int, unit_size: int = 32,
                expert_mask=None):
    """Stable counting sort of (token, slot) pairs by expert with block padding.

    Returns numpy arrays (sorted_ids i32 [Rmax], sorted_weights f32 [Rmax],
    sorted_expert_ids i32 [B], num_valid_ids i32 [2]).  Packed id = slot<<24 | token,
    pad sentinel = topk<<24 | T, unused block ids = -1.
    """
    ids = np.asarray(topk_ids, dtype=np.int64)
    wts = np.asarray(topk_weights, dtype=np.float32)
    M, topk = ids.shape
    rmax = ids.size + num_experts * unit_size - topk
    nblk = (rmax + unit_size - 1) // unit_size
    sentinel = (topk << 24) | M
    sorted_ids = np.full((rmax,), sentinel, dtype=np.int32)
    sorted_w = np.zeros((rmax,), dtype=np.float32)
    sorted_e = np.full((nblk,), -1, dtype=np.int32)
    nvalid = np.zeros((2,), dtype=np.int32)
    mask = None if expert_mask is None else np.asarray(expert_mask).astype(bool)

    cur = 0
    ecur = 0
    skipped = 0
    for e in range(num_experts):
        if mask is not None and not mask[e]:
            skipped += 1
            continue
        tok, slot = np.nonzero(ids == e)           # row-major: token ascending
        cnt = tok.size
        if cnt == 0:
            continue
        nb = (cnt + unit_size - 1) // unit_size
        sorted_ids[cur:cur + cnt] = ((slot << 24) | tok).astype(np.int32)
        sorted_w[cur:cur + cnt] = wts[tok, slot]
        cur += nb * unit_size
        sorted_e[ecur:ecur + nb] = e - skipped
        ecur += nb
    nvalid[0] = cur
    nvalid[1] = M
    return sorted_ids, sorted_w, sorted_e, nvalid


# --------------------------------------------------------------------------- quantisers
def pertoken_quant(x: torch.Tensor, quant_dtype=FP8, dtype_max: float | None = None):
    """amax over the last dim / dtype max -> scale (0 -> 1); q = (x/scale).to(dtype)."""
    x = x.to(torch.float32)
    if dtype_max is None:
        dtype_max = float(torch.finfo(quant_dtype).max)
    x = torch.nan_to_num(x, nan=0.0, posinf=dtype_max, neginf=-dtype_max)
    amax = torch.maximum(torch.amax(x, dim=-1, keepdim=True), -torch.amin(x, dim=-1, keepdim=True))
    scale = amax / dtype_max
    scale[scale == 0] = 1
    scale = torch.nan_to_num(scale, nan=1.0, posinf=1.0, neginf=1.0)
    q = (x / scale).to(quant_dtype)
    return q, scale.to(torch.float32)


def quant_act_1x128(x: torch.Tensor):
    """[R,K] float -> (q e4m3 [R,K], scale f32 [R,K/128]) with 1x128 groups."""
    R, K = x.shape
    q, s = pertoken_quant(x.reshape(R, K // BLK, BLK))
    return q.reshape(R, K), s.reshape(R, K // BLK)


def quant_weight_128x128(w: torch.Tensor):
    """[N,K] float -> (q e4m3 [N,K], scale f32 [N/128,K/128]) with 128x128 blocks."""
    N, K = w.shape
    nbn, nbk = N // BLK, K // BLK
    t = w.to(torch.float32).view(nbn, BLK, nbk, BLK).permute(0, 2, 1, 3).reshape(nbn * nbk, BLK * BLK)
    q, s = pertoken_quant(t)
    q = q.view(nbn, nbk, BLK, BLK).permute(0, 2, 1, 3).reshape(N, K)
    return q.contiguous(), s.view(nbn, nbk).contiguous()


def shuffle_weight(w: torch.Tensor) -> torch.Tensor:
    """[..., N, K] one- or two-byte elements -> 16x16 preshuffle order (same shape): groups of 16 rows x
    32 elements, inside which 16 bytes of one row (16 or 8 elements) stay together."""
    assert w.element_size() in (1, 2)
    kk = 16 // w.element_size()
    N, K = w.shape[-2], w.shape[-1]
    carrier = torch.uint8 if w.element_size() == 1 else torch.int16
    v = w.view(carrier).reshape(-1, N // 16, 16, K // 32, 32 // kk, kk)
    v = v.permute(0, 1, 3, 4, 2, 5).contiguous()
    return v.view(*w.shape).view(w.dtype)


def unshuffle_weight(w: torch.Tensor) -> torch.Tensor:
    """Inverse of shuffle_weight."""
    assert w.element_size() in (1, 2)
    kk = 16 // w.element_size()
    N, K = w.shape[-2], w.shape[-1]
    carrier = torch.uint8 if w.element_size() == 1 else torch.int16
    v = w.view(carrier).reshape(-1, N // 16, K // 32, 32 // kk, 16, kk)
    v = v.permute(0, 1, 4, 2, 3, 5).contiguous()
    return v.view(*w.shape).view(w.dtype)


# --------------------------------------------------------------------------- GEMM stages
def _dequant_w(wq_e: torch.Tensor, ws_e: torch.Tensor) -> torch.Tensor:
    """One expert: e4m3 [N,K] * block scales [N/128,K/128] -> f32 [N,K]."""
    N, K = wq_e.shape
    s = ws_e.view(N // BLK, 1, K // BLK, 1).expand(N // BLK, BLK, K // BLK, BLK).reshape(N, K)
    return wq_e.to(torch.float32) * s


def _dequant_a(aq: torch.Tensor, a_scale: torch.Tensor) -> torch.Tensor:
    R, K = aq.shape
    return (aq.to(torch.float32).view(R, K // BLK, BLK) * a_scale.view(R, K // BLK, 1)).view(R, K)


def stage1(xq, x_scale, w1q, w1_scale, topk_ids, inter_dim: int):
    """silu(x W1g^T) * (x W1u^T) per (token, slot).  Returns f32 [T, k, I].

    xq e4m3 [T,H]; x_scale f32 [T,H/128]; w1q e4m3 [E,2I,H];
    w1_scale f32 [E,2I/128,H/128]; topk_ids [T,k].  w1q / w1_scale may be any
    sequence indexable by expert id (only experts that received a token are read).
    """
    T, _H = xq.shape
    ids = torch.as_tensor(topk_ids).to(torch.int64)
    k = ids.shape[1]
    E = len(w1q)
    x = _dequant_a(xq, x_scale)
    out = torch.zeros((T, k, inter_dim), dtype=torch.float32)
    for e in range(E):
        mask = ids == e
        if mask.any():
            tok = mask.nonzero()[:, 0]
            act = x[tok] @ _dequant_w(w1q[e], w1_scale[e]).T
            gate, up = act.split([inter_dim, inter_dim], dim=-1)
            out[mask] = F.silu(gate) * up
    return out


def requant(out1: torch.Tensor, via_f16: bool = False):
    """[T,k,I] f32 -> (a2q e4m3 [T*k,I], a2_scale f32 [T*k, I/128])."""
    T, k, I = out1.shape
    v = out1.to(torch.float16).to(torch.float32) if via_f16 else out1
    return quant_act_1x128(v.reshape(T * k, I))


def stage2(a2q, a2_scale, w2q, w2_scale, topk_ids, topk_weights, model_dim: int,
           reduce: bool = True):
    """out[t] = sum_s w[t,s] * (a2[t,s] W2_e^T).  Returns f32 [T,H] (or [T,k,H])."""
    ids = torch.as_tensor(topk_ids).to(torch.int64)
    T, k = ids.shape
    E = len(w2q)
    I = a2q.shape[1]
    a = _dequant_a(a2q, a2_scale).view(T, k, I)
    out = torch.zeros((T, k, model_dim), dtype=torch.float32)
    for e in range(E):
        mask = ids == e
        if mask.any():
            out[mask] = a[mask] @ _dequant_w(w2q[e], w2_scale[e]).T
    out = out * torch.as_tensor(topk_weights).to(torch.float32).view(T, k, 1)
    return out.sum(dim=1) if reduce else out


def topk_reduce(x: torch.Tensor, valid_mask=None) -> torch.Tensor:
    """Y[t,:] = sum_s X[t,s,:] (fp32 accumulate), optional u8 mask [T,k]."""
    v = x.to(torch.float32)
    if valid_mask is not None:
        v = v * valid_mask.to(torch.float32).unsqueeze(-1)
    return v.sum(dim=1).to(x.dtype)


def moe_layer(logits, xq, x_scale, w1q, w1_scale, w2q, w2_scale, topk: int,
              out_dtype=torch.bfloat16, via_f16: bool = False):
    """Whole path on identical pre-quantised inputs.  Returns a dict of every stage."""
    I = w2q.shape[2]
    H = w2q.shape[1]
    w, idx, tei = topk_gating_softmax(logits, topk, True)
    o1 = stage1(xq, x_scale, w1q, w1_scale, idx, I)
    a2q, a2s = requant(o1, via_f16=via_f16)
    o2 = stage2(a2q, a2s, w2q, w2_scale, idx, w, H)
    return {"topk_weights": w, "topk_ids": idx, "tei": tei, "out1": o1,
            "a2q": a2q, "a2_scale": a2s, "out": o2.to(out_dtype), "out_f32": o2}


# --------------------------------------------------------------------------- per-token-scale family
def quant_rows(x: torch.Tensor, quant_dtype=FP8, dtypeMax=None):
    """One scale per row of the last dim: (q, scale [..., 1]); int8 uses dtype max 127, or ``dtypeMax``
    (7 for the values that are packed to int4; the keyword is spelled as in tests/utils.py:35)."""
    dmax = float(dtypeMax) if dtypeMax is not None else (127.0 if quant_dtype == torch.int8 else None)
    return pertoken_quant(x, quant_dtype=quant_dtype, dtype_max=dmax)


def pack_int4_preshuffled(w_int8: torch.Tensor) -> torch.Tensor:
    """[..., N, K] int8 values in [-8, 7] -> the packed bytes the int4 variants take (N*K/2 int8, flat):
    the 16x16 preshuffle of the one-byte tensor, then every eight consecutive values v0..v7 become the four
    bytes (v4<<4)|v0, (v5<<4)|v1, (v6<<4)|v2, (v7<<4)|v3 (tests/kernels/test_moe_gemm.py:49-65)."""
    u = (shuffle_weight(w_int8).contiguous().view(-1).to(torch.int16) & 0xF).to(torch.uint8).view(-1, 8)
    return (u[:, :4] | (u[:, 4:] << 4)).contiguous().view(-1).view(torch.int8)


def _group_dequant(w_q: torch.Tensor, group_scale: torch.Tensor, group_size: int) -> torch.Tensor:
    """w[n, k] * scale[k // group_size, n] for one expert (tests/kernels/test_ref.py:133-141)."""
    return w_q.to(torch.float32) * group_scale.to(torch.float32).t().repeat_interleave(group_size, dim=1)


def pertoken_stage1(x_q, scale_x, w1_q, scale_w1, topk_ids, topk_weights, inter_dim: int,
                    doweight_stage1: bool = False, group_size: int = -1, scale_w1_groups=None, raw_sums: bool = False):
    """silu(x W1g^T) * (x W1u^T) with x = x_q * scale_x (per row) and W = w_q * scale_w (per row).

    x_q [T,K] (or [T,k,K] when every (token, slot) pair brings its own row) of e4m3/int8, scale_x
    [T,1] ([T,k,1]); w1_q [E,2I,K], scale_w1 [E,2I,1].  f16/bf16 operands come with ``None`` scales
    (no dequantisation, tests/kernels/test_ref.py:57-69 of the reference).  ``group_size > 0``: the weights
    are scaled per K group with ``scale_w1_groups`` [E, K/group_size, 2I] instead of per row.
    Returns f32 [T,k,I]; with ``raw_sums`` the pre-activation sums [T,k,2I] (gate columns first) that the
    reference's split-K launches leave to the caller (tests/kernels/test_moe_gemm.py:708-713)."""
    ids = torch.as_tensor(topk_ids).to(torch.int64)
    T, k = ids.shape
    E = w1_q.shape[0]
    x = x_q.to(torch.float32) if scale_x is None else x_q.to(torch.float32) * scale_x
    out = torch.zeros((T, k, 2 * inter_dim if raw_sums else inter_dim), dtype=torch.float32)
    for e in range(E):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        if group_size > 0 and scale_w1_groups is not None:
            w = _group_dequant(w1_q[e], scale_w1_groups[e], group_size)
        else:
            w = w1_q[e].to(torch.float32) if scale_w1 is None else w1_q[e].to(torch.float32) * scale_w1[e]
        rows = x[tok] if x.dim() == 2 else x[tok, slot]
        y2 = F.linear(rows, w)
        if raw_sums:
            out[tok, slot] = y2
            continue
        y = F.silu(y2[:, :inter_dim]) * y2[:, inter_dim:]
        if doweight_stage1:
            y = y * torch.as_tensor(topk_weights)[tok, slot].unsqueeze(-1)
        out[tok, slot] = y
    return out


def pertoken_stage2(a2_q, scale_a2, w2_q, scale_w2, topk_ids, topk_weights, model_dim: int,
                    doweight_stage2: bool = True, reduce: bool = True, group_size: int = -1, scale_w2_groups=None):
    """out[t] = sum_s (w[t,s]) * (a2[t,s] W2_e^T); a2_q [T,k,I] with scale_a2 [T,k,1], w2_q [E,H,I]
    with scale_w2 [E,H,1].  Returns f32 [T,H] (or [T,k,H] with ``reduce=False``)."""
    ids = torch.as_tensor(topk_ids).to(torch.int64)
    T, k = ids.shape
    E = w2_q.shape[0]
    a2 = a2_q.to(torch.float32) if scale_a2 is None else a2_q.to(torch.float32) * scale_a2
    out = torch.zeros((T, k, model_dim), dtype=torch.float32)
    for e in range(E):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        if group_size > 0 and scale_w2_groups is not None:
            w = _group_dequant(w2_q[e], scale_w2_groups[e], group_size)      # scale_w2_groups [E, I/group_size, H]
        else:
            w = w2_q[e].to(torch.float32) if scale_w2 is None else w2_q[e].to(torch.float32) * scale_w2[e]
        y = F.linear(a2[tok, slot], w)
        if doweight_stage2:
            y = y * torch.as_tensor(topk_weights)[tok, slot].unsqueeze(-1)
        out[tok, slot] = y
    return out.sum(dim=1) if reduce else out


# --------------------------------------------------------------------------- dense GEMM
def blockscale_gemm(xq: torch.Tensor, x_scale: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor,
                    dtype=torch.float32) -> torch.Tensor:
    """c = (xq * x_scale per 1x128) . (wq * w_scale per 128x128)^T in fp32, cast to ``dtype``.

    xq e4m3 [M, K]; x_scale f32 [M, K/128]; wq e4m3 [N, K]; w_scale f32 [ceil(N/128), K/128]."""
    x = _dequant_a(xq, x_scale)
    n, k = wq.shape
    w = wq.float() * w_scale.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)[:, :k]
    return F.linear(x, w).to(dtype)


# --------------------------------------------------------------------------- comparisons
def e4m3_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in representable e4m3 steps between two code tensors (uint8 or fp8)."""
    def ordinal(c):
        c = c.view(torch.uint8).to(torch.int32)
        mag = c & 0x7F
        return torch.where((c & 0x80) != 0, -mag, mag)
    return (ordinal(a) - ordinal(b)).abs()
