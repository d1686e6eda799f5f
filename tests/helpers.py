"""Shared test helpers: golden fixture loading and tensor conversions."""
from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
FP8 = torch.float8_e4m3fn


def load(name: str):
    return np.load(GOLDEN / name, allow_pickle=False)


def fp8_from_u8(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(FP8)


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def gen_sort_inputs(T, E, k, masked, device="cpu"):
    """Same generator as tests/golden/make_golden.py (unique experts per token)."""
    gg = torch.Generator().manual_seed(42 + T * 1000 + E * 10 + k)
    ids = torch.stack([torch.randperm(E, generator=gg)[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand((T, k), generator=gg, dtype=torch.float32)
    mask = None
    if masked:
        mask = (torch.rand(E, generator=gg) < 0.5).to(torch.int32)
        mask[0] = 1
    return ids.to(device), w.to(device), (None if mask is None else mask.to(device))


def fast_sort_inputs(T, E, k, seed, device="cpu"):
    """Vectorised unique-expert routing for large T."""
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand((T, E), generator=g)
    ids = torch.topk(scores, k, dim=1).indices.to(torch.int32)
    w = torch.rand((T, k), generator=g, dtype=torch.float32)
    return ids.to(device), w.to(device)


def pertoken_inputs(in_dtype, T, H, I, E, k, seed, quant):
    """Seeded inputs of the per-token-scale MoE family, following the reference test's recipe
    (tests/kernels/test_moe_gemm.py:380-400, :446-488 in the reference project): randn activations,
    randn/10 weights, routing = top-k of a softmax of random scores.  ``quant(x, quant_dtype=...)`` is
    the row quantiser (the reference's own when the fixtures are generated, the oracle's in the tests).
    "fp16" / "bf16" cast instead of quantising and have ``None`` scales (:451-462 there); "int4" / "int4_bf16"
    quantise the weights to int8 values in [-7, 7] (``dtypeMax=7``, :489-499; returned unpacked) with int8
    per-token or bf16 unscaled activations.
    Returns xq ([T,H], or [T,k,H] for "int8smooth"), sx, w1q [E,2I,H], sw1, w2q [E,H,I], sw2, ids, weights."""
    g = torch.Generator().manual_seed(seed)
    qd = FP8 if in_dtype == "fp8" else torch.int8
    x = torch.randn((T, H), generator=g)
    w1 = torch.randn((E, 2 * I, H), generator=g) / 10
    w2 = torch.randn((E, H, I), generator=g) / 10
    score = torch.softmax(torch.randn((T, E), generator=g), dim=1)
    tw, ti = torch.topk(score, k, dim=1)
    tw = tw.to(torch.float32)
    if in_dtype in ("fp16", "bf16"):
        dt = torch.float16 if in_dtype == "fp16" else torch.bfloat16
        return x.to(dt), None, w1.to(dt), None, w2.to(dt), None, ti.to(torch.int32), tw
    if in_dtype in ("int4", "int4_bf16"):
        if in_dtype == "int4":
            xq, sx = quant(x, quant_dtype=torch.int8)
        else:
            xq, sx = x.to(torch.bfloat16), None
        w1q, sw1 = quant(w1, quant_dtype=torch.int8, dtypeMax=7)
        w2q, sw2 = quant(w2, quant_dtype=torch.int8, dtypeMax=7)
        return xq, sx, w1q, sw1, w2q, sw2, ti.to(torch.int32), tw
    if in_dtype == "int8smooth":
        smooth = 0.75 + 0.5 * torch.rand((E, H), generator=g)
        xr = x[:, None, :] * smooth[ti.to(torch.int64)]
        amax = xr.abs().amax(dim=-1, keepdim=True)
        sx = amax / 127.0
        sx[sx == 0] = 1.0
        xq = (xr / sx).to(torch.int8)                       # [T, k, H], scales [T, k, 1]
    else:
        xq, sx = quant(x, quant_dtype=qd)
    w1q, sw1 = quant(w1, quant_dtype=qd)
    w2q, sw2 = quant(w2, quant_dtype=qd)
    return xq, sx, w1q, sw1, w2q, sw2, ti.to(torch.int32), tw


def group_scales(E, H, I, seed):
    """Group-wise weight scales of the W4A16 variant (one per 32-wide K group and weight row), as the reference's
    test draws them (tests/kernels/test_moe_gemm.py:512-514 there): f32 [E, H/32, 2I] and [E, I/32, H]."""
    g = torch.Generator().manual_seed(seed)
    g1 = torch.rand((E, H // 32, 2 * I), generator=g) * 0.05 + 0.005
    g2 = torch.rand((E, I // 32, H), generator=g) * 0.05 + 0.005
    return g1, g2
