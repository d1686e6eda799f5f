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
