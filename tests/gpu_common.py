"""Helpers shared by the GPU GEMM / layer tests (not collected by pytest)."""
from __future__ import annotations

import torch

from flydsl_b200 import workloads as wl
from flydsl_b200.kernels.moe_sorting_kernel import moe_sorting_flydsl
from oracle import moe_oracle as orc

FP8 = torch.float8_e4m3fn


class Problem:
    """Seeded inputs of one configuration, on the CPU and on the GPU, with CPU routing."""

    def __init__(self, cfg: wl.MoEConfig, weights_on: str = "cpu"):
        self.cfg = cfg
        self.logits = wl.make_logits(cfg)
        _x, self.xq, self.xs = wl.make_activations(cfg)
        self.w1q, self.w1s, self.w2q, self.w2s = wl.make_weights(cfg, device=weights_on)
        self.tw, self.ids, self.tei = orc.topk_gating_softmax(self.logits, cfg.topk, True)
        d = "cuda"
        self.d_logits = self.logits.to(d)
        self.d_xq = self.xq.to(d)
        self.d_xs_t = self.xs.t().contiguous().to(d)          # [H/128, T]
        self.d_w1q, self.d_w1s = self.w1q.to(d), self.w1s.to(d)
        self.d_w2q, self.d_w2s = self.w2q.to(d), self.w2s.to(d)
        self.d_ids, self.d_tw = self.ids.to(d), self.tw.to(d)

    def sort(self, unit: int):
        cfg = self.cfg
        T, k, E = cfg.tokens, cfg.topk, cfg.experts
        cap = T * k + E * unit - k
        nblk = (cap + unit - 1) // unit
        d = "cuda"
        s_ids = torch.empty(cap, dtype=torch.int32, device=d)
        s_w = torch.empty(cap, dtype=torch.float32, device=d)
        s_e = torch.empty(nblk, dtype=torch.int32, device=d)
        nv = torch.empty(2, dtype=torch.int32, device=d)
        moe_sorting_flydsl(self.d_ids, self.d_tw, s_ids, s_w, s_e, nv, None, E, unit)
        return s_ids, s_w, s_e, nv, nblk


def ulp_stats(codes_a: torch.Tensor, codes_b: torch.Tensor):
    d = orc.e4m3_ulp_distance(codes_a.cpu(), codes_b.cpu())
    return float((d <= 1).float().mean()), float((d == 0).float().mean()), int(d.max())


def assert_close(actual: torch.Tensor, ref: torch.Tensor, rtol: float, atol: float, what: str):
    a, r = actual.detach().float().cpu(), ref.detach().float().cpu()
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    err = (a - r).abs()
    bad = err > (atol + rtol * r.abs())
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.numel()} outside rtol={rtol} atol={atol}; "
                           f"max abs err {float(err.max()):.4g}, ref max {float(r.abs().max()):.4g}")


def covering_subset(topk_ids: torch.Tensor, min_tokens: int = 32, base=()) -> list:
    """Tokens (ascending) such that every expert that received a token is hit by at least one of them,
    padded with evenly spaced tokens up to ``min_tokens``: the oracle then dequantises, and the check
    compares, the weight tiles of every active expert."""
    ids = torch.as_tensor(topk_ids).to(torch.int64)
    T = ids.shape[0]
    chosen = set(int(t) for t in base)
    covered = set(ids[sorted(chosen)].reshape(-1).tolist()) if chosen else set()
    active = set(ids.reshape(-1).tolist())
    for t in range(T):
        if covered >= active:
            break
        row = set(ids[t].tolist())
        if not row <= covered:
            chosen.add(t)
            covered |= row
    want = min(min_tokens, T)
    i = 0
    while len(chosen) < want:
        chosen.add(int(round(i * (T - 1) / max(1, want - 1))))
        i += 1
        if i > 4 * want:
            chosen.update(range(want))
    return sorted(chosen)


class LazyExperts:
    """Expert-indexable view that copies one expert's weights to the CPU on demand."""

    def __init__(self, t):
        self.t = t

    def __len__(self):
        return self.t.shape[0]

    def __getitem__(self, e):
        return self.t[e].cpu()
