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
