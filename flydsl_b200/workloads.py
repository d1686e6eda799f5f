"""Seeded synthetic inputs for the FP8 block-scaled MoE layer.

Stand-ins for real model weights/activations: shapes, dtypes and value
distributions of the five benchmark configurations, generated from fixed seeds
with torch ops on whichever device is asked for (CPU for the parity fixtures,
CUDA for the benchmark).  Quantisation here follows the reference's test-side
quantiser (tests/utils.py:29-73 in the reference project: scale = amax/448 with
0 -> 1, q = (x/scale).to(e4m3)), so the CPU oracle and the CUDA kernels see
byte-identical pre-quantised tensors.  This is input preparation, not part of
the measured path.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
BLK = 128


@dataclass(frozen=True)
class MoEConfig:
    name: str
    tokens: int
    model_dim: int
    inter_dim: int
    experts: int
    topk: int
    seed: int
    routing: str = "uniform"  # "uniform" | "zipf"

    @property
    def pairs(self) -> int:
        return self.tokens * self.topk

    def flops(self) -> float:
        """Algorithmic FLOPs of the layer: 6*T*k*H*I (pad rows, scales, SiLU not counted)."""
        return 6.0 * self.tokens * self.topk * self.model_dim * self.inter_dim

    def with_tokens(self, tokens: int) -> "MoEConfig":
        return replace(self, tokens=tokens, name=f"{self.name}-T{tokens}")


CONFIGS = {
    "c1": MoEConfig("c1-tiny", 32, 1024, 512, 8, 2, 0),
    "c2": MoEConfig("c2-mixtral", 1024, 4096, 14336, 8, 2, 1),
    "c3": MoEConfig("c3-dsv3-decode", 64, 7168, 2048, 256, 8, 2),
    "c4a": MoEConfig("c4a-dsv3-prefill-uniform", 4096, 7168, 2048, 256, 8, 3, "uniform"),
    "c4b": MoEConfig("c4b-dsv3-prefill-zipf", 4096, 7168, 2048, 256, 8, 3, "zipf"),
    "c5a": MoEConfig("c5a-dsv3-ep-uniform", 16384, 7168, 2048, 256, 8, 4, "uniform"),
    "c5b": MoEConfig("c5b-dsv3-ep-zipf", 16384, 7168, 2048, 256, 8, 4, "zipf"),
}
C2_TOKEN_SWEEP = (1, 16, 128, 1024, 8192)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def quant_groups(x: torch.Tensor):
    """Quantise along the last dim: returns (q e4m3, scale f32 [..., 1])."""
    x = x.to(torch.float32)
    amax = torch.maximum(x.amax(dim=-1, keepdim=True), -x.amin(dim=-1, keepdim=True))
    scale = amax / FP8_MAX
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    return (x / scale).to(FP8), scale


def quant_act_1x128(x: torch.Tensor):
    """[R,K] -> (q e4m3 [R,K], scale f32 [R,K/128])."""
    R, K = x.shape
    q, s = quant_groups(x.reshape(R, K // BLK, BLK))
    return q.reshape(R, K), s.reshape(R, K // BLK)


def quant_weight_128x128(w: torch.Tensor):
    """[N,K] -> (q e4m3 [N,K], scale f32 [N/128,K/128])."""
    N, K = w.shape
    nbn, nbk = N // BLK, K // BLK
    t = w.to(torch.float32).view(nbn, BLK, nbk, BLK).permute(0, 2, 1, 3).reshape(nbn * nbk, BLK * BLK)
    q, s = quant_groups(t)
    q = q.view(nbn, nbk, BLK, BLK).permute(0, 2, 1, 3).reshape(N, K).contiguous()
    return q, s.view(nbn, nbk).contiguous()


def make_logits(cfg: MoEConfig, device="cpu", rank: int = 0) -> torch.Tensor:
    """Router logits f32 [T,E] ~ N(0,1); 'zipf' adds -2.2*ln(rank_e) over a seeded permutation."""
    g = _gen(cfg.seed * 1000 + 17 + rank, device)
    logits = torch.randn((cfg.tokens, cfg.experts), generator=g, device=device, dtype=torch.float32)
    if cfg.routing == "zipf":
        gp = _gen(cfg.seed * 1000 + 23, "cpu")
        perm = torch.randperm(cfg.experts, generator=gp)
        rank_of = torch.empty(cfg.experts, dtype=torch.float32)
        rank_of[perm] = torch.arange(1, cfg.experts + 1, dtype=torch.float32)
        bias = 2.0 * torch.log(rank_of.pow(-1.1))
        logits = logits + bias.to(device).view(1, -1)
    elif cfg.routing != "uniform":
        raise ValueError(f"unknown routing {cfg.routing!r}")
    return logits


def make_activations(cfg: MoEConfig, device="cpu", rank: int = 0):
    """x bf16 ~ N(0,1) [T,H] -> (x_bf16, xq e4m3 [T,H], x_scale f32 [T,H/128])."""
    g = _gen(cfg.seed * 1000 + 31 + rank, device)
    x = torch.randn((cfg.tokens, cfg.model_dim), generator=g, device=device, dtype=torch.float32)
    x = x.to(torch.bfloat16)
    xq, xs = quant_act_1x128(x)
    return x, xq, xs


def make_weights(cfg: MoEConfig, device="cpu", experts: range | None = None, std: float = 0.02):
    """W1 [E,2I,H], W2 [E,H,I] ~ N(0,std), one expert at a time -> e4m3 + 128x128 block scales.

    ``experts`` selects a sub-range of global expert ids (expert parallelism);
    each expert's values depend only on (seed, expert id).
    """
    ex = range(cfg.experts) if experts is None else experts
    n = len(ex)
    H, I = cfg.model_dim, cfg.inter_dim
    w1q = torch.empty((n, 2 * I, H), dtype=FP8, device=device)
    w1s = torch.empty((n, 2 * I // BLK, H // BLK), dtype=torch.float32, device=device)
    w2q = torch.empty((n, H, I), dtype=FP8, device=device)
    w2s = torch.empty((n, H // BLK, I // BLK), dtype=torch.float32, device=device)
    for j, e in enumerate(ex):
        g = _gen(cfg.seed * 100003 + 7919 * e + 1, device)
        w1 = torch.randn((2 * I, H), generator=g, device=device, dtype=torch.float32) * std
        w1q[j], w1s[j] = quant_weight_128x128(w1)
        del w1
        w2 = torch.randn((H, I), generator=g, device=device, dtype=torch.float32) * std
        w2q[j], w2s[j] = quant_weight_128x128(w2)
        del w2
    return w1q, w1s, w2q, w2s


def weight_bytes_active(cfg: MoEConfig, topk_ids: torch.Tensor) -> float:
    """Algorithmic HBM bytes of the layer: fp8 weights (+ block scales) of experts that
    received at least one token, plus activations, fp8 intermediate, output and routing."""
    H, I, T, k = cfg.model_dim, cfg.inter_dim, cfg.tokens, cfg.topk
    e_act = int(torch.unique(topk_ids).numel())
    w = e_act * 3.0 * H * I
    ws = e_act * (2 * I * H + H * I) / (BLK * BLK) * 4.0
    x = T * H * (1 + 4.0 / BLK)
    inter = 2.0 * T * k * I * (1 + 4.0 / BLK)
    out = T * H * 2.0
    rmax = T * k + cfg.experts * 128 - k
    routing = T * cfg.experts * 4.0 + 5.0 * rmax * 4.0
    return w + ws + x + inter + out + routing


def describe(cfg: MoEConfig) -> dict:
    return {"workload": cfg.name, "tokens": cfg.tokens, "model_dim": cfg.model_dim,
            "inter_dim": cfg.inter_dim, "experts": cfg.experts, "topk": cfg.topk,
            "seed": cfg.seed, "routing": cfg.routing,
            "gflop": round(cfg.flops() / 1e9, 3)}
