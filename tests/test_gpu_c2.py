"""GPU parity on the Mixtral-8x7B-shaped configuration (H=4096, I=14336, E=8, top-2, seed 1) over its
token sweep T in {1, 16, 128, 1024, 8192}: 112 K blocks in stage 2 and thousands of rows per expert,
shapes no other test reaches.  Per T: routing bit-exact against the oracle; a token subset that
hits every active expert (at least 32 tokens, all of them for small T) compared with the CPU oracle
at the bars (fused e4m3 intermediate within 1 step on >= 99.9 %, bf16 output rtol/atol 2e-2); the
whole output against the CUDA-core implementation for T <= 1024.  One T also goes through the
reference's launcher signatures with the reference's preshuffled weight layout
(tests/kernels/test_moe_blockscale.py:405-421, :492-506 in the reference project)."""
import pytest
import torch

from flydsl_b200 import workloads as wl
from flydsl_b200.kernels import moe_blockscale_2stage as bs
from flydsl_b200.layer import FusedMoEBlockscale
from oracle import moe_oracle as orc
from tests.gpu_common import LazyExperts, assert_close, covering_subset, ulp_stats

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 2e-2
C2 = wl.CONFIGS["c2"]
_weights = {}


def weights():
    """The 1.4 GB of e4m3 expert weights depend only on the seed and the expert id: made once, on the GPU."""
    if "w" not in _weights:
        _weights["w"] = wl.make_weights(C2, device="cuda")
    return _weights["w"]


def tile_for(T):
    rows = T * C2.topk / C2.experts
    return 16 if rows <= 16 else 32 if rows <= 32 else 64 if rows <= 64 else 128


def oracle_subset(cfg, sel, xq, xs, ids, tw):
    w1q, w1s, w2q, w2s = (LazyExperts(t) for t in weights())
    o1 = orc.stage1(xq[sel], xs[sel], w1q, w1s, ids[sel], cfg.inter_dim)
    a2q, a2s = orc.requant(o1)
    return a2q, a2s, orc.stage2(a2q, a2s, w2q, w2s, ids[sel], tw[sel], cfg.model_dim)


@pytest.mark.parametrize("T", wl.C2_TOKEN_SWEEP)
def test_c2_layer(T):
    cfg = C2.with_tokens(T)
    k, H, I = cfg.topk, cfg.model_dim, cfg.inter_dim
    w1q, w1s, w2q, w2s = weights()
    logits = wl.make_logits(cfg)
    _x, xq, xs = wl.make_activations(cfg)
    tw, ids, _ = orc.topk_gating_softmax(logits, k)
    d_logits, d_xq, d_xs_t = logits.cuda(), xq.cuda(), xs.t().contiguous().cuda()
    tile_m = tile_for(T)
    layer = FusedMoEBlockscale(w1q, w1s, w2q, w2s, k, max_tokens=T, tile_m=tile_m)
    out = layer(d_logits, d_xq, d_xs_t)
    torch.cuda.synchronize()
    assert torch.equal(layer.topk_ids[:T].cpu(), ids), "routing must be bit-exact"
    assert torch.allclose(layer.topk_weights[:T].cpu(), tw, atol=1e-6, rtol=1e-5)
    assert torch.isfinite(out.float()).all()

    sel = torch.tensor(covering_subset(ids, 32))
    a2q, _a2s, ref = oracle_subset(cfg, sel, xq, xs, ids, tw)
    # the layer's intermediate, mapped back from sorted order to (token, slot) rows
    nv = int(layer.num_valid_ids[0])
    sid = layer.sorted_ids[:nv].cpu()
    tok, slot = sid & 0xFFFFFF, sid >> 24
    valid = tok < T
    assert int(valid.sum()) == T * k
    codes = torch.zeros((T * k, I), dtype=torch.uint8)
    codes[(tok * k + slot)[valid].long()] = layer.a2q[:nv].cpu()[valid]
    pair_rows = (sel.view(-1, 1) * k + torch.arange(k).view(1, -1)).reshape(-1)
    within1, _exact, worst = ulp_stats(codes[pair_rows].view(torch.float8_e4m3fn), a2q)
    assert within1 >= 0.999, f"T={T}: intermediate {within1:.5f} within 1 e4m3 step (worst {worst})"
    step = 2.0 ** -7 * float(ref.abs().max()) if T > 1 else 0.0       # bf16 atomics: one rounding step of the sum
    assert_close(out[sel.cuda()], ref, RTOL, ATOL + step, f"c2 T={T} subset vs oracle")

    if T <= 1024:
        simt = FusedMoEBlockscale(w1q, w1s, w2q, w2s, k, max_tokens=T, tile_m=tile_m, impl="simt")
        out_s = simt(d_logits, d_xq, d_xs_t)
        torch.cuda.synchronize()
        assert_close(out, out_s, RTOL, ATOL + 2.0 ** -7 * float(out_s.float().abs().max()), f"c2 T={T} tcgen05 vs simt")


def test_c2_reference_launcher_signatures():
    """T=128 through compile_moe_blockscale_gemm1/2 exactly as the reference's test drives them: flattened
    views, preshuffled weights, f16 stage-1 output, requantisation outside, atomic stage 2."""
    from flydsl_b200.kernels.moe_sorting_kernel import moe_sorting_flydsl
    T = 128
    cfg = C2.with_tokens(T)
    k, H, I, E = cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
    w1q, w1s, w2q, w2s = weights()
    logits = wl.make_logits(cfg)
    _x, xq, xs = wl.make_activations(cfg)
    tw, ids, _ = orc.topk_gating_softmax(logits, k)
    unit = 32
    cap = T * k + E * unit - k
    nblk = (cap + unit - 1) // unit
    d = "cuda"
    s_ids = torch.empty(cap, dtype=torch.int32, device=d)
    s_w = torch.empty(cap, dtype=torch.float32, device=d)
    s_e = torch.empty(nblk, dtype=torch.int32, device=d)
    nv = torch.empty(2, dtype=torch.int32, device=d)
    moe_sorting_flydsl(ids.cuda(), tw.cuda(), s_ids, s_w, s_e, nv, None, E, unit)
    w1_shuf = bs.shuffle_weight(w1q, E * 2 * I, H).view(-1)
    w2_shuf = bs.shuffle_weight(w2q, E * H, I).view(-1)
    exe1 = bs.compile_moe_blockscale_gemm1(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=unit, tile_n=128,
                                           tile_k=128, doweight_stage1=False, out_dtype="f16")
    out1 = torch.empty((T, k, I), dtype=torch.float16, device=d)
    exe1(out1.view(-1), xq.cuda().view(-1), w1_shuf, xs.t().contiguous().cuda().view(-1), w1s.view(-1), s_ids, s_e, s_w,
         nv, T, I, H, nblk, torch.cuda.current_stream())
    torch.cuda.synchronize()
    lw = [LazyExperts(t) for t in (w1q, w1s, w2q, w2s)]
    ref1 = orc.stage1(xq, xs, lw[0], lw[1], ids, I)
    assert_close(out1.cpu(), ref1, RTOL, ATOL, "c2 stage 1 through the reference launcher")
    a2q, a2s = orc.requant(out1.float().cpu())                    # the reference requantises its own f16 output
    exe2 = bs.compile_moe_blockscale_gemm2(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=unit, tile_n=256,
                                           tile_k=128, doweight_stage2=True, out_dtype="bf16")
    out2 = torch.zeros((T, H), dtype=torch.bfloat16, device=d)
    exe2(out2.view(-1), a2q.cuda().view(-1), w2_shuf, a2s.t().contiguous().cuda().view(-1), w2s.view(-1), s_ids, s_e,
         s_w, nv, T, H, I, nblk, torch.cuda.current_stream())
    torch.cuda.synchronize()
    ref2 = orc.stage2(a2q, a2s, lw[2], lw[3], ids, tw, H)
    assert_close(out2.cpu(), ref2, RTOL, ATOL + 2.0 ** -7 * float(ref2.abs().max()), "c2 stage 2 through the reference launcher")
    bs.clear_weight_cache()
