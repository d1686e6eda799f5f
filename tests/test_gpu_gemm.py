"""GPU parity of the two grouped FP8 GEMM stages, called through the reference's launcher
signatures (kernels/moe_blockscale_2stage.py:1142-1157 and :2335-2350), against the CPU
oracle.  Bars: 16-bit outputs within rtol 2e-2 / atol 2e-2; the fused e4m3 intermediate
within 1 e4m3 step on at least 99.9 % of elements."""
import pytest
import torch

from flydsl_b200 import workloads as wl
from flydsl_b200.kernels import moe_blockscale_2stage as bs
from oracle import moe_oracle as orc
from tests.gpu_common import Problem, assert_close, ulp_stats

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 2e-2

MINI = wl.MoEConfig("mini", 16, 256, 128, 4, 2, 7)
SMALL = wl.MoEConfig("small", 200, 512, 256, 8, 2, 21)            # several row blocks per expert
REFSHAPE = wl.MoEConfig("ref-small-E8", 16, 7168, 256, 8, 2, 5)   # tests/kernels/test_moe_blockscale.py:225
ODD_N = wl.MoEConfig("odd-n", 48, 384, 128, 4, 2, 9)              # model_dim not a multiple of 256
_problems = {}


def problem(cfg):
    if cfg.name not in _problems:
        _problems[cfg.name] = Problem(cfg)
    return _problems[cfg.name]


def run_stage1(p, tile_m, impl, out_dtype, w_layout, doweight=False):
    cfg = p.cfg
    T, k, H, I, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
    s_ids, s_w, s_e, nv, nblk = p.sort(tile_m)
    exe = bs.compile_moe_blockscale_gemm1(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=128,
                                          tile_k=128, doweight_stage1=doweight, out_dtype=out_dtype,
                                          w_layout=w_layout, impl=impl)
    w = p.d_w1q if w_layout == "plain" else bs.shuffle_weight(p.d_w1q, E * 2 * I, H).view(-1)
    guard = 64
    if out_dtype == "fp8":
        out = torch.full((T * k + guard, I), 0x55, dtype=torch.uint8, device="cuda")
        osc = torch.full((I // 128, T * k), -1.0, dtype=torch.float32, device="cuda")
        exe(out.view(-1)[: T * k * I], p.d_xq.view(-1), w, p.d_xs_t.view(-1), p.d_w1s.view(-1), s_ids, s_e, s_w, nv,
            T, I, H, nblk, torch.cuda.current_stream(), arg_out_scale=osc)
        torch.cuda.synchronize()
        assert int((out[T * k:] != 0x55).sum()) == 0, "stage 1 wrote past its output rows"
        return out[: T * k].cpu(), osc.cpu()
    dt = {"f16": torch.float16, "bf16": torch.bfloat16}[out_dtype]
    out = torch.full((T * k + guard, I), 77.0, dtype=dt, device="cuda")
    exe(out.view(-1)[: T * k * I], p.d_xq.view(-1), w, p.d_xs_t.view(-1), p.d_w1s.view(-1), s_ids, s_e, s_w, nv,
        T, I, H, nblk, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert bool((out[T * k:] == 77.0).all()), "stage 1 wrote past its output rows"
    return out[: T * k].view(T, k, I).cpu(), None


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("cfg,tile_m,out_dtype,w_layout", [
    (MINI, 128, "f16", "plain"), (MINI, 16, "bf16", "preshuffle16x16"), (MINI, 32, "f16", "plain"),
    (MINI, 64, "bf16", "plain"), (SMALL, 128, "bf16", "preshuffle16x16"), (SMALL, 32, "f16", "plain"),
    (wl.CONFIGS["c1"], 128, "bf16", "plain"), (REFSHAPE, 16, "f16", "preshuffle16x16"),
])
def test_stage1_16bit_output(cfg, tile_m, out_dtype, w_layout, impl):
    p = problem(cfg)
    out, _ = run_stage1(p, tile_m, impl, out_dtype, w_layout)
    ref = orc.stage1(p.xq, p.xs, p.w1q, p.w1s, p.ids, cfg.inter_dim)
    assert_close(out, ref, RTOL, ATOL, f"stage1 {cfg.name} {impl}")
    # tighter than the bar: error dominated by the 16-bit rounding of the output
    eps = 2.0 ** -8 if out_dtype == "bf16" else 2.0 ** -11
    assert_close(out, ref, 2 * eps, 1e-4, f"stage1-tight {cfg.name} {impl}")


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("cfg,tile_m", [(MINI, 128), (SMALL, 64), (wl.CONFIGS["c1"], 128), (REFSHAPE, 16)])
def test_stage1_fused_requant(cfg, tile_m, impl):
    p = problem(cfg)
    codes, scales = run_stage1(p, tile_m, impl, "fp8", "plain")
    ref = orc.stage1(p.xq, p.xs, p.w1q, p.w1s, p.ids, cfg.inter_dim)
    for via_f16 in (False, True):
        rq, rs = orc.requant(ref, via_f16=via_f16)
        within1, exact, worst = ulp_stats(codes.view(torch.float8_e4m3fn), rq)
        assert within1 >= 0.999, f"{cfg.name} {impl}: only {within1:.5f} within 1 e4m3 step (worst {worst})"
        assert torch.allclose(scales.t(), rs, rtol=2e-3 if via_f16 else 1e-4, atol=0)
    assert exact > 0.98


def test_stage1_doweight():
    p = problem(MINI)
    out, _ = run_stage1(p, 128, "tcgen05", "f16", "plain", doweight=True)
    ref = orc.stage1(p.xq, p.xs, p.w1q, p.w1s, p.ids, MINI.inter_dim) * p.tw.view(MINI.tokens, MINI.topk, 1)
    assert_close(out, ref, RTOL, ATOL, "stage1 doweight")


def run_stage2(p, a2q, a2s, tile_m, impl, out_dtype, w_layout, accumulate=True, doweight=True):
    cfg = p.cfg
    T, k, H, I, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
    s_ids, s_w, s_e, nv, nblk = p.sort(tile_m)
    exe = bs.compile_moe_blockscale_gemm2(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256,
                                          tile_k=128, doweight_stage2=doweight, out_dtype=out_dtype,
                                          accumulate=accumulate, w_layout=w_layout, impl=impl)
    w = p.d_w2q if w_layout == "plain" else bs.shuffle_weight(p.d_w2q, E * H, I).view(-1)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[out_dtype]
    rows = T if accumulate else T * k
    out = torch.zeros((rows + 8, H), dtype=dt, device="cuda")
    exe(out.view(-1)[: rows * H], a2q.cuda().view(-1), w, a2s.t().contiguous().cuda().view(-1), p.d_w2s.view(-1),
        s_ids, s_e, s_w, nv, T, H, I, nblk, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert float(out[rows:].float().abs().sum()) == 0.0, "stage 2 wrote past its output rows"
    return out[:rows].cpu()


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("cfg,tile_m,out_dtype,w_layout", [
    (MINI, 128, "f16", "plain"), (MINI, 16, "bf16", "preshuffle16x16"), (MINI, 64, "f32", "plain"),
    (SMALL, 128, "bf16", "plain"), (SMALL, 32, "f32", "preshuffle16x16"), (ODD_N, 128, "bf16", "plain"),
    (ODD_N, 32, "f32", "plain"), (wl.CONFIGS["c1"], 128, "bf16", "plain"), (REFSHAPE, 16, "f16", "preshuffle16x16"),
])
def test_stage2_atomic(cfg, tile_m, out_dtype, w_layout, impl):
    p = problem(cfg)
    a2q, a2s = orc.requant(orc.stage1(p.xq, p.xs, p.w1q, p.w1s, p.ids, cfg.inter_dim))
    out = run_stage2(p, a2q, a2s, tile_m, impl, out_dtype, w_layout)
    ref = orc.stage2(a2q, a2s, p.w2q, p.w2s, p.ids, p.tw, cfg.model_dim)
    assert_close(out, ref, RTOL, ATOL, f"stage2 {cfg.name} {impl} {out_dtype}")
    if out_dtype == "f32":
        assert_close(out, ref, 1e-4, 1e-5 * float(ref.abs().max()), f"stage2-tight {cfg.name} {impl}")


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("cfg,tile_m", [(MINI, 128), (SMALL, 64), (ODD_N, 16)])
def test_stage2_no_atomic_and_reduce(cfg, tile_m, impl):
    p = problem(cfg)
    T, k, H = cfg.tokens, cfg.topk, cfg.model_dim
    a2q, a2s = orc.requant(orc.stage1(p.xq, p.xs, p.w1q, p.w1s, p.ids, cfg.inter_dim))
    pair = run_stage2(p, a2q, a2s, tile_m, impl, "bf16", "plain", accumulate=False)
    ref_pair = orc.stage2(a2q, a2s, p.w2q, p.w2s, p.ids, p.tw, H, reduce=False)
    assert_close(pair.view(T, k, H), ref_pair, RTOL, ATOL, f"stage2 pair rows {cfg.name} {impl}")
    red = bs.compile_moe_reduction(topk=k, model_dim=H, dtype_str="bf16")
    y = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    red(pair.cuda().view(T, k, H), y, torch.empty((0, k), dtype=torch.uint8, device="cuda"), T,
        torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(y.cpu(), orc.topk_reduce(pair.view(T, k, H)))
    # the wrapper that chains both, as the reference's "reduce" mode does
    exe = bs.compile_moe_blockscale_gemm2_ex(model_dim=H, inter_dim=cfg.inter_dim, experts=cfg.experts, topk=k,
                                             tile_m=tile_m, tile_n=256, tile_k=128, doweight_stage2=True,
                                             out_dtype="bf16", mode=bs.MoeGemm2Mode.REDUCE, w_layout="plain",
                                             impl=impl)
    s_ids, s_w, s_e, nv, nblk = p.sort(tile_m)
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    exe(out.view(-1), a2q.cuda().view(-1), p.d_w2q, a2s.t().contiguous().cuda().view(-1), p.d_w2s.view(-1), s_ids,
        s_e, s_w, nv, T, H, cfg.inter_dim, nblk)
    torch.cuda.synchronize()
    assert_close(out, orc.stage2(a2q, a2s, p.w2q, p.w2s, p.ids, p.tw, H), RTOL, ATOL, "stage2 reduce mode")


@pytest.mark.parametrize("cfg,tile_m", [(SMALL, 128), (SMALL, 64), (MINI, 16), (wl.CONFIGS["c1"], 32)])
def test_in_kernel_row_gather_through_the_c_abi(cfg, tile_m):
    """x_layout BY_TOKEN / a_layout BY_PAIR on the tensor-core path: the kernel fetches every sorted row by
    index itself (the launchers choose this only for 16- and 32-row blocks; any block size must be right)."""
    from flydsl_b200 import _lib
    lib = _lib.load()
    p = problem(cfg)
    T, k, H, I, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
    s_ids, s_w, s_e, nv, nblk = p.sort(tile_m)
    st = torch.cuda.current_stream().cuda_stream
    out1 = torch.full((T * k + 8, I), 77.0, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.flymoe_moe_gemm1(
        out1.data_ptr(), None, 0, p.d_xq.data_ptr(), p.d_xs_t.data_ptr(), T, 1, p.d_w1q.data_ptr(), p.d_w1s.data_ptr(),
        s_ids.data_ptr(), s_e.data_ptr(), s_w.data_ptr(), nv.data_ptr(), T, I, H, nblk, E, k, tile_m, 0, _lib.BF16,
        _lib.ROWS_BY_TOKEN, _lib.ROWS_BY_TOKEN, _lib.ROWS_BY_PAIR, _lib.IMPL_TCGEN05, st), "gemm1")
    torch.cuda.synchronize()
    ref1 = orc.stage1(p.xq, p.xs, p.w1q, p.w1s, p.ids, I)
    assert bool((out1[T * k:] == 77.0).all())
    assert_close(out1[: T * k].view(T, k, I), ref1, RTOL, ATOL, f"stage 1, rows gathered in the kernel, {cfg.name}")
    a2q, a2s = orc.requant(ref1)
    out2 = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    a2s_t = a2s.t().contiguous().cuda()
    _lib.check(lib.flymoe_moe_gemm2(
        out2.data_ptr(), a2q.cuda().data_ptr(), a2s_t.data_ptr(), T * k, p.d_w2q.data_ptr(), p.d_w2s.data_ptr(),
        s_ids.data_ptr(), s_e.data_ptr(), s_w.data_ptr(), nv.data_ptr(), T, H, I, nblk, E, k, tile_m, 1, _lib.F32, 1,
        _lib.ROWS_BY_PAIR, _lib.ROWS_BY_PAIR, _lib.IMPL_TCGEN05, st), "gemm2")
    torch.cuda.synchronize()
    ref2 = orc.stage2(a2q, a2s, p.w2q, p.w2s, p.ids, p.tw, H)
    assert_close(out2, ref2, 1e-4, 1e-5 * float(ref2.abs().max()), f"stage 2, rows gathered in the kernel, {cfg.name}")
