"""GPU parity of the per-token / per-channel-scale MoE family (kernels.moe_gemm_2stage) against
the CPU oracle, called through the reference's launcher signatures
(kernels/moe_gemm_2stage.py:1730-1745 and :3151-3166) on the shapes of the reference's own test
(tests/kernels/test_moe_gemm.py:1661-1672: S, M and the aiter-style L).  The oracle is pinned to
the reference's torch_moe_gemm1/2 by tests/golden/moe_pertoken.npz.  Bars: 16-bit and fp32
outputs within rtol 2e-2 / atol 2e-2 (16-bit atomics: plus one rounding step of the largest sum)."""
import pytest
import torch

from flydsl_b200.kernels import moe_gemm_2stage as pt
from flydsl_b200.kernels.moe_blockscale_2stage import shuffle_weight
from flydsl_b200.kernels.moe_sorting_kernel import moe_sorting_flydsl
from oracle import moe_oracle as orc
from tests import helpers as hp
from tests.gpu_common import assert_close

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 2e-2

#            tokens H     I     E   k  tile_m
SHAPES = {"S": (64, 256, 128, 4, 2, 16), "M": (129, 1024, 256, 8, 2, 32), "L": (333, 4096, 2048, 17, 9, 64),
          "T128": (700, 512, 256, 4, 2, 128)}
_cache = {}


def inputs(shape, in_dtype):
    key = (shape, in_dtype)
    if key not in _cache:
        T, H, I, E, k, _ = SHAPES[shape]
        _cache[key] = hp.pertoken_inputs(in_dtype, T, H, I, E, k, 77 + len(shape), orc.quant_rows)
    return _cache[key]


def sort(ids, tw, E, unit):
    T, k = ids.shape
    cap = T * k + E * unit - k
    nblk = (cap + unit - 1) // unit
    d = "cuda"
    s_ids = torch.empty(cap, dtype=torch.int32, device=d)
    s_w = torch.empty(cap, dtype=torch.float32, device=d)
    s_e = torch.empty(nblk, dtype=torch.int32, device=d)
    nv = torch.empty(2, dtype=torch.int32, device=d)
    moe_sorting_flydsl(ids.cuda(), tw.cuda(), s_ids, s_w, s_e, nv, None, E, unit)
    return s_ids, s_w, s_e, nv, nblk


HALF = {"fp16": torch.float16, "bf16": torch.bfloat16}


def scale_arg(s):
    """Scales as the launcher takes them; the 16-bit variants have none and get the reference's empty tensor."""
    return torch.empty(0, dtype=torch.float32, device="cuda") if s is None else s.cuda().view(-1)


def dev_weight(wq, layout, in_dtype="fp8"):
    E, N, K = wq.shape
    if in_dtype in ("int4", "int4_bf16"):          # the reference's packed bytes (preshuffled order only)
        return orc.pack_int4_preshuffled(wq).cuda()
    w = wq.cuda()
    return w if layout == "plain" else shuffle_weight(w, E * N, K).view(-1)


def run_stage1(shape, in_dtype, out_dtype, impl, w_layout, doweight):
    T, H, I, E, k, tile_m = SHAPES[shape]
    xq, sx, w1q, sw1, _w2q, _sw2, ids, tw = inputs(shape, in_dtype)
    s_ids, s_w, s_e, nv, nblk = sort(ids, tw, E, tile_m)
    exe = pt.compile_moe_gemm1(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=128, tile_k=128,
                               doweight_stage1=doweight, in_dtype=in_dtype, out_dtype=out_dtype, w_layout=w_layout,
                               impl=impl)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16}[out_dtype]
    out = torch.full((T * k + 16, I), 77.0, dtype=dt, device="cuda")
    if in_dtype == "int8smooth":      # per-(token, slot) rows travel slot-major, as the reference's kernel reads them
        x_arg, sx_arg = xq.permute(1, 0, 2).contiguous().cuda().view(-1, H), scale_arg(sx.permute(1, 0, 2).contiguous())
    else:
        x_arg, sx_arg = xq.cuda().view(-1, H), scale_arg(sx)
    exe(out.view(-1)[: T * k * I], x_arg, dev_weight(w1q, w_layout, in_dtype), sx_arg,
        scale_arg(sw1), s_ids, s_e, s_w, nv, T, I, H, nblk, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert bool((out[T * k:] == 77.0).all()), "stage 1 wrote past its output rows"
    ref = orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I, doweight)
    return out[: T * k].view(T, k, I).cpu(), ref


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("shape,in_dtype,out_dtype,w_layout,doweight", [
    ("S", "fp8", "f16", "plain", False), ("S", "int8", "bf16", "preshuffle16x16", False),
    ("S", "int8smooth", "f16", "plain", False), ("M", "fp8", "bf16", "preshuffle16x16", True),
    ("M", "int8", "f16", "plain", False), ("M", "int8smooth", "bf16", "plain", False),
    ("T128", "fp8", "bf16", "plain", False), ("T128", "int8", "f16", "plain", True),
])
def test_pertoken_stage1(shape, in_dtype, out_dtype, w_layout, doweight, impl):
    out, ref = run_stage1(shape, in_dtype, out_dtype, impl, w_layout, doweight)
    assert_close(out, ref, RTOL, ATOL, f"per-token stage 1 {shape} {in_dtype} {impl}")
    eps = 2.0 ** -8 if out_dtype == "bf16" else 2.0 ** -11
    assert_close(out, ref, 2 * eps, 1e-3, f"per-token stage 1 tight {shape} {in_dtype} {impl}")


def run_stage2(shape, in_dtype, out_dtype, impl, w_layout, mode, doweight=True):
    T, H, I, E, k, tile_m = SHAPES[shape]
    xq, sx, w1q, sw1, w2q, sw2, ids, tw = inputs(shape, in_dtype)
    qd = hp.FP8 if in_dtype == "fp8" else torch.int8
    o1 = orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I, False)
    if in_dtype in HALF or in_dtype == "int4_bf16":
        a2q, sa2 = o1.to(HALF.get(in_dtype, torch.bfloat16)), None
    else:
        a2q, sa2 = orc.quant_rows(o1, qd)
    s_ids, s_w, s_e, nv, nblk = sort(ids, tw, E, tile_m)
    common = dict(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256, tile_k=128,
                  doweight_stage2=doweight, in_dtype=in_dtype, out_dtype=out_dtype, w_layout=w_layout, impl=impl)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[out_dtype]
    w = dev_weight(w2q, w_layout, in_dtype)
    args = (a2q.cuda().view(-1, I), w, scale_arg(sa2), scale_arg(sw2), s_ids, s_e, s_w, nv, T, H, I, nblk)
    if mode == "rows":
        exe = pt.compile_moe_gemm2(accumulate=False, **common)
        out = torch.zeros((T * k + 8, H), dtype=dt, device="cuda")
        exe(out.view(-1)[: T * k * H], *args, torch.cuda.current_stream())
        rows = T * k
    else:
        exe = pt.compile_moe_gemm2_ex(mode=mode, **common)
        out = torch.zeros((T + 8, H), dtype=dt, device="cuda")
        if mode == "reduce":
            exe(out.view(-1)[: T * H], *args)
            exe(out.view(-1)[: T * H], *args)          # second call reuses the wrapper's row buffer
        else:
            exe(out.view(-1)[: T * H], *args, torch.cuda.current_stream())
        rows = T
    torch.cuda.synchronize()
    assert float(out[rows:].float().abs().sum()) == 0.0, "stage 2 wrote past its output rows"
    pair = orc.pertoken_stage2(a2q, sa2, w2q, sw2, ids, tw, H, doweight, reduce=False)
    ref = pair.view(rows, H) if mode == "rows" else pair.sum(dim=1)
    return out[:rows].cpu(), ref, float(pair.abs().max())


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("shape,in_dtype,out_dtype,w_layout,mode", [
    ("S", "fp8", "f16", "plain", "atomic"), ("S", "fp8", "f32", "preshuffle16x16", "atomic"),
    ("S", "int8", "bf16", "plain", "reduce"), ("S", "int8smooth", "f16", "plain", "rows"),
    ("M", "fp8", "bf16", "plain", "atomic"), ("M", "fp8", "f16", "preshuffle16x16", "reduce"),
    ("M", "int8", "f32", "plain", "atomic"), ("T128", "fp8", "bf16", "plain", "reduce"),
    ("T128", "int8", "bf16", "plain", "atomic"),
])
def test_pertoken_stage2(shape, in_dtype, out_dtype, w_layout, mode, impl):
    out, ref, pair_peak = run_stage2(shape, in_dtype, out_dtype, impl, w_layout, mode)
    # 16-bit outputs round every (token, slot) term (per-pair rows, or the running sum of the atomics):
    # allow one rounding step of the largest term on top of the bar (terms of opposite sign cancel)
    step = 0.0 if out_dtype == "f32" or mode == "rows" else 2.0 ** (-7 if out_dtype == "bf16" else -10) * pair_peak
    assert_close(out, ref, RTOL, ATOL + step, f"per-token stage 2 {shape} {in_dtype} {mode} {impl}")
    if out_dtype == "f32":
        assert_close(out, ref, 1e-4, 1e-5 * pair_peak, f"per-token stage 2 tight {shape} {in_dtype} {impl}")


@pytest.mark.parametrize("shape,in_dtype,out_dtype,w_layout,doweight", [
    ("S", "bf16", "bf16", "preshuffle16x16", False), ("S", "fp16", "f16", "plain", True),
    ("M", "bf16", "f16", "plain", False), ("M", "fp16", "f16", "preshuffle16x16", False),
    ("T128", "bf16", "bf16", "preshuffle16x16", False), ("T128", "fp16", "bf16", "plain", True),
])
def test_pertoken_stage1_16bit_operands(shape, in_dtype, out_dtype, w_layout, doweight):
    """fp16 / bf16 activations and weights, no scales (tests/kernels/test_moe_gemm.py:451-462, :569-579 of
    the reference): the same launcher, the scale arguments are the reference's empty tensors."""
    out, ref = run_stage1(shape, in_dtype, out_dtype, "tcgen05", w_layout, doweight)
    assert_close(out, ref, RTOL, ATOL, f"16-bit stage 1 {shape} {in_dtype}")
    eps = 2.0 ** -8 if out_dtype == "bf16" else 2.0 ** -11
    assert_close(out, ref, 2 * eps, 1e-3, f"16-bit stage 1 tight {shape} {in_dtype}")


@pytest.mark.parametrize("shape,in_dtype,out_dtype,w_layout,mode", [
    ("S", "bf16", "f32", "plain", "atomic"), ("S", "fp16", "f16", "preshuffle16x16", "rows"),
    ("M", "bf16", "bf16", "preshuffle16x16", "reduce"), ("M", "fp16", "f32", "plain", "atomic"),
    ("T128", "bf16", "bf16", "plain", "atomic"), ("T128", "fp16", "f16", "preshuffle16x16", "reduce"),
])
def test_pertoken_stage2_16bit_operands(shape, in_dtype, out_dtype, w_layout, mode):
    out, ref, pair_peak = run_stage2(shape, in_dtype, out_dtype, "tcgen05", w_layout, mode)
    step = 0.0 if out_dtype == "f32" or mode == "rows" else 2.0 ** (-7 if out_dtype == "bf16" else -10) * pair_peak
    assert_close(out, ref, RTOL, ATOL + step, f"16-bit stage 2 {shape} {in_dtype} {mode}")
    if out_dtype == "f32":
        assert_close(out, ref, 1e-4, 1e-5 * pair_peak, f"16-bit stage 2 tight {shape} {in_dtype}")


@pytest.mark.parametrize("shape,in_dtype,out_dtype,doweight", [
    ("S", "int4", "f16", False), ("S", "int4_bf16", "bf16", True), ("M", "int4", "bf16", True),
    ("M", "int4_bf16", "f16", False), ("T128", "int4", "bf16", False), ("T128", "int4_bf16", "bf16", False),
])
def test_pertoken_stage1_packed_int4_weights(shape, in_dtype, out_dtype, doweight):
    """W4A8 / W4A16 (tests/kernels/test_moe_gemm.py:489-499 of the reference): the weights arrive as its packed
    int4 bytes; the launcher unpacks them once and runs the int8 / bf16 kernels."""
    out, ref = run_stage1(shape, in_dtype, out_dtype, "tcgen05", "preshuffle16x16", doweight)
    assert_close(out, ref, RTOL, ATOL, f"int4 stage 1 {shape} {in_dtype}")
    eps = 2.0 ** -8 if out_dtype == "bf16" else 2.0 ** -11
    assert_close(out, ref, 2 * eps, 1e-3, f"int4 stage 1 tight {shape} {in_dtype}")


@pytest.mark.parametrize("shape,in_dtype,out_dtype,mode", [
    ("S", "int4", "f32", "atomic"), ("S", "int4_bf16", "f32", "atomic"), ("M", "int4", "bf16", "reduce"),
    ("M", "int4_bf16", "f16", "rows"), ("T128", "int4", "f32", "atomic"), ("T128", "int4_bf16", "bf16", "reduce"),
])
def test_pertoken_stage2_packed_int4_weights(shape, in_dtype, out_dtype, mode):
    out, ref, pair_peak = run_stage2(shape, in_dtype, out_dtype, "tcgen05", "preshuffle16x16", mode)
    step = 0.0 if out_dtype == "f32" or mode == "rows" else 2.0 ** (-7 if out_dtype == "bf16" else -10) * pair_peak
    assert_close(out, ref, RTOL, ATOL + step, f"int4 stage 2 {shape} {in_dtype} {mode}")
    if out_dtype == "f32":
        assert_close(out, ref, 1e-4, 1e-5 * pair_peak, f"int4 stage 2 tight {shape} {in_dtype}")


@pytest.mark.parametrize("shape,scale_is_bf16", [("S", False), ("M", True), ("T128", False)])
def test_pertoken_groupwise_int4_weights(shape, scale_is_bf16):
    """W4A16 with one weight scale per 32-wide K group (group_size=32; the reference's layouts: f32 [E, K/32, N],
    or bf16 [E, K/64, N, 2] from tests/utils.py:99-129): both stages against the oracle's group-wise dequantisation.
    The scales are folded into the bf16 weights while unpacking, hence one bf16 rounding (2^-9 relative) per
    weight on top of the oracle's fp32 dequantisation: the bar gets one bf16 step of the largest output on
    top of atol (the reference's own bar for its int4 kernels is rtol = atol = 0.5,
    tests/kernels/test_moe_gemm.py:730-731)."""
    T, H, I, E, k, tile_m = SHAPES[shape]
    xq, _, w1q, _, w2q, _, ids, tw = inputs(shape, "int4_bf16")
    g1, g2 = hp.group_scales(E, H, I, 4242)
    if scale_is_bf16:
        g1, g2 = g1.to(torch.bfloat16), g2.to(torch.bfloat16)

    def prepared(gs):          # the layout the launcher takes
        if gs.dtype == torch.bfloat16:
            e, g, n = gs.shape
            gs = gs.view(e, g // 2, 2, n).permute(0, 1, 3, 2)
        return gs.contiguous().cuda().view(-1)
    s_ids, s_w, s_e, nv, nblk = sort(ids, tw, E, tile_m)
    common = dict(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=128, tile_k=128,
                  in_dtype="int4_bf16", group_size=32, scale_is_bf16=scale_is_bf16)
    none = scale_arg(None)
    out1 = torch.zeros((T * k, I), dtype=torch.bfloat16, device="cuda")
    pt.compile_moe_gemm1(doweight_stage1=False, out_dtype="bf16", **common)(
        out1.view(-1), xq.cuda(), dev_weight(w1q, "preshuffle16x16", "int4_bf16"), none, prepared(g1),
        s_ids, s_e, s_w, nv, T, I, H, nblk)
    ref1 = orc.pertoken_stage1(xq, None, w1q, None, ids, tw, I, False, group_size=32, scale_w1_groups=g1.float())
    assert_close(out1.cpu().view(T, k, I), ref1, RTOL, ATOL + 2.0 ** -8 * float(ref1.abs().max()),
                 f"group-wise stage 1 {shape}")
    a2 = ref1.to(torch.bfloat16)
    out2 = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    pt.compile_moe_gemm2(doweight_stage2=True, out_dtype="f32", **common)(
        out2.view(-1), a2.cuda().view(-1, I), dev_weight(w2q, "preshuffle16x16", "int4_bf16"), none, prepared(g2),
        s_ids, s_e, s_w, nv, T, H, I, nblk)
    torch.cuda.synchronize()
    ref2 = orc.pertoken_stage2(a2, None, w2q, None, ids, tw, H, True, group_size=32, scale_w2_groups=g2.float())
    assert_close(out2.cpu(), ref2, RTOL, ATOL + 2.0 ** -8 * float(ref2.abs().max()), f"group-wise stage 2 {shape}")


def test_int4_unpack_matches_reference_packing():
    """flymoe_unpack_int4_weight inverts the reference's shuffle + packer (bytes stored in the fixture)."""
    from flydsl_b200.kernels.moe_blockscale_2stage import unpack_int4_weight
    g = hp.load("moe_pertoken.npz")
    seen = 0
    for i in range(int(g["n"][0])):
        in_dtype = str(g[f"p{i}_dtype"][0])
        if in_dtype not in ("int4", "int4_bf16"):
            continue
        seen += 1
        T, H, I, E, k, _, seed = (int(v) for v in g[f"p{i}_cfg"])
        _, _, w1q, _, w2q, _, _, _ = hp.pertoken_inputs(in_dtype, T, H, I, E, k, seed, orc.quant_rows)
        for wq, key, rows, cols in ((w1q, "w1_packed", E * 2 * I, H), (w2q, "w2_packed", E * H, I)):
            packed = torch.from_numpy(g[f"p{i}_{key}"]).cuda()
            as_i8 = unpack_int4_weight(packed, rows, cols, torch.int8)
            assert torch.equal(as_i8.cpu().view(rows, cols), wq.view(rows, cols))
            as_bf = unpack_int4_weight(packed, rows, cols, torch.bfloat16)
            assert torch.equal(as_bf.cpu().float().view(rows, cols), wq.view(rows, cols).float())
    assert seen == 3          # W4A8, W4A16 and the group-wise W4A16 case


def test_pertoken_16bit_golden_fixture():
    """The two 16-bit cases of the fixture generated from the reference's own torch_moe_gemm1/2."""
    g = hp.load("moe_pertoken.npz")
    seen = 0
    for i in range(int(g["n"][0])):
        in_dtype = str(g[f"p{i}_dtype"][0])
        if in_dtype not in HALF:
            continue
        seen += 1
        T, H, I, E, k, doweight1, seed = (int(v) for v in g[f"p{i}_cfg"])
        xq, _, w1q, _, w2q, _, ids, tw = hp.pertoken_inputs(in_dtype, T, H, I, E, k, seed, orc.quant_rows)
        s_ids, s_w, s_e, nv, nblk = sort(ids, tw, E, 16)
        common = dict(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=16, tile_n=128, tile_k=128, in_dtype=in_dtype)
        none = scale_arg(None)
        out1 = torch.zeros((T * k, I), dtype=HALF[in_dtype], device="cuda")
        pt.compile_moe_gemm1(doweight_stage1=bool(doweight1), out_dtype="f16" if in_dtype == "fp16" else "bf16", **common)(
            out1.view(-1), xq.cuda(), dev_weight(w1q, "preshuffle16x16"), none, none, s_ids, s_e, s_w, nv, T, I, H, nblk)
        ref1 = torch.from_numpy(g[f"p{i}_out1"])
        assert_close(out1.cpu().view(T, k, I), ref1, RTOL, ATOL, f"fixture case {i} stage 1")
        a2 = torch.from_numpy(g[f"p{i}_a2q"]).view(HALF[in_dtype]).cuda()          # the reference's own stage-2 input
        out2 = torch.zeros((T, H), dtype=torch.float32, device="cuda")
        pt.compile_moe_gemm2(doweight_stage2=not bool(doweight1), out_dtype="f32", **common)(
            out2.view(-1), a2.view(-1, I), dev_weight(w2q, "preshuffle16x16"), none, none, s_ids, s_e, s_w, nv, T, H, I, nblk)
        torch.cuda.synchronize()
        assert_close(out2.cpu(), torch.from_numpy(g[f"p{i}_out2"]), RTOL, ATOL, f"fixture case {i} stage 2")
    assert seen == 2


@pytest.mark.parametrize("in_dtype", ["fp8", "int8"])
def test_pertoken_large_reference_shape(in_dtype):
    """The reference's aiter-style L shape (333 tokens, 4096 x 2048, 17 experts, top-9), both stages."""
    out1, ref1 = run_stage1("L", in_dtype, "bf16", "tcgen05", "plain", False)
    assert_close(out1, ref1, RTOL, ATOL, f"per-token stage 1 L {in_dtype}")
    out2, ref2, pair_peak = run_stage2("L", in_dtype, "f32", "tcgen05", "plain", "atomic")
    assert_close(out2, ref2, RTOL, ATOL, f"per-token stage 2 L {in_dtype}")
    out2r, _, _ = run_stage2("L", in_dtype, "bf16", "tcgen05", "plain", "reduce")
    assert_close(out2r, ref2, RTOL, ATOL + 2.0 ** -7 * pair_peak, f"per-token stage 2 L reduce {in_dtype}")



@pytest.mark.parametrize("shape,in_dtype,k_batch", [("S", "fp8", 2), ("M", "int8", 2), ("M", "fp16", 4), ("T128", "fp8", 2),
                                                    ("S", "int8smooth", 2)])
def test_pertoken_stage1_split_k_output_contract(shape, in_dtype, k_batch):
    """k_batch > 1: the launcher adds the scaled gate|up sums (no activation, no routing weight, even with
    doweight_stage1) to a zeroed fp32 [tokens*topk, 2*inter] buffer; the caller finishes silu(gate)*up
    (tests/kernels/test_moe_gemm.py:582-587, :708-713 of the reference).  Launching twice doubles the sums."""
    T, H, I, E, k, tile_m = SHAPES[shape]
    xq, sx, w1q, sw1, _, _, ids, tw = inputs(shape, in_dtype)
    s_ids, s_w, s_e, nv, nblk = sort(ids, tw, E, tile_m)
    exe = pt.compile_moe_gemm1(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=128, tile_k=64,
                               doweight_stage1=True, in_dtype=in_dtype, out_dtype="f16", k_batch=k_batch)
    if in_dtype == "int8smooth":
        x_arg, sx_arg = xq.permute(1, 0, 2).contiguous().cuda().view(-1, H), scale_arg(sx.permute(1, 0, 2).contiguous())
    else:
        x_arg, sx_arg = xq.cuda().view(-1, H), scale_arg(sx)
    out = torch.zeros((T * k + 4, 2 * I), dtype=torch.float32, device="cuda")
    args = (out.view(-1)[: T * k * 2 * I], x_arg, dev_weight(w1q, "preshuffle16x16", in_dtype), sx_arg, scale_arg(sw1),
            s_ids, s_e, s_w, nv, T, I, H, nblk)
    exe(*args)
    torch.cuda.synchronize()
    raw = out[: T * k].cpu().view(T, k, 2 * I)
    assert float(out[T * k:].abs().sum()) == 0.0, "wrote past the output rows"
    ref_raw = orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I, raw_sums=True)
    peak = float(ref_raw.abs().max())
    assert_close(raw, ref_raw, 1e-4, 1e-5 * peak + (2e-3 * peak if in_dtype == "fp16" else 0.0), f"raw sums {shape} {in_dtype}")
    done = torch.nn.functional.silu(raw[..., :I]) * raw[..., I:]
    assert_close(done, orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I, False), RTOL, ATOL, f"finished {shape} {in_dtype}")
    exe(*args)                                  # the contract is accumulation: a second launch doubles every sum
    torch.cuda.synchronize()
    assert_close(out[: T * k].cpu().view(T, k, 2 * I), 2 * ref_raw, 1e-4, 2e-5 * peak + (4e-3 * peak if in_dtype == "fp16" else 0.0),
                 f"accumulated {shape} {in_dtype}")


@pytest.mark.parametrize("in_dtype", ["fp8", "bf16", "int4"])
def test_pertoken_empty_batch_is_a_no_op(in_dtype):
    """Zero tokens: both launchers return without touching their outputs (the reference's kernels exit early on
    an empty sorted list, kernels/moe_gemm_2stage.py:441-460)."""
    H, I, E, k, tile_m = 256, 128, 4, 2, 16
    _, _, w1q, sw1, w2q, sw2, _, _ = hp.pertoken_inputs(in_dtype, 8, H, I, E, k, 5, orc.quant_rows)
    d = "cuda"
    s_ids = torch.full((E * tile_m,), (k << 24), dtype=torch.int32, device=d)
    s_w = torch.zeros(E * tile_m, dtype=torch.float32, device=d)
    s_e = torch.full((E,), -1, dtype=torch.int32, device=d)
    nv = torch.zeros(2, dtype=torch.int32, device=d)
    x_dt = {"fp8": hp.FP8, "bf16": torch.bfloat16, "int4": torch.int8}[in_dtype]
    x = torch.empty((0, H), dtype=x_dt, device=d)
    sx = torch.empty(0, dtype=torch.float32, device=d)
    common = dict(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=128, tile_k=128, in_dtype=in_dtype)
    out1 = torch.full((4, I), 3.0, dtype=torch.bfloat16, device=d)
    pt.compile_moe_gemm1(doweight_stage1=False, out_dtype="bf16", **common)(
        out1.view(-1)[:0], x, dev_weight(w1q, "preshuffle16x16", in_dtype), sx, scale_arg(sw1), s_ids, s_e, s_w, nv,
        0, I, H, E)
    out2 = torch.full((4, H), 3.0, dtype=torch.float32, device=d)
    a2 = torch.empty((0, I), dtype=x_dt, device=d)
    pt.compile_moe_gemm2(doweight_stage2=True, out_dtype="f32", **common)(
        out2.view(-1)[:0], a2, dev_weight(w2q, "preshuffle16x16", in_dtype), sx, scale_arg(sw2), s_ids, s_e, s_w, nv,
        0, H, I, E)
    torch.cuda.synchronize()
    assert bool((out1 == 3.0).all()) and bool((out2 == 3.0).all())
    assert _lib_status() == 0


def _lib_status():
    from flydsl_b200 import _lib
    return _lib.device_status()
