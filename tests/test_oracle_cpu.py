"""The CPU oracle against the golden fixtures produced by the reference's own functions."""
import numpy as np
import torch

from flydsl_b200 import workloads as wl
from oracle import moe_oracle as orc
from tests import helpers as hp


def test_pertoken_quant_and_shuffle_match_reference():
    g = hp.load("quant_shuffle.npz")
    x = torch.from_numpy(g["x"])
    q, s = orc.quant_act_1x128(x)
    assert np.array_equal(hp.u8(q), g["q"])
    assert np.array_equal(s.numpy(), g["scale"])
    # the workload generator's quantiser is the same function
    q2, s2 = wl.quant_act_1x128(x)
    assert np.array_equal(hp.u8(q2), g["q"]) and np.array_equal(s2.numpy(), g["scale"])
    w = hp.fp8_from_u8(g["w"])
    shuf = orc.shuffle_weight(w)
    assert np.array_equal(hp.u8(shuf), g["w_shuffled"])
    assert np.array_equal(hp.u8(orc.unshuffle_weight(shuf)), g["w"])
    # two-byte elements keep 8 of a row together (16 bytes), so the pattern differs from the one-byte one
    w16 = torch.from_numpy(g["w16"]).view(torch.bfloat16)
    shuf16 = orc.shuffle_weight(w16)
    assert np.array_equal(shuf16.view(torch.int16).numpy(), g["w16_shuffled"])
    assert torch.equal(orc.unshuffle_weight(shuf16).view(torch.int16), w16.view(torch.int16))


def test_sorting_matches_reference():
    g = hp.load("sorting.npz")
    for i in range(int(g["n"][0])):
        T, E, k, unit, masked = (int(v) for v in g[f"c{i}_cfg"])
        mask = g[f"c{i}_mask"] if masked else None
        a, b, c, d = orc.moe_sorting(g[f"c{i}_ids"], g[f"c{i}_w"], E, unit, mask)
        assert np.array_equal(a, g[f"c{i}_sorted_ids"]), (T, E, k, unit)
        assert np.array_equal(b, g[f"c{i}_sorted_w"])
        assert np.array_equal(c, g[f"c{i}_sorted_e"])
        assert np.array_equal(d, g[f"c{i}_nvalid"])
        ids, w, m = hp.gen_sort_inputs(T, E, k, bool(masked))
        assert np.array_equal(ids.numpy(), g[f"c{i}_ids"]) and np.array_equal(w.numpy(), g[f"c{i}_w"])


def test_gating_matches_reference_expression():
    g = hp.load("gating.npz")
    for i in range(int(g["n"][0])):
        T, E, k, renorm = (int(v) for v in g[f"g{i}_cfg"])
        logits = torch.from_numpy(g[f"g{i}_logits_f32"])
        w, idx, tei = orc.topk_gating_softmax(logits, k, bool(renorm))
        rows = torch.from_numpy(g[f"g{i}_distinct"])
        assert rows.sum() > 0
        assert torch.equal(idx[rows], torch.from_numpy(g[f"g{i}_idx"])[rows])
        assert torch.allclose(w[rows], torch.from_numpy(g[f"g{i}_w"])[rows], atol=1e-7, rtol=1e-6)
        exp_tei = torch.arange(k, dtype=torch.int32).view(1, k) * T + torch.arange(T, dtype=torch.int32).view(T, 1)
        assert torch.equal(tei, exp_tei)
        assert orc.gating_prob_rule_differs(logits, k) == 0


def _check_moe(fname, cfg, stored_inputs):
    g = hp.load(fname)
    if stored_inputs:
        logits = torch.from_numpy(g["logits"])
        xq, xs = hp.fp8_from_u8(g["xq"]), torch.from_numpy(g["x_scale"])
        w1q, w1s = hp.fp8_from_u8(g["w1q"]), torch.from_numpy(g["w1_scale"])
        w2q, w2s = hp.fp8_from_u8(g["w2q"]), torch.from_numpy(g["w2_scale"])
    logits_g = wl.make_logits(cfg)
    _x, xq_g, xs_g = wl.make_activations(cfg)
    w1q_g, w1s_g, w2q_g, w2s_g = wl.make_weights(cfg)
    digest = hp.sha(logits_g.numpy(), hp.u8(xq_g), xs_g.numpy(), hp.u8(w1q_g), w1s_g.numpy(), hp.u8(w2q_g),
                    w2s_g.numpy())
    assert digest == str(g["input_sha"][0]), "seeded generator no longer reproduces the fixture inputs"
    if not stored_inputs:
        logits, xq, xs, w1q, w1s, w2q, w2s = logits_g, xq_g, xs_g, w1q_g, w1s_g, w2q_g, w2s_g
    else:
        assert torch.equal(logits, logits_g) and np.array_equal(hp.u8(xq), hp.u8(xq_g))
    res = orc.moe_layer(logits, xq, xs, w1q, w1s, w2q, w2s, cfg.topk, via_f16=False)
    assert np.array_equal(res["topk_ids"].numpy(), g["topk_ids"])
    assert np.allclose(res["topk_weights"].numpy(), g["topk_weights"], atol=1e-7, rtol=1e-6)
    out1_ref = torch.from_numpy(g["out1"])
    assert torch.allclose(res["out1"], out1_ref, rtol=2e-5, atol=1e-6)
    # requantised intermediate: identical scales up to fp32 round-off of out1, codes within 1 step
    d = orc.e4m3_ulp_distance(res["a2q"], hp.fp8_from_u8(g["a2q_from_f32"]))
    assert int(d.max()) <= 1 and float((d == 0).float().mean()) > 0.999
    assert np.allclose(res["a2_scale"].numpy(), g["a2_scale_from_f32"], rtol=1e-5)
    out2_ref = torch.from_numpy(g["out2_from_f32"])
    scale = out2_ref.abs().max().item()
    assert torch.allclose(res["out_f32"], out2_ref, rtol=1e-3, atol=2e-3 * scale)
    # the reference's own pipeline (intermediate rounded to f16 first) and its single-shot fused oracle
    res16 = orc.moe_layer(logits, xq, xs, w1q, w1s, w2q, w2s, cfg.topk, via_f16=True)
    d16 = orc.e4m3_ulp_distance(res16["a2q"], hp.fp8_from_u8(g["a2q_via_f16"]))
    assert int(d16.max()) <= 1 and float((d16 == 0).float().mean()) > 0.999
    out2_16 = torch.from_numpy(g["out2_via_f16"])
    assert torch.allclose(res16["out_f32"], out2_16, rtol=1e-3, atol=2e-3 * scale)
    fused = torch.from_numpy(g["fused_bf16_bits"]).view(torch.bfloat16).float()
    assert torch.allclose(res["out"].float(), fused, rtol=2e-2, atol=2e-2 * max(scale, 1.0))


def test_moe_mini_matches_reference():
    _check_moe("moe_mini.npz", wl.MoEConfig("mini", 16, 256, 128, 4, 2, 7), True)


def test_moe_c1_matches_reference():
    _check_moe("moe_c1.npz", wl.CONFIGS["c1"], False)


def test_dense_blockscale_gemm_matches_reference():
    """oracle.blockscale_gemm against run_torch_blockscale of the reference's own test
    (tests/kernels/test_blockscale_preshuffle_gemm.py:101-125), on that test's input recipe."""
    g = hp.load("blockscale_gemm.npz")
    for i in range(int(g["n_cases"][0])):
        c = orc.blockscale_gemm(hp.fp8_from_u8(g[f"x{i}"]), torch.from_numpy(g[f"x_scale{i}"]),
                                hp.fp8_from_u8(g[f"w{i}"]), torch.from_numpy(g[f"w_scale{i}"]))
        want = torch.from_numpy(g[f"c{i}"])
        assert c.shape == want.shape
        assert torch.allclose(c, want, rtol=1e-5, atol=1e-6), float((c - want).abs().max())


def test_ulp_distance():
    a = torch.tensor([0.0, 1.0, -1.0, 448.0]).to(hp.FP8)
    b = torch.tensor([0.0, 1.125, -0.9375, 416.0]).to(hp.FP8)
    assert orc.e4m3_ulp_distance(a, b).tolist() == [0, 1, 1, 1]


def test_pertoken_family_matches_reference_functions():
    """oracle.pertoken_stage1/2 and quant_rows against torch_moe_gemm1/2 and pertoken_quant of the
    reference (fixture moe_pertoken.npz): inputs regenerated from the seed must hash to the stored
    value (which pins the quantiser), outputs must agree to fp32 round-off."""
    g = hp.load("moe_pertoken.npz")
    for i in range(int(g["n"][0])):
        T, H, I, E, k, doweight1, seed = (int(v) for v in g[f"p{i}_cfg"])
        in_dtype = str(g[f"p{i}_dtype"][0])
        qd = hp.FP8 if in_dtype == "fp8" else torch.int8
        half = {"fp16": torch.float16, "bf16": torch.bfloat16}.get(in_dtype)
        grouped = bool(int(g[f"p{i}_grouped"][0]))
        xq, sx, w1q, sw1, w2q, sw2, ids, tw = hp.pertoken_inputs(in_dtype, T, H, I, E, k, seed, orc.quant_rows)
        gkw1, gkw2 = {}, {}
        if grouped:
            g1, g2 = hp.group_scales(E, H, I, int(g[f"p{i}_group_seed"][0]))
            got_sha = hp.sha(hp.u8(xq), hp.u8(w1q), hp.u8(w2q), g1.numpy(), g2.numpy(), ids.numpy(), tw.numpy())
            half, sw1, sw2 = torch.bfloat16, None, None
            gkw1, gkw2 = dict(group_size=32, scale_w1_groups=g1), dict(group_size=32, scale_w2_groups=g2)
        elif half is not None:
            got_sha = hp.sha(hp.u8(xq), hp.u8(w1q), hp.u8(w2q), ids.numpy(), tw.numpy())
        elif in_dtype == "int4_bf16":
            got_sha = hp.sha(hp.u8(xq), hp.u8(w1q), sw1.numpy(), hp.u8(w2q), sw2.numpy(), ids.numpy(), tw.numpy())
            half = torch.bfloat16                  # its stage-2 input is the bf16 cast of stage 1, too
        else:
            got_sha = hp.sha(hp.u8(xq), sx.numpy(), hp.u8(w1q), sw1.numpy(), hp.u8(w2q), sw2.numpy(), ids.numpy(), tw.numpy())
        assert got_sha == str(g[f"p{i}_input_sha"][0]), f"case {i}: regenerated inputs differ from the fixture's"
        if i == 0:
            assert np.array_equal(hp.u8(xq), g["p0_xq"]) and np.array_equal(sw1.numpy(), g["p0_sw1"])
        o1 = orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I, bool(doweight1), **gkw1)
        ref1 = torch.from_numpy(g[f"p{i}_out1"])
        assert torch.allclose(o1, ref1, rtol=1e-5, atol=1e-5 * float(ref1.abs().max())), f"case {i} stage 1"
        if half is not None:
            a2q, sa2 = ref1.to(half), None
            assert np.array_equal(hp.u8(a2q), g[f"p{i}_a2q"])
        else:
            a2q, sa2 = orc.quant_rows(ref1, qd)
            assert np.array_equal(hp.u8(a2q), g[f"p{i}_a2q"]) and np.array_equal(sa2.numpy(), g[f"p{i}_sa2"])
        o2 = orc.pertoken_stage2(a2q, sa2, w2q, sw2, ids, tw, H, not bool(doweight1), **gkw2)
        ref2 = torch.from_numpy(g[f"p{i}_out2"])
        assert torch.allclose(o2, ref2, rtol=1e-5, atol=1e-5 * float(ref2.abs().max())), f"case {i} stage 2"
        if in_dtype in ("int4", "int4_bf16"):      # the oracle's packer against the reference's shuffle + packer
            assert int(w1q.abs().max()) <= 7
            assert np.array_equal(hp.u8(orc.pack_int4_preshuffled(w1q)), g[f"p{i}_w1_packed"])
            assert np.array_equal(hp.u8(orc.pack_int4_preshuffled(w2q)), g[f"p{i}_w2_packed"])


def test_pertoken_raw_sums_finish_to_stage1():
    """The split-K output contract: silu(gate) * up of the raw sums is stage 1 (what the reference's test does
    on the host, tests/kernels/test_moe_gemm.py:708-713)."""
    T, H, I, E, k = 24, 256, 128, 4, 2
    xq, sx, w1q, sw1, _, _, ids, tw = hp.pertoken_inputs("fp8", T, H, I, E, k, 31, orc.quant_rows)
    raw = orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I, raw_sums=True)
    assert raw.shape == (T, k, 2 * I)
    done = torch.nn.functional.silu(raw[..., :I]) * raw[..., I:]
    assert torch.allclose(done, orc.pertoken_stage1(xq, sx, w1q, sw1, ids, tw, I), rtol=1e-6, atol=1e-6)
