"""Generate the golden fixtures in this directory from the reference project's own code.

Run once, in a container that has the reference checkout; its location is given by the
``FLYMOE_REFERENCE_DIR`` environment variable:

    FLYMOE_REFERENCE_DIR=<path to the FlyDSL checkout> python tests/golden/make_golden.py

The reference's torch oracles live in test files that import the (AMD-only)
compiler at module level, so they cannot be imported; this script lifts the pure-torch
functions out of those files by AST at generation time, executes them on seeded
inputs and stores inputs/outputs as ``.npz``.  No reference source is copied into
this repository; the fixtures hold only numbers.  The test-suite then checks the CPU
oracle (``oracle/moe_oracle.py``) against these files, which pins the oracle to the
reference's behaviour.

Lifted functions (reference paths):
  tests/kernels/test_moe_blockscale.py: _expand_blockscale, torch_stage1_blockscale_ref,
      torch_stage2_blockscale_ref, torch_moe_blockscale_ref
  tests/kernels/test_moe_sorting.py:    moe_sorting_reference
  tests/utils.py (imported directly):   pertoken_quant, shuffle_weight
  tests/kernels/test_ref.py:            torch_moe_gemm1, torch_moe_gemm2 and their helpers (the text
      ``device="cuda"`` becomes ``device="cpu"`` and the ``is_cuda`` assertion is dropped while lifting,
      since the fixtures are generated without a GPU; nothing else changes)
Gating has no reference function; the fixture stores the result of the reference test's
inline expression (softmax -> topk -> renormalise, test_topk_gating_softmax.py:84-89).
"""

from __future__ import annotations

import ast
import hashlib
import importlib.util
import math
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = Path(os.environ["FLYMOE_REFERENCE_DIR"]) if "FLYMOE_REFERENCE_DIR" in os.environ else None
sys.path.insert(0, str(REPO))

from flydsl_b200 import workloads as wl  # noqa: E402

FP8 = torch.float8_e4m3fn


def lift(path: Path, names: list[str], extra_globals: dict, replace: dict | None = None) -> dict:
    text = path.read_text()
    for old, new in (replace or {}).items():
        if old not in text:
            raise RuntimeError(f"{path}: expected text not found: {old!r}")
        text = text.replace(old, new)
    tree = ast.parse(text)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in wanted}
    if missing:
        raise RuntimeError(f"{path}: functions not found: {sorted(missing)}")
    mod = ast.Module(body=wanted, type_ignores=[])
    ns = dict(extra_globals)
    exec(compile(mod, str(path), "exec"), ns)
    return {n: ns[n] for n in names}


def import_file(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main() -> None:
    if REF is None or not REF.exists():
        raise SystemExit("set FLYMOE_REFERENCE_DIR to the reference checkout")
    only = set(sys.argv[1:])          # optional: names of the fixtures to (re)write, e.g. moe_pertoken.npz

    def save(name: str, **arrays) -> None:
        if not only or name in only:
            np.savez_compressed(HERE / name, **arrays)
    utils = import_file(REF / "tests" / "utils.py", "ref_tests_utils")
    bs = lift(REF / "tests" / "kernels" / "test_moe_blockscale.py",
              ["_expand_blockscale", "torch_stage1_blockscale_ref", "torch_stage2_blockscale_ref",
               "torch_moe_blockscale_ref"], {"torch": torch, "F": F, "math": math})
    srt = lift(REF / "tests" / "kernels" / "test_moe_sorting.py", ["moe_sorting_reference"],
               {"torch": torch, "UNIT_SIZE": 32})
    pertoken_quant, shuffle_weight = utils.pertoken_quant, utils.shuffle_weight

    # ------------------------------------------------------------------ quantiser + shuffle
    g = torch.Generator().manual_seed(11)
    xs = torch.randn((24, 384), generator=g) * 3.0
    xs[3, :128] = 0.0                       # an all-zero group -> scale 1
    xs[5, 130] = 1e-9
    q, s = pertoken_quant(xs.view(24, 3, 128), quant_dtype=FP8)
    wq_small = (torch.randn((2, 64, 128), generator=g) * 50).to(FP8)
    shuf = shuffle_weight(wq_small.clone(), layout=(16, 16))
    w16 = torch.randn((2, 32, 64), generator=g).to(torch.bfloat16)          # two-byte elements: 8 per 16-byte chunk
    shuf16 = shuffle_weight(w16.clone(), layout=(16, 16))
    save("quant_shuffle.npz", x=xs.numpy(), q=u8(q.view(24, 384)),
                        scale=s.view(24, 3).numpy(), w=u8(wq_small), w_shuffled=u8(shuf),
                        w16=bf16_bits(w16), w16_shuffled=bf16_bits(shuf16))

    # ------------------------------------------------------------------ sorting
    sort_cases = [(1, 8, 2, 32, False), (7, 32, 5, 32, False), (31, 64, 6, 16, False), (64, 256, 8, 32, False),
                  (16, 257, 9, 32, False), (128, 256, 8, 128, False), (300, 32, 5, 64, True),
                  (1500, 256, 8, 128, False), (1500, 64, 6, 32, True)]
    out = {}
    for i, (T, E, k, unit, masked) in enumerate(sort_cases):
        gg = torch.Generator().manual_seed(42 + T * 1000 + E * 10 + k)
        ids = torch.stack([torch.randperm(E, generator=gg)[:k] for _ in range(T)]).to(torch.int32)
        w = torch.rand((T, k), generator=gg, dtype=torch.float32)
        mask = None
        if masked:
            mask = (torch.rand(E, generator=gg) < 0.5).to(torch.int32)
            mask[0] = 1
        a, b, c, d = srt["moe_sorting_reference"](ids, w, E, unit_size=unit, expert_mask=mask)
        out[f"c{i}_cfg"] = np.array([T, E, k, unit, int(masked)], dtype=np.int32)
        out[f"c{i}_ids"], out[f"c{i}_w"] = ids.numpy(), w.numpy()
        if mask is not None:
            out[f"c{i}_mask"] = mask.numpy()
        out[f"c{i}_sorted_ids"], out[f"c{i}_sorted_w"] = a.numpy(), b.numpy()
        out[f"c{i}_sorted_e"], out[f"c{i}_nvalid"] = c.numpy(), d.numpy()
    out["n"] = np.array([len(sort_cases)], dtype=np.int32)
    save("sorting.npz", **out)

    # ------------------------------------------------------------------ gating
    gate_cases = [(64, 8, 2, "f32", True), (64, 256, 8, "f32", True), (33, 128, 6, "bf16", True),
                  (16, 64, 2, "f16", False)]
    out = {}
    for i, (T, E, k, dt, renorm) in enumerate(gate_cases):
        gg = torch.Generator().manual_seed(1234 + i)
        td = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dt]
        logits = (torch.rand((T, E), generator=gg) * 4.0 - 2.0).to(td)
        lf = logits.to(torch.float32)
        # rows whose k+1 largest probabilities are strictly decreasing leave torch.topk no tie freedom
        probs = torch.softmax(lf, dim=1)
        rw, ri = torch.topk(probs, k, dim=1)
        if renorm:
            rw = rw / rw.sum(dim=1, keepdim=True).clamp(min=1e-20)
        top = torch.sort(probs, dim=1, descending=True).values[:, :min(k + 1, E)]
        distinct = (top[:, :-1] > top[:, 1:]).all(dim=1)
        out[f"g{i}_cfg"] = np.array([T, E, k, int(renorm)], dtype=np.int32)
        out[f"g{i}_dtype"] = np.array([dt])
        out[f"g{i}_logits_f32"] = lf.numpy()
        out[f"g{i}_w"], out[f"g{i}_idx"] = rw.numpy(), ri.to(torch.int32).numpy()
        out[f"g{i}_distinct"] = distinct.numpy()
    out["n"] = np.array([len(gate_cases)], dtype=np.int32)
    save("gating.npz", **out)

    # ------------------------------------------------------------------ GEMM stages
    def run_moe(cfg: wl.MoEConfig, store_inputs: bool, fname: str):
        logits = wl.make_logits(cfg)
        _x, xq, xs_ = wl.make_activations(cfg)
        w1q, w1s, w2q, w2s = wl.make_weights(cfg)
        # routing exactly as the reference test does it for given scores: topk then softmax is its
        # own choice; here the routing under test is softmax -> topk -> renormalise
        probs = torch.softmax(logits, dim=1)
        tw, ti = torch.topk(probs, cfg.topk, dim=1)
        tw = (tw / tw.sum(dim=1, keepdim=True)).to(torch.float32)
        I, H = cfg.inter_dim, cfg.model_dim
        out1 = bs["torch_stage1_blockscale_ref"](xq, w1q, ti, xs_, w1s.view(cfg.experts, -1), (128, 128), I)
        out1_f16 = out1.to(torch.float16)
        a2q_f16, a2s_f16 = pertoken_quant(out1_f16.float().view(-1, I // 128, 128), quant_dtype=FP8)
        a2q_f32, a2s_f32 = pertoken_quant(out1.view(-1, I // 128, 128), quant_dtype=FP8)
        a2q_f16, a2s_f16 = a2q_f16.view(-1, I), a2s_f16.squeeze(-1)
        a2q_f32, a2s_f32 = a2q_f32.view(-1, I), a2s_f32.squeeze(-1)
        out2_f16 = bs["torch_stage2_blockscale_ref"](a2q_f16, w2q, ti, tw, a2s_f16, w2s.view(cfg.experts, -1),
                                                     (128, 128), cfg.tokens, H, I, cfg.topk)
        out2_f32 = bs["torch_stage2_blockscale_ref"](a2q_f32, w2q, ti, tw, a2s_f32, w2s.view(cfg.experts, -1),
                                                     (128, 128), cfg.tokens, H, I, cfg.topk)
        fused = bs["torch_moe_blockscale_ref"](xq, w1q, w2q, tw, ti, torch.bfloat16, (128, 128), xs_,
                                               w1s.view(cfg.experts, -1), w2s.view(cfg.experts, -1))
        rec = {
            "cfg": np.array([cfg.tokens, cfg.model_dim, cfg.inter_dim, cfg.experts, cfg.topk, cfg.seed], dtype=np.int32),
            "input_sha": np.array([sha(logits.numpy(), u8(xq), xs_.numpy(), u8(w1q), w1s.numpy(), u8(w2q), w2s.numpy())]),
            "topk_ids": ti.to(torch.int32).numpy(), "topk_weights": tw.numpy(),
            "out1": out1.numpy(),
            "a2q_via_f16": u8(a2q_f16), "a2_scale_via_f16": a2s_f16.numpy(),
            "a2q_from_f32": u8(a2q_f32), "a2_scale_from_f32": a2s_f32.numpy(),
            "out2_via_f16": out2_f16.numpy(), "out2_from_f32": out2_f32.numpy(),
            "fused_bf16_bits": bf16_bits(fused),
        }
        if store_inputs:
            rec.update({"logits": logits.numpy(), "xq": u8(xq), "x_scale": xs_.numpy(), "w1q": u8(w1q),
                        "w1_scale": w1s.numpy(), "w2q": u8(w2q), "w2_scale": w2s.numpy()})
        save(fname, **rec)

    run_moe(wl.MoEConfig("mini", 16, 256, 128, 4, 2, 7), True, "moe_mini.npz")
    run_moe(wl.CONFIGS["c1"], False, "moe_c1.npz")

    # ------------------------------------------------------------------ dense block-scaled GEMM
    dense = lift(REF / "tests" / "kernels" / "test_blockscale_preshuffle_gemm.py", ["run_torch_blockscale"],
                 {"torch": torch, "F": F, "BLOCK_SHAPE": (128, 128)})["run_torch_blockscale"]
    out = {}
    for i, (M, N, K) in enumerate([(5, 256, 384), (33, 384, 256), (1, 128, 128)]):
        g = torch.Generator().manual_seed(40 + i)
        # the reference test's own input recipe (test_blockscale_preshuffle_gemm.py:208-212)
        x = (torch.rand((M, K), generator=g, dtype=torch.float32) / 10).to(torch.float16).to(FP8)
        w = (torch.rand((N, K), generator=g, dtype=torch.float32) / 10).to(torch.float16).to(FP8)
        x_scale = torch.rand((M, K // 128), generator=g, dtype=torch.float32)
        w_scale = torch.rand((N // 128, K // 128), generator=g, dtype=torch.float32)
        c = dense(x, w, x_scale, w_scale, dtype=torch.float32)
        out.update({f"x{i}": u8(x), f"w{i}": u8(w), f"x_scale{i}": x_scale.numpy(), f"w_scale{i}": w_scale.numpy(),
                    f"c{i}": c.numpy()})
    out["n_cases"] = np.array([3], dtype=np.int32)
    save("blockscale_gemm.npz", **out)
    # ------------------------------------------------------------------ per-token-scale MoE family
    pt = lift(REF / "tests" / "kernels" / "test_ref.py",
              ["_detect_scale_kind", "_logical_k", "_dequant", "torch_moe_gemm1", "torch_moe_gemm2"],
              {"torch": torch, "F": F, "_FP4_DTYPES": (torch.uint8,)},
              replace={'device="cuda"': 'device="cpu"', "assert a2_q.is_cuda and w2_q.is_cuda": "pass"})
    from tests.helpers import pertoken_inputs
    out = {}
    cases = [("fp8", 64, 256, 128, 4, 2, False), ("int8", 64, 256, 128, 4, 2, False),
             ("int8smooth", 33, 256, 128, 4, 2, False), ("fp8", 129, 512, 256, 8, 2, True),
             ("bf16", 64, 256, 128, 4, 2, False), ("fp16", 40, 256, 128, 4, 2, True),
             ("int4", 48, 256, 128, 4, 2, False), ("int4_bf16", 48, 256, 128, 4, 2, False),
             ("int4_bf16_g32", 48, 256, 128, 4, 2, False)]
    half = {"fp16": torch.float16, "bf16": torch.bfloat16}
    pack4 = lift(REF / "tests" / "kernels" / "test_moe_gemm.py", ["_pack_shuffled_int8_to_packed_int4_no_perm"],
                 {"torch": torch})["_pack_shuffled_int8_to_packed_int4_no_perm"]
    for i, (in_dtype, T, H, I, E, k, doweight1) in enumerate(cases):
        qd = FP8 if in_dtype == "fp8" else torch.int8
        grouped = in_dtype.endswith("_g32")      # W4A16 with one weight scale per 32-wide K group instead of per row
        in_dtype = in_dtype[:-4] if grouped else in_dtype
        xq, sx, w1q, sw1, w2q, sw2, ti, tw = pertoken_inputs(in_dtype, T, H, I, E, k, 900 + i, pertoken_quant)
        if grouped:
            gg = torch.Generator().manual_seed(7000 + i)         # test_moe_gemm.py:512-514 of the reference
            g1 = torch.rand((E, H // 32, 2 * I), generator=gg) * 0.05 + 0.005
            g2 = torch.rand((E, I // 32, H), generator=gg) * 0.05 + 0.005
            o1 = pt["torch_moe_gemm1"](xq, w1q.view(E * 2 * I, H), None, None, ti, tw, I, doweight1, 32, g1)
            a2q, sa2 = o1.to(torch.bfloat16), None
            o2 = pt["torch_moe_gemm2"](a2q, w2q, None, None, ti, tw, H, not doweight1, 32, g2)
            digest = sha(u8(xq), u8(w1q), u8(w2q), g1.numpy(), g2.numpy(), ti.numpy(), tw.numpy())
            out[f"p{i}_group_seed"] = np.array([7000 + i], dtype=np.int32)
        elif in_dtype in half:          # no scales; the stage-2 input is stage 1's output in the same 16-bit type
            o1 = pt["torch_moe_gemm1"](xq, w1q.view(E * 2 * I, H), None, None, ti, tw, I, doweight1)
            a2q, sa2 = o1.to(half[in_dtype]), None
            o2 = pt["torch_moe_gemm2"](a2q, w2q, None, None, ti, tw, H, not doweight1)
            digest = sha(u8(xq), u8(w1q), u8(w2q), ti.numpy(), tw.numpy())
        elif in_dtype == "int4_bf16":  # W4A16: bf16 activations without scales, int8 weight values with row scales
            o1 = pt["torch_moe_gemm1"](xq, w1q.view(E * 2 * I, H), None, sw1.view(E * 2 * I, 1), ti, tw, I, doweight1)
            a2q, sa2 = o1.to(torch.bfloat16), None
            o2 = pt["torch_moe_gemm2"](a2q, w2q, None, sw2.view(E, H, 1), ti, tw, H, not doweight1)
            digest = sha(u8(xq), u8(w1q), sw1.numpy(), u8(w2q), sw2.numpy(), ti.numpy(), tw.numpy())
        else:
            o1 = pt["torch_moe_gemm1"](xq, w1q.view(E * 2 * I, H), sx, sw1.view(E * 2 * I, 1), ti, tw, I, doweight1)
            a2q, sa2 = pertoken_quant(o1, quant_dtype=qd)
            o2 = pt["torch_moe_gemm2"](a2q, w2q, sa2, sw2.view(E, H, 1), ti, tw, H, not doweight1)
            digest = sha(u8(xq), sx.numpy(), u8(w1q), sw1.numpy(), u8(w2q), sw2.numpy(), ti.numpy(), tw.numpy())
        out.update({f"p{i}_cfg": np.array([T, H, I, E, k, int(doweight1), 900 + i], dtype=np.int32),
                    f"p{i}_dtype": np.array([in_dtype]), f"p{i}_grouped": np.array([int(grouped)], dtype=np.int32),
                    f"p{i}_input_sha": np.array([digest]),
                    f"p{i}_out1": o1.numpy(), f"p{i}_a2q": u8(a2q), f"p{i}_out2": o2.numpy()})
        if sa2 is not None:
            out[f"p{i}_sa2"] = sa2.numpy()
        if in_dtype in ("int4", "int4_bf16"):   # the bytes the kernels receive: the reference's shuffle, then its packer
            out[f"p{i}_w1_packed"] = u8(pack4(shuffle_weight(w1q.clone(), layout=(16, 16)).view(E * 2 * I, H)))
            out[f"p{i}_w2_packed"] = u8(pack4(shuffle_weight(w2q.clone(), layout=(16, 16)).view(E * H, I)))
        if i == 0:     # the first case also carries its inputs; the others are regenerated from their seeds
            out.update({f"p{i}_xq": u8(xq), f"p{i}_sx": sx.numpy(), f"p{i}_w1q": u8(w1q), f"p{i}_sw1": sw1.numpy(),
                        f"p{i}_w2q": u8(w2q), f"p{i}_sw2": sw2.numpy(), f"p{i}_ids": ti.numpy(), f"p{i}_tw": tw.numpy()})
    out["n"] = np.array([len(cases)], dtype=np.int32)
    save("moe_pertoken.npz", **out)

    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
