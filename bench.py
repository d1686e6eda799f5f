#!/usr/bin/env python
"""Benchmark of the FP8 block-scaled fused-MoE layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one pass of the whole path (gating -> sort -> [gather] -> stage 1 -> stage 2)
over one batch of seeded synthetic tokens.  N=1 runs the DeepSeek-V3-shaped prefill
layer (T=4096, H=7168, I=2048, E=256, top-8; workload ``c4a``); N>1 runs the
expert-parallel configuration (T=16384 tokens per GPU, experts sharded over the ranks,
NCCL all-to-all dispatch/combine; workload ``c5a``), launched by torchrun with one rank
per GPU.  Rank 0 prints ONE JSON line.

``value`` is algorithmic TFLOP/s (6*T*k*H*I per step, whole job) with inputs resident in
HBM; ``e2e`` is the same metric through the public layer call with host (pinned) buffers,
host<->device copies inside the timed region.  ``roofline`` describes the dominant kernel
(stage 1), timed with CUDA events inside the timed region.  ``decode`` (N=1 default run only)
is the other half of the metric: the T=64 decode layer's weight-streaming GB/s.
``parity_check`` compares a few tokens of the timed layer's output with the CPU oracle after
the timed region; the run exits non-zero when it fails.  ``cpu_baseline`` times the CPU
oracle (the reference's torch path restated) on a bounded sample on the host cores.
``--impl reference`` times only that CPU path and prints the same line shape.
``--wait-accounting`` (with FLYMOE_LIB pointing at a ``python -m flydsl_b200.build --prof`` build)
prints where the grouped-GEMM roles wait instead of the JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from flydsl_b200 import workloads as wl  # noqa: E402
from flydsl_b200.benchutil import METRIC, UNIT, ClockSampler, load_peaks, physical_gpu_index  # noqa: E402


# ------------------------------------------------------------------------------------ CPU arm
def cpu_baseline(cfg: wl.MoEConfig, n_sample_experts: int, device_weights=None, ids=None, tw=None,
                 xq=None, xs=None) -> dict:
    """Time the CPU oracle on the tokens routed to the first ``n_sample_experts`` experts."""
    from oracle import moe_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if ids is None:
        logits = wl.make_logits(cfg)
        _x, xq, xs = wl.make_activations(cfg)
        tw, ids, _ = orc.topk_gating_softmax(logits, cfg.topk)
    n = min(n_sample_experts, cfg.experts)
    if device_weights is not None:
        w1q, w1s, w2q, w2s = (t[:n].cpu() for t in device_weights)
    else:
        w1q, w1s, w2q, w2s = wl.make_weights(cfg, experts=range(n))
    ids_s = torch.where(ids < n, ids, torch.full_like(ids, -1))
    pairs = int((ids_s >= 0).sum())
    t0 = time.perf_counter()
    tw_r, ids_r, _ = orc.topk_gating_softmax(wl.make_logits(cfg), cfg.topk)
    orc.moe_sorting(ids_r.numpy(), tw_r.numpy(), cfg.experts, 128)
    o1 = orc.stage1(xq, xs, w1q, w1s, ids_s, cfg.inter_dim)
    a2q, a2s = orc.requant(o1)
    orc.stage2(a2q, a2s, w2q, w2s, ids_s, tw, cfg.model_dim)
    dt = time.perf_counter() - t0
    flops = 6.0 * pairs * cfg.model_dim * cfg.inter_dim
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"whole routing plus experts 0..{n - 1} of {cfg.experts} with the {pairs} (token, slot) "
                      f"pairs routed to them ({pairs / max(1, cfg.pairs):.3f} of the layer's FLOPs), "
                      f"{dt:.2f} s of CPU work; the rate of this sample stands for the whole layer",
            "sample_fraction_of_layer_flops": round(pairs / max(1, cfg.pairs), 4),
            "extrapolated_from_sample": bool(pairs < cfg.pairs), "seconds": round(dt, 3)}


def run_reference_arm(args, cfg, rank: int) -> None:
    if rank != 0:
        return
    # Each step is one bounded sample (~1.5 s of CPU work).  W warm-up samples and up to K timed ones are
    # run, but no more than fit into about a minute, so that large K still ends within minutes.
    from oracle import moe_oracle as orc
    n = min(args.cpu_experts, cfg.experts)
    weights = wl.make_weights(cfg, experts=range(n))               # generated once, outside every timed sample
    logits = wl.make_logits(cfg)
    _x, xq, xs = wl.make_activations(cfg)
    tw, ids, _ = orc.topk_gating_softmax(logits, cfg.topk)
    sample = dict(device_weights=weights, ids=ids, tw=tw, xq=xq, xs=xs)
    budget_s, t_begin = 60.0, time.perf_counter()
    warm = 0
    for _ in range(min(max(args.warmup, 0), 2)):
        cpu_baseline(cfg, n, **sample)
        warm += 1
    vals = []
    last = None
    for _ in range(max(1, args.steps)):
        last = cpu_baseline(cfg, n, **sample)
        vals.append(last["value"])
        if time.perf_counter() - t_begin > budget_s:
            break
    v = statistics.median(vals)
    last["value"] = v
    line = {"metric": METRIC, "value": v, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
            "steps": len(vals), "steps_requested": args.steps, "warmup": warm,
            "ms_per_step": last["seconds"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 (CPU dequantised fp8)", "data": "synthetic",
            "config": wl.describe(cfg), "cpu_baseline": last,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def auto_tile_m(cfg: wl.MoEConfig, world: int = 1) -> int:
    """Row block = sort unit: the smallest of 16/32/64/128 that covers the mean rows per expert."""
    rows = cfg.tokens * cfg.topk / cfg.experts * 1.0
    for m in (16, 32, 64):
        if rows <= m:
            return m
    return 128


# DRAM bytes per launch of the stage-1 kernel from ncu (dram__bytes_read.sum + dram__bytes_write.sum),
# keyed by (workload, tile_m); sources and scaling are in profiles/.
MEASURED_TRAFFIC = {
    ("c4a-dsv3-prefill-uniform", 128): 8.164e9,   # 8 x the T=512/E=32 capture (same tokens per expert)
    ("c3-dsv3-decode", 16): 6.60e9,               # full-size capture
}


class ExpertTable:
    """Expert-indexable view for the oracle: ``fetch(e)`` returns one expert's tensor on the CPU."""

    def __init__(self, experts: int, fetch):
        self.n, self.fetch, self.cache = experts, fetch, {}

    def __len__(self):
        return self.n

    def __getitem__(self, e):
        if e not in self.cache:
            self.cache[e] = self.fetch(e)
        return self.cache[e]


def parity_check(cfg: wl.MoEConfig, tokens, logits_c, xq_c, xs_c, out_rows, fetch_expert) -> dict:
    """Checker, run after the timed region: the layer's output rows ``out_rows`` (bf16, one per entry of
    ``tokens``) against the CPU oracle on the same pre-quantised inputs (bar: rtol 2e-2 / atol 2e-2).
    ``fetch_expert(e)`` returns (w1q, w1_scale, w2q, w2_scale) of global expert e; only the experts the
    chosen tokens route to are fetched."""
    from oracle import moe_oracle as orc
    sel = torch.as_tensor(tokens, dtype=torch.int64)
    tw, ids, _ = orc.topk_gating_softmax(logits_c[sel], cfg.topk)
    cache = {}

    def fetch(e):
        if e not in cache:
            cache[e] = fetch_expert(e)
        return cache[e]
    tabs = [ExpertTable(cfg.experts, (lambda e, j=j: fetch(e)[j])) for j in range(4)]
    o1 = orc.stage1(xq_c[sel], xs_c[sel], tabs[0], tabs[1], ids, cfg.inter_dim)
    a2q, a2s = orc.requant(o1)
    ref = orc.stage2(a2q, a2s, tabs[2], tabs[3], ids, tw, cfg.model_dim)
    got = out_rows.float().cpu()
    err = (got - ref).abs()
    ok = bool(torch.isfinite(got).all()) and bool((err <= 2e-2 + 2e-2 * ref.abs()).all())
    return {"tokens": [int(t) for t in tokens], "experts_checked": len(cache), "max_abs_err": round(float(err.max()), 5),
            "ref_max_abs": round(float(ref.abs().max()), 4), "rtol": 2e-2, "atol": 2e-2, "ok": ok}


def wait_accounting(args, cfg) -> None:
    """Mean cycles per 128-wide K block that each role of the grouped-GEMM kernels spends waiting, read
    from a library built with -DFLYMOE_PROF (FLYMOE_LIB=flydsl_b200/libflymoe_sm100_prof.so)."""
    import ctypes
    import numpy as np
    from flydsl_b200 import _lib
    from flydsl_b200.layer import FusedMoEBlockscale
    lib = _lib.load()
    if not hasattr(lib, "flymoe_prof_read"):
        raise SystemExit("this library was built without -DFLYMOE_PROF: run `python -m flydsl_b200.build --prof` "
                         "and set FLYMOE_LIB=flydsl_b200/libflymoe_sm100_prof.so")
    lib.flymoe_prof_read.argtypes = [ctypes.c_void_p]
    dev = torch.device("cuda", 0)
    T, k, H, I, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
    w1q, w1s, w2q, w2s = wl.make_weights(cfg, device=dev)
    logits = wl.make_logits(cfg).to(dev)
    _x, xq_c, xs_c = wl.make_activations(cfg)
    xq, xs_t = xq_c.to(dev), xs_c.t().contiguous().to(dev)
    layer = FusedMoEBlockscale(w1q, w1s, w2q, w2s, k, max_tokens=T, tile_m=args.tile_m)
    for _ in range(max(args.warmup, 10)):
        layer(logits, xq, xs_t)
    torch.cuda.synchronize()
    buf = np.zeros((256, 3, 8), dtype=np.int64)

    def show(tag):
        lib.flymoe_prof_read(buf.ctypes.data)
        b = buf[:torch.cuda.get_device_properties(dev).multi_processor_count].astype(np.float64)
        p, m, e = b[:, 0], b[:, 1], b[:, 2]
        nkb = max(m[:, 6].mean(), 1.0)
        print(json.dumps({"kernel": tag, "workload": cfg.name, "k_blocks_per_cta": round(nkb, 1),
                          "cycles_per_k_block": round(m[:, 0].mean() / nkb, 1),
                          "tma_role_cycles_per_k_block": round(p[:, 0].mean() / nkb, 1),
                          "epilogue_role_cycles_per_k_block": round(e[:, 0].mean() / nkb, 1),
                          "tma_wait_free_smem_stage": round(p[:, 1].mean() / nkb, 1),
                          "mma_wait_tmem_stage": round(m[:, 1].mean() / nkb, 1),
                          "mma_wait_operands": round(m[:, 2].mean() / nkb, 1),
                          "mma_issue_and_commit": round(m[:, 4].mean() / nkb, 1),
                          "epilogue_wait_mma": round(e[:, 1].mean() / nkb, 1),
                          "tile_end_cycles_per_tile": round(e[:, 2].mean() / max(e[:, 5].mean(), 1.0), 1)}), flush=True)
    show("stage 2 (last launch of the layer)")
    # stage 1 alone, so that its counters are the last ones written
    U = layer.tile_m
    cap = T * k + E * U - k
    blocks = (cap + U - 1) // U
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        _lib.check(lib.flymoe_moe_gemm1(
            layer.a2q.data_ptr(), layer.a2_scale.data_ptr(), layer.cap_rows,
            xq.data_ptr() if layer.gather_in_kernel else layer.xs.data_ptr(), xs_t.data_ptr(), T, 1,
            w1q.data_ptr(), w1s.data_ptr(), layer.sorted_ids.data_ptr(), layer.sorted_expert_ids.data_ptr(),
            layer.sorted_weights.data_ptr(), layer.num_valid_ids.data_ptr(), T, I, H, blocks, E, k, U, 0, _lib.E4M3,
            _lib.ROWS_BY_TOKEN if layer.gather_in_kernel else _lib.ROWS_SORTED, _lib.ROWS_BY_TOKEN, _lib.ROWS_SORTED,
            0, st), "moe_gemm1")
    torch.cuda.synchronize()
    show("stage 1")


# ------------------------------------------------------------------------------------ GPU arm
def run_single_gpu(args, cfg, with_e2e: bool = True, with_cpu: bool = True, with_parity: bool = True) -> dict:
    from flydsl_b200 import _lib
    from flydsl_b200.layer import FusedMoEBlockscale
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    T, k, H, I, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
    w1q, w1s, w2q, w2s = wl.make_weights(cfg, device=dev)
    logits = wl.make_logits(cfg).to(dev)
    _x, xq_c, xs_c = wl.make_activations(cfg)
    xq, xs_t = xq_c.to(dev), xs_c.t().contiguous().to(dev)
    layer = FusedMoEBlockscale(w1q, w1s, w2q, w2s, k, max_tokens=T, tile_m=args.tile_m,
                               stage2_mode=args.stage2_mode)
    stream = torch.cuda.current_stream()

    def step():
        return layer(logits, xq, xs_t)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side timeout during warm-up")

    # ---- timed region: K steps, stage-1/2 kernels bracketed by their own events
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    layer.timing_events = []
    sampler = ClockSampler(physical_gpu_index(torch.cuda.current_device()))
    torch.cuda.synchronize()
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    total_ms = ev0.elapsed_time(ev1)
    ms_per_step = total_ms / args.steps
    g1 = [a.elapsed_time(b) for (name, a, b) in layer.timing_events if name == "gemm1"]
    g2 = [a.elapsed_time(b) for (name, a, b) in layer.timing_events if name == "gemm2"]
    layer.timing_events = None
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side timeout during the timed region")
    flops = cfg.flops()
    value = flops / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel (stage 1)
    ids = layer.topk_ids[:T].cpu()
    e_act = int(torch.unique(ids).numel())
    rows = int(layer.num_valid_ids[0])
    # algorithmic bytes of one stage-1 launch: W1 of the active experts with their block scales, the
    # activations with their 1x128 scales once per token, the e4m3 intermediate with its scales once per
    # (token, slot) pair.  What the design moves on top of that (every sorted row's activations fetched by index,
    # mostly from L2, and the padded rows of the intermediate) is reported apart.
    s1_bytes = (e_act * 2.0 * I * H * (1 + 4.0 / (128 * 128)) + T * H * (1 + 4.0 / 128)
                + T * k * I * (1 + 4.0 / 128))
    s1_moved = (e_act * 2.0 * I * H * (1 + 4.0 / (128 * 128)) + rows * H + T * (H // 128) * 4.0
                + rows * I * (1 + 4.0 / 128))
    s1_ms = statistics.mean(g1) if g1 else float("nan")
    s2_ms = statistics.mean(g2) if g2 else float("nan")
    achieved = s1_bytes / (s1_ms * 1e-3) / 1e9
    s1_flops = 2.0 * T * k * 2 * I * H
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    roofline = {"kernel": "moe_gemm_sm100_kernel<1> (stage 1)", "bound": "hbm", "achieved": round(achieved, 1),
                "peak": peaks["hbm_gbs"], "peak_source": peaks["source"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4),
                "traffic": MEASURED_TRAFFIC.get((cfg.name, args.tile_m)),
                "algorithmic_bytes_per_launch": int(s1_bytes), "bytes_moved_by_design": int(s1_moved),
                "ms_per_launch": round(s1_ms, 4),
                "stage2_ms_per_launch": round(s2_ms, 4),
                "tensor_tflops": round(s1_flops / (s1_ms * 1e-3) / 1e12, 1),
                "tensor_frac_of_2x_bf16_peak": round(s1_flops / (s1_ms * 1e-3) / 1e12 / fp8_peak, 4),
                "active_experts": e_act, "padded_rows": rows}
    total_bytes = wl.weight_bytes_active(cfg, ids)

    parity = None
    if with_parity:
        n_chk = min(8, T)
        toks = sorted({int(round(i * (T - 1) / max(1, n_chk - 1))) for i in range(n_chk)})
        out_d = step()
        torch.cuda.synchronize()
        parity = parity_check(cfg, toks, logits.cpu(), xq_c, xs_c, out_d[torch.tensor(toks, device=dev)],
                              lambda e: (w1q[e].cpu(), w1s[e].cpu(), w2q[e].cpu(), w2s[e].cpu()))

    result = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
              "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
              "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate and scales)",
              "data": "synthetic",
              "config": {**wl.describe(cfg), "tile_m": args.tile_m, "stage2_mode": args.stage2_mode,
                         "parallelism": "single GPU",
                         "l2_policy": "inputs exceed L2: %.1f GB of expert weights stream per step" % (e_act * 3.0 * H * I / 1e9)},
              "layer_hbm_gbs": round(total_bytes / (ms_per_step * 1e-3) / 1e9, 1),
              "layer_hbm_frac": round(total_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
              "roofline": roofline, "parity_check": parity, "cpu_baseline": None, "e2e": None, "clocks": clocks,
              "gpu_launches": args.steps * layer.kernel_launches(T)}
    if not with_e2e:
        return result

    # ---- end to end: pinned host inputs -> device -> layer -> pinned host output, every step,
    # through the host-streaming front end (copies of neighbouring steps overlap this step's kernels)
    from flydsl_b200.host_pipeline import HostPipeline
    h_logits = logits.cpu().pin_memory()
    h_xq = xq_c.view(torch.uint8).pin_memory()
    h_xs = xs_c.t().contiguous().pin_memory()
    h_outs = [torch.empty((T, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    pipe = HostPipeline(layer, T, logits_dtype=logits.dtype, depth=2)
    for i in range(min(3, args.warmup)):
        pipe.submit(h_logits, h_xq, h_xs, h_outs[i % 2])
    pipe.drain()
    e0 = pipe.mark()
    for i in range(args.steps):
        pipe.submit(h_logits, h_xq, h_xs, h_outs[i % 2])
    e1 = pipe.mark()
    pipe.drain()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    if not bool(torch.isfinite(h_outs[(args.steps - 1) % 2].float()).all()):
        raise RuntimeError("end-to-end output contains non-finite values")
    h2d = h_logits.numel() * 4 + h_xq.numel() + h_xs.numel() * 4
    d2h = h_outs[0].numel() * 2
    e2e = {"value": round(flops / (e2e_ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
           "how": "HostPipeline, depth 2: pinned host in, pinned host out, copies overlapped across steps"}

    result["e2e"] = e2e
    if with_cpu and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(cfg, args.cpu_experts, device_weights=(w1q, w1s, w2q, w2s), ids=ids,
                                              tw=layer.topk_weights[:T].cpu(), xq=xq_c, xs=xs_c)
    return result


def run_decode_leg(args) -> dict:
    """The decode half of the metric for the default line: the T=64 DeepSeek-V3-shaped layer (workload c3,
    row block 16), whose time is the streaming of the routed experts' weights from HBM."""
    import copy
    a = copy.copy(args)
    a.tile_m, a.steps, a.warmup = 16, max(50, min(args.steps, 200)), max(args.warmup, 5)
    r = run_single_gpu(a, wl.CONFIGS["c3"], with_e2e=False, with_cpu=False)
    keep = ("ms_per_step", "steps", "layer_hbm_gbs", "layer_hbm_frac", "value", "roofline", "parity_check", "clocks")
    d = {"workload": r["config"]["workload"], "tile_m": 16, "metric": "weight-streaming HBM GB/s of the decode layer",
         **{kk: r[kk] for kk in keep}}
    d["tflops"] = d.pop("value")
    return d


def run_dense_gemm(args) -> dict:
    """`--workload gemm`: the dense block-scaled FP8 GEMM (kernels.blockscale_preshuffle_gemm) on one
    GPU.  Weight copies rotate so that every launch streams weights that are not in L2."""
    from flydsl_b200 import _lib
    from flydsl_b200.kernels.blockscale_preshuffle_gemm import compile_blockscale_preshuffle_gemm
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    M, N, K = args.tokens or 4096, args.gemm_n, args.gemm_k
    tile_m = args.tile_m if args.tile_m else (16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128)
    g = torch.Generator().manual_seed(5)
    x = (torch.rand((M, K), generator=g) / 10).to(torch.float16).to(torch.float8_e4m3fn).to(dev)
    sa = torch.rand((K // 128, M), generator=g).to(dev)
    copies = max(2, int(2 * 126e6 // (N * K)) + 1)                       # > 2 x L2 of weights in rotation
    ws = [(torch.rand((N, K), generator=g) / 10).to(torch.float16).to(torch.float8_e4m3fn).to(dev)
          for _ in range(copies)]
    sb = torch.rand((N // 128, K // 128), generator=g).to(dev)
    c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    exe = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=tile_m, tile_n=128, tile_k=128, w_layout="plain")
    stream = torch.cuda.current_stream()
    for i in range(args.warmup):
        exe(c, x, ws[i % copies], sa, sb, M, N, stream)
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        exe(c, x, ws[i % copies], sa, sb, M, N, stream)
    e1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side timeout")
    ms = e0.elapsed_time(e1) / args.steps
    flops = 2.0 * M * N * K
    nbytes = M * K + N * K + M * N * 2 + (M * (K // 128) + (N // 128) * (K // 128)) * 4
    tf, gbs = flops / (ms * 1e-3) / 1e12, nbytes / (ms * 1e-3) / 1e9
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    t_tensor, t_hbm = flops / (fp8_peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)
    bound = "tensor" if t_tensor >= t_hbm else "hbm"
    return {"metric": "fp8_blockscale_gemm_tflops", "value": round(tf, 2), "unit": UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate and scales)",
            "data": "synthetic",
            "config": {"workload": f"dense-gemm-M{M}-N{N}-K{K}", "tile_m": tile_m,
                       "l2_policy": f"{copies} weight copies in rotation ({copies * N * K / 1e6:.0f} MB > 2 x L2)"},
            "roofline": {"kernel": "moe_gemm_sm100_kernel<2> (one expert, identity routing)", "bound": bound,
                         "achieved": round(tf if bound == "tensor" else gbs, 1),
                         "peak": fp8_peak if bound == "tensor" else peaks["hbm_gbs"],
                         "peak_source": peaks["source"] + (": 2 x burst cuBLAS bf16" if bound == "tensor" else ""),
                         "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
                         "frac": round(max(t_tensor, t_hbm) * 1e3 / ms, 4), "traffic": None,
                         "algorithmic_bytes_per_launch": int(nbytes), "gbs": round(gbs, 1)},
            "cpu_baseline": None, "e2e": None, "clocks": clocks, "gpu_launches": 2 * args.steps}


def run_pertoken(args, cfg) -> dict:
    """`--scaling pertoken`: the two grouped GEMM stages of the per-token / per-channel-scale family
    (kernels.moe_gemm_2stage, fp8) on the workload's shapes and routing.  The whole K range accumulates in
    tensor memory and every tile is drained once, so this is the control for the block-scaled kernels: same
    main loop without the per-K-block scale pass.  Stage 2's input is the quantised stage-1 output, prepared
    outside the timed region (the reference quantises between the stages outside its kernels, too)."""
    from flydsl_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    lib = _lib.load()
    T, k, H, I, E, U = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts, args.tile_m
    g = torch.Generator(device=dev).manual_seed(cfg.seed)
    half = args.in_dtype == "bf16"          # 16-bit operands: no scales at all, twice the operand bytes
    wdt = torch.bfloat16 if half else torch.float8_e4m3fn
    in_code, ebytes = (_lib.BF16, 2) if half else (_lib.E4M3, 1)
    w1q = torch.empty((E, 2 * I, H), dtype=wdt, device=dev)
    w2q = torch.empty((E, H, I), dtype=wdt, device=dev)
    sw1 = torch.empty((E, 2 * I), dtype=torch.float32, device=dev)
    sw2 = torch.empty((E, H), dtype=torch.float32, device=dev)
    for e in range(E):
        if half:
            w1q[e] = (torch.randn((2 * I, H), generator=g, device=dev) * 0.02).to(wdt)
            w2q[e] = (torch.randn((H, I), generator=g, device=dev) * 0.02).to(wdt)
            continue
        q, sc = wl.quant_groups(torch.randn((2 * I, H), generator=g, device=dev) * 0.02)
        w1q[e], sw1[e] = q, sc.view(-1)
        q, sc = wl.quant_groups(torch.randn((H, I), generator=g, device=dev) * 0.02)
        w2q[e], sw2[e] = q, sc.view(-1)
    if half:
        xq, sx = torch.randn((T, H), generator=g, device=dev).to(wdt), None
    else:
        xq, sx = wl.quant_groups(torch.randn((T, H), generator=g, device=dev))
    scale_ptr = (lambda t: None) if half else (lambda t: t.data_ptr())
    logits = wl.make_logits(cfg).to(dev)
    i32, f32 = torch.int32, torch.float32
    tw, ids, tei = (torch.empty((T, k), dtype=dt, device=dev) for dt in (f32, i32, i32))
    cap = T * k + E * U - k
    blocks = (cap + U - 1) // U
    rows = blocks * U
    s_ids, s_w = torch.empty(rows, dtype=i32, device=dev), torch.empty(rows, dtype=f32, device=dev)
    s_e, nv = torch.empty(blocks, dtype=i32, device=dev), torch.zeros(2, dtype=i32, device=dev)
    ws = torch.empty(max(1, int(lib.flymoe_moe_sorting_workspace_elems(T, E, k, U))), dtype=i32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.flymoe_topk_gating_softmax(logits.data_ptr(), _lib.F32, tw.data_ptr(), ids.data_ptr(), tei.data_ptr(),
                                              T, E, k, 1, st), "gating")
    _lib.check(lib.flymoe_moe_sorting(ids.data_ptr(), tw.data_ptr(), s_ids.data_ptr(), s_w.data_ptr(), s_e.data_ptr(),
                                      nv.data_ptr(), None, 0, None, ws.data_ptr(), ws.numel(), T, E, k, U, st), "sorting")
    xs = torch.empty((rows, H * ebytes), dtype=torch.uint8, device=dev)
    _lib.check(lib.flymoe_gather_rows(xq.data_ptr(), xs.data_ptr(), s_ids.data_ptr(), nv.data_ptr(), T, k, H * ebytes,
                                      _lib.ROWS_BY_TOKEN, rows, st), "gather")
    out1 = torch.zeros((rows, I), dtype=torch.bfloat16, device=dev)
    out2 = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)

    def stage1():
        _lib.check(lib.flymoe_moe_gemm1_pertoken(
            out1.data_ptr(), xs.data_ptr(), scale_ptr(sx), w1q.data_ptr(), scale_ptr(sw1), s_ids.data_ptr(),
            s_e.data_ptr(), s_w.data_ptr(), nv.data_ptr(), T, I, H, blocks, E, k, U, 0, in_code, _lib.BF16,
            _lib.ROWS_SORTED, _lib.ROWS_BY_TOKEN, _lib.ROWS_SORTED, _lib.IMPL_TCGEN05, st), "gemm1_pertoken")
    stage1()
    if half:
        a2q, sa2 = out1, None
    else:
        a2q, sa2 = wl.quant_groups(out1.float())
        sa2 = sa2.view(-1).contiguous()

    def stage2():
        _lib.check(lib.flymoe_moe_gemm2_pertoken(
            out2.data_ptr(), a2q.data_ptr(), scale_ptr(sa2), w2q.data_ptr(), scale_ptr(sw2), s_ids.data_ptr(),
            s_e.data_ptr(), s_w.data_ptr(), nv.data_ptr(), T, H, I, blocks, E, k, U, 1, in_code, _lib.BF16, 1,
            _lib.ROWS_SORTED, _lib.ROWS_SORTED, _lib.IMPL_TCGEN05, st), "gemm2_pertoken")
    stream = torch.cuda.current_stream()
    for _ in range(args.warmup):
        stage1()
        stage2()
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    evs[0].record(stream)
    for i in range(args.steps):
        stage1()
        evs[2 * i + 1].record(stream)
        out2.zero_()
        stage2()
        evs[2 * i + 2].record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel reported a device-side timeout")
    s1 = statistics.mean(evs[2 * i].elapsed_time(evs[2 * i + 1]) for i in range(args.steps))
    s2 = statistics.mean(evs[2 * i + 1].elapsed_time(evs[2 * i + 2]) for i in range(args.steps))
    f1, f2 = 4.0 * T * k * I * H, 2.0 * T * k * H * I
    fp8_peak = (1.0 if half else 2.0) * peaks["bf16_tflops"]      # dense tensor peak of the operand type
    e_act = int(torch.unique(ids).numel())
    wbytes1, wbytes2 = e_act * 2.0 * I * H * ebytes, e_act * 1.0 * I * H * ebytes
    if half:
        return {"metric": "bf16_moe_gemm_tflops", "value": round((f1 + f2) / ((s1 + s2) * 1e-3) / 1e12, 2), "unit": UNIT,
                "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(s1 + s2, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16 (fp32 accumulate, no scales)", "data": "synthetic",
                "config": {**wl.describe(cfg), "tile_m": U, "what": "stage 1 + stage 2 kernels of kernels.moe_gemm_2stage only"},
                "stage1": {"ms": round(s1, 4), "tflops": round(f1 / (s1 * 1e-3) / 1e12, 1),
                           "frac_of_bf16_peak": round(f1 / (s1 * 1e-3) / 1e12 / fp8_peak, 4)},
                "stage2": {"ms": round(s2, 4), "tflops": round(f2 / (s2 * 1e-3) / 1e12, 1),
                           "frac_of_bf16_peak": round(f2 / (s2 * 1e-3) / 1e12 / fp8_peak, 4)},
                "roofline": {"bound": "tensor", "achieved": round((f1 + f2) / ((s1 + s2) * 1e-3) / 1e12, 1),
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": round((f1 + f2) / ((s1 + s2) * 1e-3) / 1e12 / peaks["bf16_tflops"], 4), "traffic": None,
                             "peak_source": peaks.get("source", "")},
                "cpu_baseline": None, "e2e": None, "clocks": clocks, "gpu_launches": 2 * args.steps}
    return {"metric": "fp8_pertoken_moe_gemm_tflops", "value": round((f1 + f2) / ((s1 + s2) * 1e-3) / 1e12, 2), "unit": UNIT,
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(s1 + s2, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate, one scale per row and per weight row)", "data": "synthetic",
            "config": {**wl.describe(cfg), "tile_m": U, "what": "stage 1 + stage 2 kernels of kernels.moe_gemm_2stage only"},
            "stage1": {"ms": round(s1, 4), "tflops": round(f1 / (s1 * 1e-3) / 1e12, 1),
                       "frac_of_2x_bf16_peak": round(f1 / (s1 * 1e-3) / 1e12 / fp8_peak, 4),
                       "weight_gbs": round(wbytes1 / (s1 * 1e-3) / 1e9, 1)},
            "stage2": {"ms": round(s2, 4), "tflops": round(f2 / (s2 * 1e-3) / 1e12, 1),
                       "frac_of_2x_bf16_peak": round(f2 / (s2 * 1e-3) / 1e12 / fp8_peak, 4),
                       "weight_gbs": round(wbytes2 / (s2 * 1e-3) / 1e9, 1)},
            "roofline": None, "cpu_baseline": None, "e2e": None, "clocks": clocks, "gpu_launches": 2 * args.steps}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None,
                    help="c1|c2|c3|c4a|c4b|c5a|c5b (default c4a, or c5a when --gpus > 1); 'gemm' = the dense "
                         "block-scaled GEMM with M = --tokens, --gemm-n, --gemm-k")
    ap.add_argument("--gemm-n", type=int, default=7168)
    ap.add_argument("--gemm-k", type=int, default=2304)
    ap.add_argument("--tokens", type=int, default=None, help="override the token count (c2 sweep)")
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (small profiling cases)")
    ap.add_argument("--tile-m", type=int, default=0,
                    help="sort unit = GEMM row block (16/32/64/128); 0 = pick from the rows per expert")
    ap.add_argument("--stage2-mode", default="atomic", choices=["atomic", "reduce"])
    ap.add_argument("--ep-chunks", type=int, default=1, help="pipeline chunks of the expert-parallel layer")
    ap.add_argument("--ep-combine", choices=("auto", "nccl", "fused", "direct"), default="auto",
                    help="expert-parallel transport: NCCL all-to-all both ways; 'fused' = combine as peer stores "
                         "from stage 2's epilogue; 'direct' = dispatch as peer stores into the owners' operand buffers too")
    ap.add_argument("--ep-host-plan", action="store_true",
                    help="expert-parallel direct dispatch: plan each step on the host (one synchronisation per step, "
                         "capacity checked with an exception) instead of on the device")
    ap.add_argument("--ep-comm-sms", type=int, default=0, help="SMs the pipelined EP step leaves to NCCL")
    ap.add_argument("--nccl-max-ctas", type=int, default=0, help="sets NCCL_MAX_CTAS before the group is created")
    ap.add_argument("--cpu-experts", type=int, default=48, help="experts in the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="block", choices=["block", "pertoken"],
                    help="'pertoken': time the per-token-scale GEMM stages (kernels.moe_gemm_2stage) on the workload's shapes")
    ap.add_argument("--in-dtype", default="fp8", choices=["fp8", "bf16"],
                    help="operand type of --scaling pertoken (bf16: 16-bit operands and weights, no scales)")
    ap.add_argument("--no-parity", action="store_true", help="skip the post-run check against the CPU oracle")
    ap.add_argument("--no-same-work", action="store_true",
                    help="multi-GPU: skip timing the same per-GPU work on one GPU (weak_scaling_eff)")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode (c3) leg of the default N=1 line")
    ap.add_argument("--wait-accounting", action="store_true",
                    help="print the grouped-GEMM wait accounting (needs a -DFLYMOE_PROF build in FLYMOE_LIB)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    name = args.workload or ("c4a" if args.gpus == 1 else "c5a")
    if name == "gemm":
        if rank == 0:
            print(json.dumps(run_dense_gemm(args)), flush=True)
        return
    cfg = wl.CONFIGS[name]
    if args.tokens is not None:
        cfg = cfg.with_tokens(args.tokens)
    if args.experts is not None:
        from dataclasses import replace
        cfg = replace(cfg, experts=args.experts, name=f"{cfg.name}-E{args.experts}")

    if args.tile_m == 0:
        args.tile_m = auto_tile_m(cfg, max(1, world))
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    if args.gpus > 1 or world > 1:
        from flydsl_b200.ep_bench import run_expert_parallel
        line = run_expert_parallel(args, cfg, parity_fn=None if args.no_parity else parity_check)
        if line is not None:
            print(json.dumps(line), flush=True)
            if line.get("parity_check") is not None and not line["parity_check"]["ok"]:
                print("[bench] parity check against the CPU oracle FAILED", file=sys.stderr)
                sys.exit(3)
        return
    if args.wait_accounting:
        wait_accounting(args, cfg)
        return
    if args.scaling == "pertoken":
        print(json.dumps(run_pertoken(args, cfg)), flush=True)
        return
    line = run_single_gpu(args, cfg, with_parity=not args.no_parity)
    default_run = args.workload is None and args.tokens is None and args.experts is None
    if default_run and not args.no_decode:
        torch.cuda.empty_cache()
        line["decode"] = run_decode_leg(args)
    print(json.dumps(line), flush=True)
    checks = [line.get("parity_check"), (line.get("decode") or {}).get("parity_check")]
    if any(c is not None and not c["ok"] for c in checks):
        print("[bench] parity check against the CPU oracle FAILED", file=sys.stderr)
        sys.exit(3)


if __name__ == "__main__":
    main()
