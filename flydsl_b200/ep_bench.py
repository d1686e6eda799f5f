"""Multi-GPU leg of the benchmark: the expert-parallel layer under torchrun (one rank per GPU).

Per-GPU work is fixed as the world grows (weak scaling): every rank gates, dispatches
and combines its own ``cfg.tokens`` tokens and runs E/world local experts.  Timing is on the
device (CUDA events between barriers), the maximum over ranks is reported.
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from . import workloads as wl
from .benchutil import METRIC, UNIT, ClockSampler, load_peaks, physical_gpu_index


def run_expert_parallel(args, cfg: wl.MoEConfig, parity_fn=None):
    """``parity_fn`` (the benchmark's checker against the CPU oracle; this package imports no oracle) is
    called on every rank after the timed region with a few of the rank's own tokens."""
    from . import _lib
    from .ep import CudaOps, ExpertParallelMoE, expert_range

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    if int(getattr(args, "nccl_max_ctas", 0)) > 0:          # bound the SMs NCCL's kernels may occupy
        os.environ["NCCL_MAX_CTAS"] = str(int(args.nccl_max_ctas))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        T, k, H, I, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.inter_dim, cfg.experts
        mine = expert_range(rank, world, E)
        w1q, w1s, w2q, w2s = wl.make_weights(cfg, device=dev, experts=mine)
        logits = wl.make_logits(cfg, rank=rank).to(dev)
        _x, xq_c, xs_c = wl.make_activations(cfg, rank=rank)
        xq, xs = xq_c.to(dev), xs_c.to(dev)
        chunks = max(1, int(getattr(args, "ep_chunks", 1)))
        comm_sms = int(getattr(args, "ep_comm_sms", 0)) if chunks > 1 else 0
        mode = getattr(args, "ep_combine", "auto")
        if chunks > 1 and mode == "auto":
            mode = "nccl"                                    # the chunked pipeline is an NCCL path
        # direct dispatch writes into fixed peer-visible buffers: size them for the routing's imbalance
        headroom = 1.3 if cfg.routing == "uniform" else 3.0

        def make_ops(m):
            return CudaOps(w1q, w1s, w2q, w2s, E, k, T, tile_m=args.tile_m, chunks=chunks, comm_sms=comm_sms,
                           fused_combine=m in ("fused", "direct"), direct_dispatch=m in ("direct", "auto"),
                           device_plan=not getattr(args, "ep_host_plan", False), headroom=headroom)
        try:
            ops = make_ops(mode)
        except RuntimeError as exc:                          # no peer mapping here: same outcome on every rank
            if mode != "auto":
                raise
            if rank == 0:
                print(f"[bench] peer buffers unavailable ({exc}); using the NCCL all-to-all path", file=sys.stderr)
            mode, ops = "nccl", make_ops("nccl")
        fused, direct = ops.fused_combine, ops.direct_dispatch
        layer = ExpertParallelMoE(ops, E, k, H, chunks=chunks)
        stream = torch.cuda.current_stream()

        def timed(fn, steps):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) / steps

        for _ in range(args.warmup):
            layer(logits, xq, xs)
        torch.cuda.synchronize()
        if _lib.device_status() != 0:
            raise RuntimeError("a kernel reported a device-side timeout during warm-up")

        sampler = ClockSampler(physical_gpu_index(local_rank)) if rank == 0 else None
        ops.inner.timing_events = []
        ms = timed(lambda: layer(logits, xq, xs), args.steps)
        ev = ops.inner.timing_events
        ops.inner.timing_events = None
        clocks = sampler.stop() if sampler is not None else None
        g1 = [a.elapsed_time(b) for (n, a, b) in ev if n == "gemm1"]
        g2 = [a.elapsed_time(b) for (n, a, b) in ev if n == "gemm2"]
        # where this rank's step goes, phase by phase (a few extra steps with one event per boundary; a wait
        # for the peers also absorbs their lag, so these are this rank's view, not a sum every rank shares)
        breakdown = None
        if direct and getattr(ops, "device_plan", False):
            acc, n_bd = {}, 3
            for _ in range(n_bd):
                layer.phase_marks = []
                layer(logits, xq, xs)
                torch.cuda.synchronize()
                marks = layer.phase_marks
                for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                    acc[name] = acc.get(name, 0.0) + a.elapsed_time(b) / n_bd
            layer.phase_marks = None
            breakdown = {name: round(v, 4) for name, v in acc.items()}
        rows_in = layer.last_plan.rows_in
        imb = torch.tensor([float(rows_in)], device=dev, dtype=torch.float64)
        imb_max = imb.clone()
        dist.all_reduce(imb_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(imb, op=dist.ReduceOp.SUM)
        imbalance = float(imb_max.item()) / (float(imb.item()) / world)

        # end to end: pinned host inputs in, pinned host output back, every step; the copies run on
        # their own streams with two input slots, so they overlap the neighbouring steps' kernels
        h_logits, h_xq, h_xs = logits.cpu().pin_memory(), xq_c.view(torch.uint8).pin_memory(), xs_c.pin_memory()
        h_out = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
        h2d_s, d2h_s = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        slots = [{"logits": torch.empty_like(logits), "xq": torch.empty_like(xq.view(torch.uint8)),
                  "xs": torch.empty_like(xs), "ready": torch.cuda.Event(), "free": torch.cuda.Event()}
                 for _ in range(2)]
        out_free = torch.cuda.Event()
        out_free.record(stream)
        ops.out_free_event = out_free
        for sl in slots:
            sl["free"].record(stream)
        step_no = [0]

        def e2e_step():
            sl = slots[step_no[0] % 2]
            step_no[0] += 1
            h2d_s.wait_event(sl["free"])
            with torch.cuda.stream(h2d_s):
                sl["logits"].copy_(h_logits, non_blocking=True)
                sl["xq"].copy_(h_xq, non_blocking=True)
                sl["xs"].copy_(h_xs, non_blocking=True)
                sl["ready"].record(h2d_s)
            stream.wait_event(sl["ready"])
            # the previous result must have left the output buffer only when this step's reduce writes
            # it: the wait sits in front of the combine (ops.out_free_event), not in front of the layer
            out = layer(sl["logits"], sl["xq"], sl["xs"])
            sl["free"].record(stream)
            done = torch.cuda.Event()
            done.record(stream)
            d2h_s.wait_event(done)
            with torch.cuda.stream(d2h_s):
                h_out.copy_(out, non_blocking=True)
                out_free.record(d2h_s)

        def e2e_timed(steps):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                e2e_step()
            stream.wait_stream(d2h_s)
            stream.wait_stream(h2d_s)
            e1.record(stream)
            torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) / steps

        for _ in range(2):
            e2e_step()
        e2e_ms = e2e_timed(max(2, args.steps // 2))
        ops.out_free_event = None
        if _lib.device_status() != 0:
            raise RuntimeError("a kernel reported a device-side timeout during the timed region")

        # host link rates with every rank copying at once (the ranks share the host's memory and PCIe
        # root): the floor of an end-to-end step is the slower direction's bytes over its achieved rate
        def copy_rate(fn, nbytes):
            dist.barrier()
            torch.cuda.synchronize()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record(stream)
            for _ in range(3):
                fn()
            c1.record(stream)
            torch.cuda.synchronize()
            t = torch.tensor([c0.elapsed_time(c1) / 3], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return nbytes / (float(t.item()) * 1e-3) / 1e9, float(t.item())

        def h2d_all():
            slots[0]["logits"].copy_(h_logits, non_blocking=True)
            slots[0]["xq"].copy_(h_xq, non_blocking=True)
            slots[0]["xs"].copy_(h_xs, non_blocking=True)
        h2d_bytes_rank = h_logits.numel() * 4 + h_xq.numel() + h_xs.numel() * 4
        d2h_bytes_rank = h_out.numel() * 2
        h2d_gbs, h2d_ms = copy_rate(h2d_all, h2d_bytes_rank)
        d2h_gbs, d2h_ms = copy_rate(lambda: h_out.copy_(ops.out, non_blocking=True), d2h_bytes_rank)

        # both directions at once, as in an end-to-end step (input of step i+1 in, result of step i out): on a
        # host whose memory or root port is shared by all ranks the two directions slow each other down
        def both_ways():
            h2d_s.wait_stream(stream)
            d2h_s.wait_stream(stream)
            with torch.cuda.stream(h2d_s):
                h2d_all()
            with torch.cuda.stream(d2h_s):
                h_out.copy_(ops.out, non_blocking=True)
            stream.wait_stream(h2d_s)
            stream.wait_stream(d2h_s)
        _, both_ms = copy_rate(both_ways, h2d_bytes_rank + d2h_bytes_rank)

        # ---- checker: a few of this rank's own tokens against the CPU oracle
        parity = None
        if parity_fn is not None:
            toks = sorted({0, T // 3, (2 * T) // 3, T - 1})
            out_d = layer(logits, xq, xs)
            torch.cuda.synchronize()

            def fetch(e):
                w = wl.make_weights(cfg, device=dev, experts=[e])
                return tuple(t[0].cpu() for t in w)
            mine_chk = parity_fn(cfg, toks, logits.cpu(), xq_c, xs_c, out_d[torch.tensor(toks, device=dev)], fetch)
            gathered = [None] * world
            dist.all_gather_object(gathered, mine_chk)
            parity = {"tokens_per_rank": len(toks), "ranks": world, "tokens": toks,
                      "experts_checked": sum(c["experts_checked"] for c in gathered),
                      "max_abs_err": max(c["max_abs_err"] for c in gathered), "rtol": 2e-2, "atol": 2e-2,
                      "ok_per_rank": [bool(c["ok"]) for c in gathered], "ok": all(c["ok"] for c in gathered)}

        # ---- the same per-GPU work on ONE GPU (rank 0 alone, every expert local, no exchange): the
        # denominator of the weak-scaling efficiency on equal work
        same_work_ms = None
        if not getattr(args, "no_same_work", False):
            if rank == 0:
                from .layer import FusedMoEBlockscale
                aw = wl.make_weights(cfg, device=dev)
                one = FusedMoEBlockscale(*aw, k, max_tokens=T, tile_m=args.tile_m)
                xs_t = xs.t().contiguous()
                for _ in range(3):
                    one(logits, xq, xs_t)
                torch.cuda.synchronize()
                s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record(stream)
                for _ in range(10):
                    one(logits, xq, xs_t)
                s1.record(stream)
                torch.cuda.synchronize()
                same_work_ms = s0.elapsed_time(s1) / 10
                del one, aw
            dist.barrier()

        # this library's kernels per step: gate, unit-1 sort, pack (2 row gathers) or the dispatch kernel,
        # the local experts (their own sort + gather unless the rows arrive sorted), inverse (2) + reduce
        sort1 = 1 if (T // chunks) * k <= 8192 else 3
        if direct:
            # gate, sort, [expert counts, 2 planner kernels when planned on the device], dispatch, 2 GEMMs,
            # inverse (2) + reduce
            launches = 1 + sort1 + (3 if ops.device_plan else 0) + 1 + 2 + 3
        else:
            launches = 1 + chunks * (sort1 + 2 + ops.inner.experts_kernel_launches(rows_in // chunks) + 3)
        if rank != 0:
            return None
        peaks = load_peaks()
        flops = cfg.flops() * world
        fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        s1_ms = sum(g1) / args.steps if g1 else float("nan")       # all chunks of one step
        s2_ms = sum(g2) / args.steps if g2 else float("nan")
        s1_flops = 2.0 * rows_in * 2 * I * H
        nplan = layer.last_plan
        remote = nplan.rows_out - nplan.send_counts[rank]
        roofline = {"kernel": "moe_gemm_sm100_kernel<1> (stage 1, rank 0)", "bound": "tensor",
                    "achieved": round(s1_flops / (s1_ms * 1e-3) / 1e12, 1), "peak": fp8_peak,
                    "peak_source": peaks["source"] + ": 2 x sustained cuBLAS bf16 (no fp8 peak is measured)",
                    "unit": "TFLOP/s", "frac": round(s1_flops / (s1_ms * 1e-3) / 1e12 / fp8_peak, 4),
                    "traffic": None, "ms_per_step_all_chunks": round(s1_ms, 4),
                    "stage2_ms_per_step_all_chunks": round(s2_ms, 4),
                    "rows_received_rank0": rows_in}
        fused_roofline = None
        if fused and s2_ms == s2_ms:
            # stage 2 + combine in one kernel: bounded by the slower of its math at the FP8 peak and its
            # peer stores at the measured per-direction NVLink rate of this pool (770 GB/s)
            s2_flops = 2.0 * rows_in * H * I
            link_bytes = float(rows_in - nplan.recv_counts[rank]) * H * 2
            t_tensor, t_link = s2_flops / (fp8_peak * 1e12), link_bytes / 770e9
            target = max(t_tensor, t_link)
            fused_roofline = {"kernel": "moe_gemm_sm100_kernel<2, true> (stage 2 + combine, rank 0)",
                              "bound": "nvlink" if t_link > t_tensor else "tensor",
                              "tensor_ms": round(t_tensor * 1e3, 4), "nvlink_ms": round(t_link * 1e3, 4),
                              "nvlink_peak_gbs": 770.0, "nvlink_bytes": int(link_bytes),
                              "measured_ms": round(s2_ms, 4), "frac": round(target * 1e3 / s2_ms, 4)}
        return {"metric": METRIC, "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate and scales)",
                "data": "synthetic",
                "config": {**wl.describe(cfg), "tokens_per_gpu": T, "experts_per_gpu": len(mine),
                           "tile_m": args.tile_m, "parallelism": f"ep{world}", "pipeline_chunks": chunks, "sms_left_to_nccl": comm_sms,
                           "dispatch": (f"peer stores into the owners' sorted operand buffers ({ops.peers.kind})"
                                        if direct else "nccl all_to_all"),
                           "step_plan": ("on the device (no host synchronisation in the step)" if ops.device_plan
                                         else "on the host (one synchronisation per step)"),
                           "combine": (f"peer stores from the stage-2 epilogue ({ops.peers.kind})" if fused
                                       else "nccl all_to_all"),
                           "l2_policy": "inputs exceed L2 (dispatched rows and expert weights are GBs per step)"},
                "roofline": roofline,
                "fused_stage2_roofline": fused_roofline,
                "comm": {"dispatch_bytes_rank0": int(remote * (H + H // 128 * 4 + (0 if direct else 4))),
                         "combine_bytes_rank0": int(remote * H * 2), "load_imbalance_max_over_mean": round(imbalance, 3)},
                "step_breakdown_ms_rank0": breakdown,
                "parity_check": parity,
                "same_work_1gpu_ms": None if same_work_ms is None else round(same_work_ms, 4),
                "weak_scaling_eff": None if same_work_ms is None else round(same_work_ms / ms, 4),
                "cpu_baseline": None,
                "e2e": {"value": round(flops / (e2e_ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
                        "h2d_bytes_per_step": int(world * h2d_bytes_rank),
                        "d2h_bytes_per_step": int(world * d2h_bytes_rank),
                        "h2d_gbs_per_rank_all_ranks_copying": round(h2d_gbs, 2),
                        "d2h_gbs_per_rank_all_ranks_copying": round(d2h_gbs, 2),
                        "pcie_floor_ms": round(max(h2d_ms, d2h_ms, both_ms), 4),
                        "pcie_ms_one_direction_at_a_time": [round(h2d_ms, 4), round(d2h_ms, 4)],
                        "bound": "pcie" if max(h2d_ms, d2h_ms) > ms else "device",
                        "how": "two input slots; the result's device-to-host copy overlaps the next step up to its reduce"},
                "clocks": clocks,
                "gpu_launches": args.steps * launches}
    finally:
        dist.destroy_process_group()
