"""Expert-parallel layer on 2 (4, 8) GPUs of one box against the single-GPU fused layer.

Each rank gates and dispatches its own tokens; experts are sharded over the ranks.  The
single-GPU layer in "reduce" mode performs the same arithmetic per (token, slot) pair
(unweighted bf16 expert output, fp32 weighted sum), so the two results must be bit-identical;
a token subset is also checked against the CPU oracle.  Skipped when the box has fewer GPUs
than ranks."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _run_ranks(world, args_of_rank):
    """Spawn one daemon process per rank, collect one result per rank, and never leave a rank behind: on a
    failure or a timeout every child is terminated (then killed) before the assertion is raised, so no
    rank keeps spinning in a collective on a shared GPU."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=args_of_rank(r, q), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    res, failure = [], None
    try:
        for _ in range(world):
            try:
                item = q.get(timeout=300)
            except Exception:                     # noqa: BLE001 - queue.Empty: a rank never reported
                failure = "a rank did not report within 300 s"
                break
            if item[0] == "error":
                failure = f"rank {item[1]} failed: {item[2]}"
                break
            res.append(item)
        if failure is None:
            for p in procs:
                p.join(timeout=120)
                if p.exitcode != 0:
                    failure = f"a rank exited with code {p.exitcode}"
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    assert failure is None, failure
    return res


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, routing, chunks, q, fused=False, direct=False):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        _run(rank, world, routing, chunks, q, fused, direct, dev)
    except Exception as exc:                      # noqa: BLE001 - the parent fails at once instead of timing out
        q.put(("error", rank, repr(exc)))
        q.close()
        q.join_thread()
        os._exit(1)                               # no collective teardown on the error path: it could block
    dist.destroy_process_group()


def _run(rank, world, routing, chunks, q, fused, direct, dev):
    import torch.distributed as dist
    from flydsl_b200 import _lib, workloads as wl
    from flydsl_b200.ep import CudaOps, ExpertParallelMoE, expert_range
    from flydsl_b200.layer import FusedMoEBlockscale
    from oracle import moe_oracle as orc
    cfg = wl.MoEConfig("ep-test", 300, 512, 256, 16, 4, 11, routing)
    T, k, H, E = cfg.tokens, cfg.topk, cfg.model_dim, cfg.experts
    w1q, w1s, w2q, w2s = wl.make_weights(cfg, device=dev)                    # all experts (for the check)
    mine = expert_range(rank, world, E)
    sl = slice(mine.start, mine.stop)
    logits = wl.make_logits(cfg, rank=rank).to(dev)
    _x, xq_c, xs_c = wl.make_activations(cfg, rank=rank)
    xq, xs = xq_c.to(dev), xs_c.to(dev)
    ops = CudaOps(w1q[sl].contiguous(), w1s[sl].contiguous(), w2q[sl].contiguous(), w2s[sl].contiguous(),
                  E, k, T, tile_m=128, headroom=float(max(world, 2)) if direct else 1.0, chunks=chunks,
                  fused_combine=fused, direct_dispatch=bool(direct), device_plan=direct == "device")
    layer = ExpertParallelMoE(ops, E, k, H, chunks=chunks)
    out = layer(logits, xq, xs).clone()
    out2 = layer(logits, xq, xs).clone()                                     # buffers are reused
    torch.cuda.synchronize()
    single = FusedMoEBlockscale(w1q, w1s, w2q, w2s, k, max_tokens=T, tile_m=128, stage2_mode="reduce")
    want = single(logits, xq, xs.t().contiguous())
    torch.cuda.synchronize()
    sel = torch.tensor([0, 7, 299])
    tw, ids, _ = orc.topk_gating_softmax(logits.cpu(), k)
    o1 = orc.stage1(xq_c[sel], xs_c[sel], w1q.cpu(), w1s.cpu(), ids[sel], cfg.inter_dim)
    a2q, a2s = orc.requant(o1)
    ref = orc.stage2(a2q, a2s, w2q.cpu(), w2s.cpu(), ids[sel], tw[sel], H)
    got = out[sel.to(dev)].float().cpu()
    oracle_ok = bool(((got - ref).abs() <= 2e-2 + 2e-2 * ref.abs()).all())
    q.put((rank, bool(torch.equal(out, want)), bool(torch.equal(out, out2)), oracle_ok, _lib.device_status(),
           layer.last_plan.rows_in, ops.peers.kind if fused else "nccl"))


@pytest.mark.parametrize("world,routing,chunks", [(2, "uniform", 1), (2, "zipf", 3), (4, "uniform", 2),
                                                  (8, "zipf", 4)])
def test_expert_parallel_matches_single_gpu(world, routing, chunks):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, found {torch.cuda.device_count()}")
    port = _free_port()
    res = _run_ranks(world, lambda r, q: (r, world, port, routing, chunks, q))
    total_rows = 0
    for rank, same_as_single, repeatable, oracle_ok, status, rows_in, _kind in res:
        assert status == 0, f"rank {rank}: device-side timeout reported"
        assert same_as_single, f"rank {rank}: expert-parallel output differs from the single-GPU layer"
        assert repeatable and oracle_ok
        total_rows += rows_in
    assert total_rows == world * 300 * 4          # every dispatched row was received exactly once


@pytest.mark.parametrize("world,routing,direct", [(1, "zipf", False), (1, "uniform", "host"), (1, "zipf", "device"),
                                                  (2, "uniform", False), (2, "zipf", "host"), (4, "zipf", False),
                                                  (4, "uniform", "device"), (8, "uniform", False),
                                                  (8, "zipf", "host"), (8, "uniform", "device")])
def test_fused_combine_matches_single_gpu(world, routing, direct):
    """Stage 2 stores the expert outputs straight into the owning ranks' buffers (peer stores from the
    GEMM epilogue, no combine all-to-all); with ``direct`` the dispatch, too, is peer stores, into the
    owners' stage-1 operand buffers at final sorted positions.  Same bits as the single-GPU layer,
    twice in a row.  The one-rank cases run the same kernels and bookkeeping with every row staying
    on the GPU, so a single-GPU box covers them too.  ``direct`` = "host" plans the step on the host
    (capacity checked with an exception), "device" with tensor operations on the GPU (no host round
    trip in the step)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, found {torch.cuda.device_count()}")
    port = _free_port()
    res = _run_ranks(world, lambda r, q: (r, world, port, routing, 1, q, True, direct))
    kinds = {r[6] for r in res}
    assert kinds == {"symmetric_memory"}
    for rank, same_as_single, repeatable, oracle_ok, status, rows_in, _kind in res:
        assert status == 0, f"rank {rank}: device-side timeout reported"
        assert same_as_single, f"rank {rank}: fused-combine output differs from the single-GPU layer"
        assert repeatable and oracle_ok
