"""The device status word: a bounded wait that really runs out, and a misaligned per-row destination.
Neither case faults, traps or hangs the GPU: the wait is given a limit of a millisecond on a barrier that
nobody arrives at and then returns; the misaligned row is dropped before any store is issued.  The
status word reads the code once, 0 afterwards, and the context stays usable (a normal layer call passes)."""
import time

import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200 import workloads as wl
from flydsl_b200.layer import FusedMoEBlockscale
from oracle import moe_oracle as orc
from tests.gpu_common import Problem, assert_close

pytestmark = pytest.mark.gpu
SMALL = wl.MoEConfig("status-small", 200, 512, 256, 8, 2, 21)


def run_small_layer():
    p = Problem(SMALL)
    layer = FusedMoEBlockscale(p.d_w1q, p.d_w1s, p.d_w2q, p.d_w2s, SMALL.topk, max_tokens=SMALL.tokens, tile_m=128)
    out = layer(p.d_logits, p.d_xq, p.d_xs_t)
    torch.cuda.synchronize()
    ref = orc.moe_layer(p.logits, p.xq, p.xs, p.w1q, p.w1s, p.w2q, p.w2s, SMALL.topk)
    assert_close(out[: SMALL.tokens], ref["out"], 2e-2, 2e-2, "layer after a reported status")


def test_bounded_wait_runs_out_and_reports_once():
    lib = _lib.load()
    assert _lib.device_status() == 0
    t0 = time.perf_counter()
    _lib.check(lib.flymoe_selftest_bounded_wait(1_000_000, torch.cuda.current_stream().cuda_stream), "selftest")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0, "the 1 ms wait must give up at once, not after the kernels' 4 s limit"
    assert _lib.device_status() == _lib.STATUS_SELFTEST_TIMEOUT
    assert _lib.device_status() == 0, "reading the status word clears it"
    run_small_layer()
    assert _lib.device_status() == 0


def test_misaligned_row_destination_is_dropped_and_reported():
    cfg = wl.MoEConfig("rows-misaligned", 64, 512, 256, 4, 1, 23)
    dev = torch.device("cuda", 0)
    w1q, w1s, w2q, w2s = wl.make_weights(cfg, device=dev)
    T, H, E = cfg.tokens, cfg.model_dim, cfg.experts
    _x, xq_c, xs_c = wl.make_activations(cfg)
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, E, (T, 1), generator=g, dtype=torch.int32).to(dev)
    ones = torch.ones((T, 1), dtype=torch.float32, device=dev)
    layer = FusedMoEBlockscale(w1q, w1s, w2q, w2s, 1, max_tokens=T, tile_m=128, stage2_mode="rows")
    s = torch.cuda.current_stream().cuda_stream
    plain = layer.experts_forward(ids, ones, xq_c.to(dev), xs_c.to(dev), T, s, x_scale_row_major=True).clone()
    target = torch.full((T + 1, H), -7.0, dtype=torch.bfloat16, device=dev)
    dst = target.data_ptr() + torch.arange(T, dtype=torch.int64) * (H * 2)
    dst[5] += 2                                             # not 16-byte aligned: this row must not be stored
    layer.experts_forward(ids, ones, xq_c.to(dev), xs_c.to(dev), T, s, x_scale_row_major=True, row_dst=dst.to(dev))
    torch.cuda.synchronize()
    assert _lib.device_status() == _lib.STATUS_ROW_DST_MISALIGNED
    assert _lib.device_status() == 0
    got = target[:T].cpu()
    keep = torch.ones(T, dtype=torch.bool)
    keep[5] = False
    assert torch.equal(got[keep], plain.cpu()[keep])
    assert bool((target[5] == -7.0).all()), "the misaligned row was dropped, nothing was written"
    assert bool((target[T] == -7.0).all())


def test_dispatch_rows_drops_rows_of_a_misaligned_destination():
    """flymoe_dispatch_rows with one expert's destination address off by 4 bytes: that expert's rows are
    not stored (the 16-byte stores would fault), the others are, and the status word reports it once."""
    lib = _lib.load()
    T, k, H, E = 8, 1, 256, 2
    dev = "cuda"
    x = torch.arange(T * H, dtype=torch.int32).remainder(251).to(torch.uint8).view(T, H).to(dev)
    xs = torch.arange(T * (H // 128), dtype=torch.float32).view(T, H // 128).to(dev)
    s_ids = torch.arange(T, dtype=torch.int32, device=dev)                 # slot 0 of token r
    s_e = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1], dtype=torch.int32, device=dev)
    nv = torch.tensor([T, T], dtype=torch.int32, device=dev)
    out_x = torch.full((T + 1, H), 0xEE, dtype=torch.uint8, device=dev)
    out_s = torch.full((T + 1, H // 128), -1.0, dtype=torch.float32, device=dev)
    dst_x = torch.tensor([out_x.data_ptr(), out_x.data_ptr() + 4], dtype=torch.int64, device=dev)   # expert 1: misaligned
    dst_s = torch.tensor([out_s.data_ptr(), out_s.data_ptr()], dtype=torch.int64, device=dev)
    _lib.check(lib.flymoe_dispatch_rows(x.data_ptr(), xs.data_ptr(), s_ids.data_ptr(), s_e.data_ptr(), nv.data_ptr(),
                                        dst_x.data_ptr(), dst_s.data_ptr(), None, 0, T, k, H, E, T,
                                        torch.cuda.current_stream().cuda_stream), "dispatch_rows")
    torch.cuda.synchronize()
    assert _lib.device_status() == _lib.STATUS_ROW_DST_MISALIGNED
    assert _lib.device_status() == 0
    assert torch.equal(out_x[:4].cpu(), x[:4].cpu()) and torch.equal(out_s[:4].cpu(), xs[:4].cpu())
    assert bool((out_x[4:] == 0xEE).all()) and bool((out_s[4:] == -1.0).all())
