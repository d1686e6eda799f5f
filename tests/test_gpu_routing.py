"""GPU parity of gating and sorting against the CPU oracle: indices, sorted ids and pad
counts are compared bit for bit.  Shapes follow the reference's own test lists
(tests/kernels/test_topk_gating_softmax.py:227-232, tests/kernels/test_moe_sorting.py:456-507,
:610-625) plus the DeepSeek-V3 routing shapes."""
import numpy as np
import pytest
import torch

from flydsl_b200.kernels.moe_sorting_kernel import moe_sorting_flydsl, moe_sorting_get_workspace_size
from flydsl_b200.kernels.topk_gating_softmax_kernel import build_topk_gating_softmax_module
from flydsl_b200 import workloads as wl
from oracle import moe_oracle as orc
from tests import helpers as hp

pytestmark = pytest.mark.gpu
DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def run_gating(logits_cpu, k, dtype_str, renorm=True):
    T, E = logits_cpu.shape
    launch = build_topk_gating_softmax_module(E, k, dtype_str, renorm)
    g = logits_cpu.cuda()
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    idx = torch.empty((T, k), dtype=torch.int32, device="cuda")
    tei = torch.empty((T, k), dtype=torch.int32, device="cuda")
    launch(g, w, idx, tei, T, stream=torch.cuda.current_stream())
    torch.cuda.synchronize()
    return w.cpu(), idx.cpu(), tei.cpu()


@pytest.mark.parametrize("T,E,k,dt", [
    (1024, 128, 6, "bf16"), (512, 64, 2, "bf16"), (256, 8, 2, "f32"), (128, 128, 6, "f16"),
    (64, 256, 8, "f32"), (4096, 256, 8, "f32"), (16384, 256, 8, "f32"), (7, 8, 2, "f32"),
    (1, 256, 8, "f32"), (33, 257, 9, "f32"), (5, 513, 9, "bf16"), (19, 1000, 32, "f32"), (3, 1, 1, "f32"),
])
@pytest.mark.parametrize("renorm", [True, False])
def test_gating_bit_exact_indices(T, E, k, dt, renorm):
    g = torch.Generator().manual_seed(1000 + T + E + k)
    logits = (torch.rand((T, E), generator=g) * 4.0 - 2.0).to(DT[dt])   # the reference test's distribution
    w, idx, tei = run_gating(logits, k, dt, renorm)
    rw, ridx, rtei = orc.topk_gating_softmax(logits, k, renorm)
    assert torch.equal(idx, ridx)
    assert torch.equal(tei, rtei)
    assert torch.allclose(w, rw, atol=1e-6, rtol=1e-5)
    if renorm:
        assert torch.allclose(w.sum(dim=1), torch.ones(T), atol=1e-5)


def test_gating_normal_logits_and_ties():
    cfg = wl.CONFIGS["c4b"]
    logits = wl.make_logits(cfg)
    w, idx, tei = run_gating(logits, cfg.topk, "f32")
    rw, ridx, _ = orc.topk_gating_softmax(logits, cfg.topk)
    assert torch.equal(idx, ridx) and torch.allclose(w, rw, atol=1e-6, rtol=1e-5)
    # exact ties: every logit equal -> experts 0..k-1 in order; two-valued rows -> lower ids first
    tied = torch.zeros((4, 64))
    tied[1, 10:] = 1.0
    tied[2, ::2] = 3.0
    tied[3, 63] = -1.0
    w, idx, _ = run_gating(tied, 4, "f32")
    _, ridx, _ = orc.topk_gating_softmax(tied, 4)
    assert torch.equal(idx, ridx)
    assert idx[0].tolist() == [0, 1, 2, 3] and idx[1].tolist() == [10, 11, 12, 13] and idx[2].tolist() == [0, 2, 4, 6]


def test_gating_golden():
    g = hp.load("gating.npz")
    for i in range(int(g["n"][0])):
        T, E, k, renorm = (int(v) for v in g[f"g{i}_cfg"])
        dt = str(g[f"g{i}_dtype"][0])
        logits = torch.from_numpy(g[f"g{i}_logits_f32"]).to(DT[dt])
        w, idx, _ = run_gating(logits, k, dt, bool(renorm))
        rows = torch.from_numpy(g[f"g{i}_distinct"])
        assert torch.equal(idx[rows], torch.from_numpy(g[f"g{i}_idx"])[rows])
        assert torch.allclose(w[rows], torch.from_numpy(g[f"g{i}_w"])[rows], atol=1e-6, rtol=1e-5)


# ------------------------------------------------------------------------------- sorting
def run_sort(ids, w, E, unit, mask=None, workspace="auto", H=64):
    T, k = ids.shape
    cap = T * k + E * unit - k
    nblk = (cap + unit - 1) // unit
    dev = "cuda"
    sorted_ids = torch.full((cap,), -7, dtype=torch.int32, device=dev)
    sorted_w = torch.full((cap,), -7.0, dtype=torch.float32, device=dev)
    sorted_e = torch.full((nblk,), -7, dtype=torch.int32, device=dev)
    nvalid = torch.full((2,), -7, dtype=torch.int32, device=dev)
    moe_buf = torch.full((max(T, 1), H), 3.0, dtype=torch.bfloat16, device=dev)
    ws = None
    if workspace == "given":
        n = moe_sorting_get_workspace_size(T, E, k, unit)
        ws = torch.full((max(n, 1),), 0x5A5A5A5A, dtype=torch.int32, device=dev)
    moe_sorting_flydsl(ids.cuda(), w.cuda(), sorted_ids, sorted_w, sorted_e, nvalid, moe_buf, E, unit,
                       None if mask is None else mask.cuda(), None, ws)
    torch.cuda.synchronize()
    return sorted_ids.cpu().numpy(), sorted_w.cpu().numpy(), sorted_e.cpu().numpy(), nvalid.cpu().numpy(), moe_buf


def check_sort(ids, w, E, unit, mask=None, workspace="auto"):
    a, b, c, d, buf = run_sort(ids, w, E, unit, mask, workspace)
    ra, rb, rc, rd = orc.moe_sorting(ids.numpy(), w.numpy(), E, unit, None if mask is None else mask.numpy())
    assert np.array_equal(d, rd), (d, rd)
    R = int(rd[0])
    assert np.array_equal(a[:R], ra[:R])
    assert np.array_equal(b[:R].view(np.int32), rb[:R].view(np.int32))    # weights moved as raw bits
    assert np.array_equal(c, rc)                                           # valid blocks and the -1 tail
    assert float(buf.float().abs().sum()) == 0.0
    # rows at or beyond the valid count are unspecified but must stay inside the buffers:
    a2, b2, c2, d2, _ = run_sort(ids, w, E, unit, mask, workspace)
    assert np.array_equal(a[:R], a2[:R]) and np.array_equal(c, c2) and np.array_equal(d, d2)
    return R


ONESHOT = [(T, 256, 8) for T in (1, 2, 4, 8, 16, 32, 64)] + [(1, 32, 5), (7, 32, 5), (31, 64, 6), (1, 257, 9),
                                                              (16, 257, 9), (16, 513, 9)]
MULTI = [(128, 256, 8), (512, 256, 8), (1024, 256, 8), (2048, 256, 8), (1024, 257, 9), (1024, 513, 9),
         (4096, 256, 8), (16384, 256, 8), (1025, 8, 2), (3000, 1000, 3)]


@pytest.mark.parametrize("T,E,k", ONESHOT + MULTI)
def test_sorting_bit_exact(T, E, k):
    if T <= 2048:
        ids, w, _ = hp.gen_sort_inputs(T, E, k, False)
    else:
        ids, w = hp.fast_sort_inputs(T, E, k, 42 + T)
    check_sort(ids, w, E, 32)


@pytest.mark.parametrize("unit", [16, 32, 64, 128])
@pytest.mark.parametrize("T,E,k", [(64, 256, 8), (777, 64, 6), (4096, 256, 8)])
def test_sorting_unit_sizes_and_workspace(T, E, k, unit):
    ids, w = hp.fast_sort_inputs(T, E, k, 7 + unit)
    check_sort(ids, w, E, unit, workspace="given")


@pytest.mark.parametrize("T,E,k", [(16, 32, 5), (64, 256, 8), (1024, 256, 8), (4096, 256, 8)])
def test_sorting_expert_mask(T, E, k):
    ids, w = hp.fast_sort_inputs(T, E, k, 99 + T)
    g = torch.Generator().manual_seed(5)
    for mask in [(torch.rand(E, generator=g) < 0.5).to(torch.int32),
                 (torch.arange(E) // (E // 4) == 1).to(torch.int32),       # one EP rank's contiguous shard
                 torch.zeros(E, dtype=torch.int32)]:
        check_sort(ids, w, E, 32, mask=mask)


def test_sorting_golden_and_skew():
    g = hp.load("sorting.npz")
    for i in range(int(g["n"][0])):
        T, E, k, unit, masked = (int(v) for v in g[f"c{i}_cfg"])
        mask = torch.from_numpy(g[f"c{i}_mask"]) if masked else None
        a, b, c, d, _ = run_sort(torch.from_numpy(g[f"c{i}_ids"]), torch.from_numpy(g[f"c{i}_w"]), E, unit, mask)
        R = int(g[f"c{i}_nvalid"][0])
        assert np.array_equal(d, g[f"c{i}_nvalid"])
        assert np.array_equal(a[:R], g[f"c{i}_sorted_ids"][:R])
        assert np.array_equal(b[:R], g[f"c{i}_sorted_w"][:R])
        assert np.array_equal(c, g[f"c{i}_sorted_e"])
    # Zipf-skewed routing from the gating kernel itself: a few experts huge, most tiny
    cfg = wl.CONFIGS["c4b"]
    logits = wl.make_logits(cfg)
    w, idx, _ = run_gating(logits, cfg.topk, "f32")
    R = check_sort(idx, w, cfg.experts, 128)
    assert R % 128 == 0
    # every token routed to expert 0 in slot 0 (maximal collision on one expert)
    ids = torch.stack([torch.arange(4, dtype=torch.int32) for _ in range(3000)])
    check_sort(ids, torch.rand(3000, 4), 16, 64)


def test_sorting_num_local_tokens_and_empty():
    ids, w = hp.fast_sort_inputs(40, 32, 4, 3)
    T, k, E, unit = 40, 4, 32, 32
    cap = T * k + E * unit - k
    out = [torch.zeros(cap, dtype=torch.int32, device="cuda"), torch.zeros(cap, dtype=torch.float32, device="cuda"),
           torch.zeros((cap + unit - 1) // unit, dtype=torch.int32, device="cuda"),
           torch.zeros(2, dtype=torch.int32, device="cuda")]
    buf = torch.ones((T, 8), dtype=torch.float16, device="cuda")
    moe_sorting_flydsl(ids.cuda(), w.cuda(), *out, buf, E, unit, None, torch.tensor(25), None)
    torch.cuda.synchronize()
    ra, rb, rc, rd = orc.moe_sorting(ids[:25].numpy(), w[:25].numpy(), E, unit)
    R = int(rd[0])
    assert out[3].cpu().tolist() == [R, 25]
    assert np.array_equal(out[0].cpu().numpy()[:R], ra[:R])
    nb = (25 * k + E * unit - k + unit - 1) // unit
    assert np.array_equal(out[2].cpu().numpy()[:nb], rc)
