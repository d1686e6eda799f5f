"""GPU parity of the helper kernels: weight (un)shuffle, row gather, top-k reduce."""
import numpy as np
import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200.kernels import moe_blockscale_2stage as bs
from oracle import moe_oracle as orc
from tests import helpers as hp

pytestmark = pytest.mark.gpu


def test_shuffle_weight_matches_reference_layout():
    g = hp.load("quant_shuffle.npz")
    w = hp.fp8_from_u8(g["w"]).cuda()
    E, N, K = w.shape
    shuf = bs.shuffle_weight(w, E * N, K)
    assert np.array_equal(hp.u8(shuf).reshape(E, N, K), g["w_shuffled"])
    assert np.array_equal(hp.u8(bs.unshuffle_weight(shuf, E * N, K)).reshape(E, N, K), g["w"])
    big = torch.randint(0, 255, (3, 256, 1024), dtype=torch.uint8)
    s2 = bs.shuffle_weight(big.cuda(), 3 * 256, 1024)
    assert torch.equal(s2.cpu().view(3, 256, 1024), orc.shuffle_weight(big))
    assert torch.equal(bs.unshuffle_weight(s2, 3 * 256, 1024).cpu().view(3, 256, 1024), big)
    # two-byte elements (fixture made by the reference's own shuffle on bf16 weights)
    w16 = torch.from_numpy(g["w16"]).view(torch.bfloat16).cuda()
    E, N, K = w16.shape
    shuf16 = bs.shuffle_weight(w16, E * N, K)
    assert np.array_equal(shuf16.view(torch.int16).cpu().numpy().reshape(E, N, K), g["w16_shuffled"])
    assert torch.equal(bs.unshuffle_weight(shuf16, E * N, K).view(E, N, K).view(torch.int16), w16.view(torch.int16))
    big16 = torch.randint(-30000, 30000, (2, 128, 512), dtype=torch.int16).view(torch.float16)
    s3 = bs.shuffle_weight(big16.cuda(), 2 * 128, 512)
    assert torch.equal(s3.cpu().view(2, 128, 512).view(torch.int16), orc.shuffle_weight(big16).view(torch.int16))


@pytest.mark.parametrize("T,k,D,dt,masked", [(1, 6, 5120, "f16", False), (5, 8, 7168, "bf16", False),
                                             (65, 8, 7168, "bf16", True), (129, 6, 5120, "f32", True),
                                             (33, 2, 136, "f16", False)])
def test_moe_reduce(T, k, D, dt, masked):
    td = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dt]
    g = torch.Generator().manual_seed(T + k)
    x = torch.randn((T, k, D), generator=g).to(td)
    mask = (torch.rand((T, k), generator=g) < 0.7).to(torch.uint8) if masked else None
    red = bs.compile_moe_reduction(topk=k, model_dim=D, dtype_str=dt, use_mask=masked)
    y = torch.empty((T, D), dtype=td, device="cuda")
    m = mask.cuda() if masked else torch.empty((0, k), dtype=torch.uint8, device="cuda")
    red(x.cuda(), y, m, T, torch.cuda.current_stream())
    torch.cuda.synchronize()
    ref = orc.topk_reduce(x, mask)
    assert torch.allclose(y.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)   # the reference test's tolerance
    assert torch.allclose(y.cpu().float(), ref.float(), rtol=2e-3 if dt != "f32" else 1e-5, atol=1e-5)


def test_gather_rows():
    T, k, H = 20, 3, 256
    src = torch.randint(0, 255, (T, H), dtype=torch.uint8, device="cuda")
    pair = torch.randint(0, 255, (T * k, H), dtype=torch.uint8, device="cuda")
    ids = torch.tensor([(1 << 24) | 5, (0 << 24) | 19, (k << 24) | T, (2 << 24) | 0, (1 << 24) | 7],
                       dtype=torch.int32, device="cuda")
    nv = torch.tensor([4, T], dtype=torch.int32, device="cuda")
    lib = _lib.load()
    for layout, s in ((_lib.ROWS_BY_TOKEN, src), (_lib.ROWS_BY_PAIR, pair)):
        dst = torch.full((8, H), 9, dtype=torch.uint8, device="cuda")
        _lib.check(lib.flymoe_gather_rows(s.data_ptr(), dst.data_ptr(), ids.data_ptr(), nv.data_ptr(), T, k, H,
                                          layout, 8, torch.cuda.current_stream().cuda_stream), "gather")
        torch.cuda.synchronize()
        pick = (lambda t, sl: s[t]) if layout == _lib.ROWS_BY_TOKEN else (lambda t, sl: s[t * k + sl])
        assert torch.equal(dst[0], pick(5, 1)) and torch.equal(dst[1], pick(19, 0)) and torch.equal(dst[3], pick(0, 2))
        assert int(dst[2].sum()) == 0                       # pad row zero-filled
        assert bool((dst[4:] == 9).all())                   # rows beyond the valid count untouched
