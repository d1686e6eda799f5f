"""Dense FP8 block-scaled GEMM (kernels.blockscale_preshuffle_gemm) against the CPU oracle.

Shapes and input recipe follow the reference's own test
(tests/kernels/test_blockscale_preshuffle_gemm.py:128-152, :208-212): DeepSeek-V3 projection sizes
with M from 1 to 1024, including M below the row block and M that is not a multiple of it, and the
2112-column weight whose last scale block holds 64 columns.  Bar:
the reference's rtol 1e-2 / atol 1e-2 on the 16-bit output."""
import pytest
import torch

from flydsl_b200 import _lib
from kernels.blockscale_preshuffle_gemm import compile_blockscale_preshuffle_gemm
from kernels.moe_blockscale_2stage import shuffle_weight
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _tile_m(M):
    return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128


def _case(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand((M, K), generator=g) / 10).to(torch.float16).to(FP8)
    w = (torch.rand((N, K), generator=g) / 10).to(torch.float16).to(FP8)
    x_scale = torch.rand((M, K // 128), generator=g)
    w_scale = torch.rand(((N + 127) // 128, K // 128), generator=g)
    return x, w, x_scale, w_scale


@pytest.mark.parametrize("N,K", [(7168, 2304), (2112, 7168), (3072, 1536), (1280, 7168), (1408, 512), (192, 256)])
@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 256, 1024])
def test_dense_blockscale_gemm_matches_oracle(M, N, K):
    dev = torch.device("cuda", 0)
    x, w, x_scale, w_scale = _case(M, N, K, 1000 + M)
    ref = orc.blockscale_gemm(x, x_scale, w, w_scale)
    d_x, d_w = x.to(dev), w.to(dev)
    d_sa = x_scale.t().contiguous().view(-1).to(dev)              # transposed [K/128, M], flattened
    d_sb = w_scale.contiguous().view(-1).to(dev)
    b_shuffled = shuffle_weight(d_w, N, K)                         # the reference's weight order
    for out_dtype, td in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        exe = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=_tile_m(M), tile_n=128, tile_k=128,
                                                 out_dtype=out_dtype)
        c = torch.full((M + 2, N), 7.0, dtype=td, device=dev)     # two canary rows behind the output
        for _ in range(2):                                         # the routing workspace is reused
            exe(c.view(-1), d_x.view(-1), b_shuffled, d_sa, d_sb, M, N, torch.cuda.current_stream())
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        got = c[:M].float().cpu()
        bad = (got - ref).abs() > 1e-2 + 1e-2 * ref.abs()
        assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} elements off (max {float((got - ref).abs().max())})"
        assert bool((c[M:] == 7.0).all()), "rows behind the output were written"
    # row-major weights give the same bits as the preshuffled ones
    exe_plain = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=_tile_m(M), tile_n=128, tile_k=128,
                                                   out_dtype="fp16", w_layout="plain")
    c2 = torch.empty((M, N), dtype=torch.float16, device=dev)
    exe_plain(c2, d_x, d_w, d_sa, d_sb, M, N)
    torch.cuda.synchronize()
    assert torch.equal(c2, c[:M])
