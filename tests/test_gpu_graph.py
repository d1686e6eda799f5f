"""The path under CUDA-graph capture, as the reference tests it for its sort
(tests/kernels/test_moe_sorting.py:686-718) and its dense GEMM (the ``graph`` variant of
tests/kernels/test_blockscale_preshuffle_gemm.py:155-161): calls only enqueue work on the given
stream -- no synchronisation, no allocation -- so a captured step can be replayed on new inputs."""
import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200 import workloads as wl
from flydsl_b200.layer import FusedMoEBlockscale
from kernels.blockscale_preshuffle_gemm import compile_blockscale_preshuffle_gemm

pytestmark = pytest.mark.gpu


def test_fused_layer_replays_from_a_cuda_graph():
    cfg = wl.MoEConfig("graph", 300, 512, 256, 16, 4, 31)
    dev = torch.device("cuda", 0)
    w1q, w1s, w2q, w2s = wl.make_weights(cfg, device=dev)
    layer = FusedMoEBlockscale(w1q, w1s, w2q, w2s, cfg.topk, max_tokens=cfg.tokens, tile_m=64,
                               stage2_mode="reduce")                # deterministic summation order
    inputs = []
    for r in range(3):
        _x, xq, xs = wl.make_activations(cfg, rank=r)
        inputs.append((wl.make_logits(cfg, rank=r).to(dev), xq.to(dev), xs.t().contiguous().to(dev)))
    eager = [layer(*inp).clone() for inp in inputs]
    torch.cuda.synchronize()
    assert not torch.equal(eager[0], eager[1])

    s_logits, s_xq, s_xs = (t.clone() for t in inputs[0])           # static input buffers of the graph
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(s_logits, s_xq, s_xs)                                 # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer(s_logits, s_xq, s_xs)
    for r in (1, 2, 0, 1):
        for dst, src in zip((s_logits, s_xq.view(torch.uint8), s_xs), inputs[r]):
            dst.copy_(src.view(torch.uint8) if src.dtype == torch.float8_e4m3fn else src)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager[r]), f"replay on input set {r} differs from the eager result"
    assert _lib.device_status() == 0


def test_dense_gemm_replays_from_a_cuda_graph():
    M, N, K = 200, 1536, 1024
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    xs = [(torch.rand((M, K), generator=g) / 10).to(torch.float16).to(torch.float8_e4m3fn).to(dev) for _ in range(2)]
    w = (torch.rand((N, K), generator=g) / 10).to(torch.float16).to(torch.float8_e4m3fn).to(dev)
    sa = torch.rand((K // 128, M), generator=g).to(dev)
    sb = torch.rand((N // 128, K // 128), generator=g).to(dev)
    exe = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=128, tile_n=128, tile_k=128, w_layout="plain")
    eager = []
    for x in xs:
        c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        exe(c, x, w, sa, sb, M, N)
        eager.append(c)
    torch.cuda.synchronize()
    x_static = xs[0].clone()
    c_static = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        exe(c_static, x_static, w, sa, sb, M, N, torch.cuda.current_stream())
    for r in (1, 0, 1):
        x_static.view(torch.uint8).copy_(xs[r].view(torch.uint8))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(c_static, eager[r])
    assert _lib.device_status() == 0
