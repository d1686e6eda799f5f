"""Host-side boundary: the C-ABI library loads without a GPU and exports every declared
symbol; builders and launchers reject bad arguments before anything is launched."""
import re
from pathlib import Path

import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200.kernels import moe_blockscale_2stage as bs
from flydsl_b200.kernels.blockscale_preshuffle_gemm import compile_blockscale_preshuffle_gemm
from flydsl_b200.kernels import moe_gemm_2stage as pt
from flydsl_b200.kernels import moe_sorting_kernel as srt
from flydsl_b200.kernels import topk_gating_softmax_kernel as gat

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "flymoe.h").read_text()
    declared = set(re.findall(r"\b(flymoe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/flymoe.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in flymoe.h but not exported"
    assert declared == set(_lib.EXPORTED_SYMBOLS), "ctypes signature table and header disagree"
    assert lib.flymoe_abi_version() == 1
    assert lib.flymoe_error_string(-4).decode() == "workspace too small"


def test_workspace_size_is_host_only(lib):
    assert lib.flymoe_moe_sorting_workspace_elems(64, 256, 8, 32) == 0
    need = lib.flymoe_moe_sorting_workspace_elems(4096, 256, 8, 128)
    assert need == (4096 * 8 // 128) * 256 + 256
    assert srt.moe_sorting_get_workspace_size(4096, 256, 8, 128) >= need
    assert srt.moe_sorting_get_workspace_size(16, 256, 8) == 0


def test_c_abi_rejects_bad_arguments_without_launching(lib):
    rc = lib.flymoe_topk_gating_softmax(None, 0, None, None, None, 4, 4096, 2, 1, None)
    assert rc == -1 and b"num_experts" in lib.flymoe_last_error()
    rc = lib.flymoe_moe_sorting(None, None, None, None, None, None, None, 0, None, None, 0, 4, 8, 300, 32, None)
    assert rc == -1 and b"topk" in lib.flymoe_last_error()
    rc = lib.flymoe_moe_gemm1(None, None, 0, None, None, 0, 1, None, None, None, None, None, None,
                              4, 100, 256, 1, 2, 2, 128, 0, 2, 0, 0, 1, 0, None)
    assert rc == -1 and b"inter_dim" in lib.flymoe_last_error()
    rc = lib.flymoe_quant_act_1x128(None, 2, None, None, 0, 4, 100, None)
    assert rc == -1
    # the expert-parallel entry points
    rc = lib.flymoe_dispatch_rows(None, None, None, None, None, None, None, None, 0, 4, 2, 256, 8, 8, None)
    assert rc == -1 and b"null pointer" in lib.flymoe_last_error()
    rc = lib.flymoe_moe_gemm2_scatter_rows(None, None, None, 0, None, None, None, None, None, None,
                                           4, 256, 128, 1, 2, 1, 128, 0, 2, 2, 2, None)
    assert rc == -1 and b"row_dst" in lib.flymoe_last_error()
    rc = lib.flymoe_set_gemm_cta_limit(-1)
    assert rc == -1


def test_builder_value_errors_match_reference_rules():
    kw = dict(model_dim=1024, inter_dim=512, experts=8, topk=2, tile_m=128, tile_n=256, tile_k=128)
    with pytest.raises(ValueError, match="out_dtype"):
        bs.compile_moe_blockscale_gemm1(doweight_stage1=False, out_dtype="f32", **kw)
    with pytest.raises(ValueError, match="scale_block_k"):
        bs.compile_moe_blockscale_gemm1(doweight_stage1=False, **{**kw, "model_dim": 1000})
    with pytest.raises(ValueError, match="divisible by 128"):
        bs.compile_moe_blockscale_gemm1(doweight_stage1=False, **{**kw, "inter_dim": 96})
    with pytest.raises(ValueError, match="tile_k_bytes"):
        bs.compile_moe_blockscale_gemm2(doweight_stage2=True, **{**kw, "tile_k": 96})
    with pytest.raises(ValueError, match="accumulate=False"):
        bs.compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype="f32", accumulate=False, **kw)
    with pytest.raises(ValueError, match="out_dtype"):
        bs.compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype="int8", **kw)
    with pytest.raises(ValueError, match="Unsupported dtype"):
        bs.compile_moe_reduction(topk=2, model_dim=1024, dtype_str="i8")
    with pytest.raises(ValueError, match="FP8-only"):
        bs.compile_moe_blockscale_gemm2_ex(doweight_stage2=True, in_dtype="int8", **kw)
    with pytest.raises(ValueError):
        gat.build_topk_gating_softmax_module(8, 9)
    with pytest.raises(ValueError):
        gat.build_topk_gating_softmax_module(8, 2, "f64")
    # builders are cached like the reference's lru_cache'd ones
    a = bs.compile_moe_blockscale_gemm1(doweight_stage1=False, **kw)
    assert a is bs.compile_moe_blockscale_gemm1(doweight_stage1=False, **kw)
    assert bs.compile_moe_blockscale_gemm2_ex(doweight_stage2=True, mode=bs.MoeGemm2Mode.REDUCE, **kw).mode == "reduce"


def test_launchers_reject_cpu_tensors():
    launch = gat.build_topk_gating_softmax_module(8, 2, "f32")
    g = torch.zeros((4, 8))
    with pytest.raises(ValueError, match="CUDA tensor"):
        launch(g, torch.zeros(4, 2), torch.zeros(4, 2, dtype=torch.int32), torch.zeros(4, 2, dtype=torch.int32), 4)
    ids = torch.zeros((4, 2), dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA tensor"):
        srt.moe_sorting_flydsl(ids, torch.zeros(4, 2), ids, ids, ids, ids, None, 8)
    exe = bs.compile_moe_blockscale_gemm1(model_dim=256, inter_dim=128, experts=4, topk=2, tile_m=128, tile_n=128,
                                          tile_k=128, doweight_stage1=False)
    z = torch.zeros(16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        exe(z, z, z, z, z, z, z, z, z, 4, 128, 256, 1, None)
    with pytest.raises(ValueError, match="launcher built for"):
        exe(z, z, z, z, z, z, z, z, z, 4, 256, 256, 1, None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_dense_blockscale_gemm_argument_rules():
    kw = dict(M=64, K=2304, tile_m=64, tile_n=128, tile_k=128)
    with pytest.raises(ValueError, match="multiple of 64"):
        compile_blockscale_preshuffle_gemm(N=2080, **kw)
    compile_blockscale_preshuffle_gemm(N=2112, **kw)               # the reference's N = 64 mod 128 case builds
    with pytest.raises(ValueError, match="out_dtype"):
        compile_blockscale_preshuffle_gemm(N=7168, out_dtype="f32", **kw)
    with pytest.raises(ValueError, match="divisible by tile_k"):
        compile_blockscale_preshuffle_gemm(N=7168, **{**kw, "tile_k": 256, "K": 2304 + 128})
    exe = compile_blockscale_preshuffle_gemm(N=7168, **kw)
    z = torch.zeros(16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        exe(z, z, z, z, z, 4, 7168)
    with pytest.raises(ValueError, match="built for N"):
        exe(z, z, z, z, z, 4, 1024)


def test_pertoken_builder_rules(lib):
    base = dict(model_dim=256, inter_dim=128, experts=4, topk=2, tile_m=16, tile_n=64, tile_k=128)
    with pytest.raises(ValueError, match="group-wise"):
        pt.compile_moe_gemm1(doweight_stage1=False, in_dtype="int4", group_size=32, **base)
    with pytest.raises(ValueError, match="only supports group_size=32"):
        pt.compile_moe_gemm1(doweight_stage1=False, in_dtype="int4_bf16", group_size=64, **base)
    assert callable(pt.compile_moe_gemm1(doweight_stage1=False, in_dtype="int4_bf16", group_size=32, **base))
    with pytest.raises(ValueError, match="preshuffled order"):
        pt.compile_moe_gemm1(doweight_stage1=False, in_dtype="int4", w_layout="plain", **base)
    assert callable(pt.compile_moe_gemm2(doweight_stage2=True, in_dtype="int4", **base))
    with pytest.raises(ValueError, match="tensor-core path only"):
        pt.compile_moe_gemm1(doweight_stage1=False, in_dtype="bf16", impl="simt", **base)
    assert callable(pt.compile_moe_gemm1(doweight_stage1=False, in_dtype="fp16", **base))
    with pytest.raises(ValueError, match="in_dtype must be one of"):
        pt.compile_moe_gemm2(doweight_stage2=True, in_dtype="fp6", **base)
    with pytest.raises(ValueError, match="only supports out_dtype"):
        pt.compile_moe_gemm2(doweight_stage2=True, out_dtype="f32", accumulate=False, **base)
    assert callable(pt.compile_moe_gemm1(doweight_stage1=False, k_batch=2, **base))     # split-K output contract
    with pytest.raises(ValueError, match="not divisible by k_batch"):
        pt.compile_moe_gemm1(doweight_stage1=False, k_batch=3, **base)
    with pytest.raises(ValueError, match="not divisible by tile_k"):
        pt.compile_moe_gemm1(doweight_stage1=False, k_batch=4, **base)
    with pytest.raises(ValueError, match="bf16 partial sums"):
        pt.compile_moe_gemm1(doweight_stage1=False, k_batch=2, in_dtype="bf16", **base)
    assert pt.compile_moe_gemm2_ex(doweight_stage2=True, mode=pt.MoeGemm2Mode.REDUCE, in_dtype="int8", **base).mode == "reduce"
    import kernels.moe_gemm_2stage as shim                      # the reference's import path
    assert shim.compile_moe_gemm1 is pt.compile_moe_gemm1
    # C ABI: int8 operands only with per-token scaling, e4m3 output only with block scaling
    rc = lib.flymoe_moe_gemm1_pertoken(None, None, None, None, None, None, None, None, None,
                                       4, 128, 256, 1, 2, 2, 16, 0, _lib.I8, _lib.E4M3, 2, 0, 1, 0, None)
    assert rc == -1 and b"out_dtype" in lib.flymoe_last_error()
    rc = lib.flymoe_moe_gemm2_pertoken(None, None, None, None, None, None, None, None, None,
                                       4, 256, 128, 1, 2, 2, 16, 1, _lib.F32, _lib.F16, 1, 2, 1, 0, None)
    assert rc == -1 and b"in_dtype" in lib.flymoe_last_error()
    rc = lib.flymoe_moe_gemm2_pertoken(None, None, None, None, None, None, None, None, None,          # 16-bit operands:
                                       4, 256, 128, 1, 2, 2, 16, 1, _lib.BF16, _lib.F16, 1, 2, 1, 1, None)   # not in the SIMT kernel
    assert rc == -1 and b"tcgen05" in lib.flymoe_last_error()
    rc = lib.flymoe_selftest_bounded_wait(0, None)
    assert rc == -1 and b"limit_ns" in lib.flymoe_last_error()


def test_sorting_rejects_topk_above_expert_count(lib):
    rc = lib.flymoe_moe_sorting(None, None, None, None, None, None, None, 0, None, None, 0, 4, 8, 9, 32, None)
    assert rc == -1 and b"topk" in lib.flymoe_last_error()
    # the pair count is formed in 64 bits: no wrap-around for a huge (tokens, topk) product
    assert lib.flymoe_moe_sorting_workspace_elems((1 << 24) - 1, 1024, 255, 32) > (1 << 31)


def test_header_is_plain_c_and_a_c_program_links(tmp_path):
    """include/flymoe.h compiles as C99 and a C caller can link the shared library and use its
    host-only entry points (no torch, no Python in the call chain)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler on this machine")
    src = tmp_path / "caller.c"
    src.write_text(
        '#include <stdio.h>\n#include <string.h>\n#include "flymoe.h"\n'
        "int main(void) {\n"
        "  if (flymoe_abi_version() != 1) return 1;\n"
        '  if (strcmp(flymoe_error_string(-4), "workspace too small") != 0) return 2;\n'
        "  if (flymoe_moe_sorting_workspace_elems(4096, 256, 8, 128) != (4096 * 8 / 128) * 256 + 256) return 3;\n"
        "  /* argument validation happens before any CUDA call: a null pointer is an error code, not a crash */\n"
        "  if (flymoe_unpack_int4_weight(NULL, NULL, 16, 32, FLYMOE_I8, NULL) != -1) return 4;\n"
        '  printf("%s\\n", flymoe_last_error());\n'
        "  return 0;\n}\n")
    exe = tmp_path / "caller"
    lib_dir = Path(_lib.LIB_PATH).resolve().parent
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
                        "-L", str(lib_dir), "-l:" + Path(_lib.LIB_PATH).name, "-Wl,-rpath," + str(lib_dir)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, f"C caller returned {run.returncode}: {run.stderr}"
    assert "unpack_int4_weight" in run.stdout
