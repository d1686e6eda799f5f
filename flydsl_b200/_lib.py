"""ctypes binding of libflymoe_sm100.so (declarations mirror include/flymoe.h).

There is no fallback: if the shared library is missing, loading raises with the
build command; every wrapper raises ``RuntimeError`` when the C call reports an
error.  Tensors cross the boundary as raw device pointers plus explicit sizes.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_uint8, c_void_p, POINTER
from pathlib import Path

import torch

LIB_NAME = "libflymoe_sm100.so"
# FLYMOE_LIB overrides the path (e.g. an instrumented build of the same sources).
LIB_PATH = Path(os.environ.get("FLYMOE_LIB", Path(__file__).resolve().parent / LIB_NAME))

F32, F16, BF16, E4M3, I8 = 0, 1, 2, 3, 4
SCALE_BLOCK128, SCALE_PER_TOKEN = 0, 1
STATUS_DISPATCH_OVERFLOW, STATUS_ROW_DST_MISALIGNED, STATUS_SELFTEST_TIMEOUT = 16, 17, 99
ROWS_BY_TOKEN, ROWS_BY_PAIR, ROWS_SORTED, ROWS_BY_SLOT = 0, 1, 2, 3
IMPL_TCGEN05, IMPL_SIMT = 0, 1

DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16,
              torch.float8_e4m3fn: E4M3, torch.uint8: E4M3, torch.int8: I8}

_P = c_void_p
_SIGNATURES = {
    "flymoe_abi_version": (c_int, []),
    "flymoe_error_string": (c_char_p, [c_int]),
    "flymoe_last_error": (c_char_p, []),
    "flymoe_device_status": (c_int, [POINTER(c_int)]),
    "flymoe_topk_gating_softmax": (c_int, [_P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "flymoe_moe_sorting_workspace_elems": (c_int64, [c_int, c_int, c_int, c_int]),
    "flymoe_moe_sorting": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, _P, _P, c_int64,
                                   c_int, c_int, c_int, c_int, _P]),
    "flymoe_moe_sorting_noalloc_max_elems": (c_int64, []),
    "flymoe_moe_sorting_noalloc": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, _P,
                                           c_int, c_int, c_int, c_int, _P]),
    "flymoe_gather_rows": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "flymoe_moe_gemm1": (c_int, [_P, _P, c_int64, _P, _P, c_int64, c_int64, _P, _P, _P, _P, _P, _P,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_int, _P]),
    "flymoe_moe_gemm2": (c_int, [_P, _P, _P, c_int64, _P, _P, _P, _P, _P, _P,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_int, _P]),
    "flymoe_moe_gemm1_pertoken": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_int, _P]),
    "flymoe_moe_gemm2_pertoken": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_int, _P]),
    "flymoe_selftest_bounded_wait": (c_int, [c_int64, _P]),
    "flymoe_moe_gemm2_scatter_rows": (c_int, [_P, _P, _P, c_int64, _P, _P, _P, _P, _P, _P,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                              c_int, c_int, _P]),
    "flymoe_dispatch_rows": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, _P]),
    "flymoe_expert_counts": (c_int, [_P, _P, _P, c_int, c_int, _P]),
    "flymoe_ep_plan_workspace_elems": (c_int64, [c_int, c_int]),
    "flymoe_ep_plan_direct": (c_int, [_P, _P, c_int64, c_int64, c_int64, _P, _P, _P, _P, _P, _P, _P, _P, c_int64,
                                      c_int, c_int, c_int, c_int, c_int, c_int64, _P]),
    "flymoe_blockscale_gemm_workspace_elems": (c_int64, [c_int, c_int]),
    "flymoe_blockscale_gemm": (c_int, [_P, _P, _P, c_int64, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, _P]),
    "flymoe_set_gemm_cta_limit": (c_int, [c_int]),
    "flymoe_moe_reduce": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "flymoe_sorted_inverse": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P]),
    "flymoe_quant_act_1x128": (c_int, [_P, c_int, _P, _P, c_int64, c_int, c_int, _P]),
    "flymoe_shuffle_weight": (c_int, [_P, _P, c_int64, c_int, c_int, _P]),
    "flymoe_shuffle_weight_elems": (c_int, [_P, _P, c_int64, c_int, c_int, c_int, _P]),
    "flymoe_unpack_int4_weight": (c_int, [_P, _P, c_int64, c_int, c_int, _P]),
    "flymoe_unpack_int4_weight_grouped": (c_int, [_P, _P, c_int64, c_int, c_int, _P, c_int, c_int, c_int, _P]),
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_NAME} is missing at {LIB_PATH}: build it with `python -m flydsl_b200.build` "
            "(this package has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.flymoe_abi_version() != 1:
        raise RuntimeError("libflymoe_sm100.so has an unexpected ABI version; rebuild it")
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = load()
        kind = lib.flymoe_error_string(rc).decode()
        detail = lib.flymoe_last_error().decode()
        raise RuntimeError(f"{what}: {kind}: {detail}")


def device_status() -> int:
    """Synchronise and return (then clear) the device status word; 0 means healthy."""
    v = c_int(0)
    check(load().flymoe_device_status(ctypes.byref(v)), "flymoe_device_status")
    return v.value


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_handle(stream) -> int:
    """None -> current torch stream; int -> raw handle; else object with .cuda_stream."""
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


def require_cuda(name: str, t: torch.Tensor, dtypes=None, min_numel: int | None = None) -> None:
    """Host-side argument check; raises before anything is launched."""
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (got device {t.device})")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {tuple(dtypes)}")
    if min_numel is not None and t.numel() < min_numel:
        raise ValueError(f"{name} has {t.numel()} elements, needs at least {min_numel}")
