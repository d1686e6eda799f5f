"""Import-path shim: ``kernels.moe_gemm_2stage`` resolves to the B200 implementation, so code
written against the reference's ``kernels`` package runs unchanged."""
from flydsl_b200.kernels.moe_gemm_2stage import *  # noqa: F401,F403
from flydsl_b200.kernels import moe_gemm_2stage as _impl

globals().update({k: v for k, v in vars(_impl).items() if k.startswith("_") and not k.startswith("__")})
