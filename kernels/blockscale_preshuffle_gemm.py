"""Import-path shim: ``kernels.blockscale_preshuffle_gemm`` resolves to the B200 implementation, so code
written against the reference's ``kernels`` package runs unchanged."""
from flydsl_b200.kernels.blockscale_preshuffle_gemm import *  # noqa: F401,F403
from flydsl_b200.kernels.blockscale_preshuffle_gemm import compile_blockscale_preshuffle_gemm  # noqa: F401
