"""Import-path shim: ``kernels.topk_gating_softmax_kernel`` resolves to the B200 implementation, so code
written against the reference's ``kernels`` package runs unchanged."""
from flydsl_b200.kernels.topk_gating_softmax_kernel import *  # noqa: F401,F403
from flydsl_b200.kernels import topk_gating_softmax_kernel as _impl

globals().update({k: v for k, v in vars(_impl).items() if k.startswith("_") and not k.startswith("__")})
