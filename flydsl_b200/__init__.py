"""flydsl_b200 — B200-native (sm_100a) FP8 block-scaled fused-MoE path.

Host code is PyTorch (device memory, streams, torch.distributed); the kernels are
hand-written CUDA behind the C ABI declared in ``include/flymoe.h``.  The package
mirrors the reference's ``kernels`` operator surface for this path
(``flydsl_b200.kernels.*``) and adds a fused layer (``flydsl_b200.layer``) and an
expert-parallel wrapper (``flydsl_b200.ep``).
"""

__version__ = "0.1.0"
