"""Drop-in operator surface of the reference's ``kernels`` package for the FP8
block-scaled fused-MoE path: same module names, function names and call
signatures (torch tensors in and out), backed by hand-written sm_100a CUDA."""
