"""Top-level ``kernels`` package name used by the reference project; every module here
re-exports the B200 implementation from ``flydsl_b200.kernels``."""
