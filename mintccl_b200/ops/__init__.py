"""Collective operations (module-level API), fused GEMM+collective ops and the LL128 layout oracle."""
