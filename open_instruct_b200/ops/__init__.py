"""Operators: ``ref`` (plain PyTorch oracles) and ``fused`` (sm_100a kernels via ``lib``)."""
