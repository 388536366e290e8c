"""Kernel backends of :mod:`ue5m3_fp4` (one: hand-written sm_100a CUDA)."""
