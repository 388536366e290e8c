"""Integration boundaries of :mod:`ue5m3_fp4` with training frameworks."""
