"""Tolerances used by the parity tests.

default_tolerance mirrors the reference's table (src/fastkernels/testing/tolerances.py:8-18);
OUT_MAX_ABS / OUT_REL_L2 are the acceptance bounds of the benchmark definition for bf16
outputs against the fp32-accumulated oracle.
"""

OUT_MAX_ABS = 2e-2
OUT_REL_L2 = 5e-3


def default_tolerance(dtype):
    name = str(dtype).lower()
    if "float64" in name:
        return 1e-8, 1e-8
    if "float32" in name:
        return 1e-4, 1e-4
    if "bfloat16" in name:
        return 3e-2, 3e-2
    if "float16" in name:
        return 2e-2, 2e-2
    return 1e-4, 1e-4
