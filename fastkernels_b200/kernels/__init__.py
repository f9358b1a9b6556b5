"""Import-path mirror of the reference's `fastkernels.kernels` package (MoE functions only)."""
