"""Operator modules with the reference's names: ``kernels.w4a8.ops`` and ``kernels.w4a4.wam_ops``."""
