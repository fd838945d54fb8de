from .ops import pack_signed_int4  # noqa: F401  (reference: kernels/w4a8/__init__.py)
