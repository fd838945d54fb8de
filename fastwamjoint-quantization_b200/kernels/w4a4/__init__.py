from ..w4a8.ops import pack_signed_int4  # noqa: F401  (reference: kernels/w4a4/__init__.py)
from . import wam_ops  # noqa: F401
