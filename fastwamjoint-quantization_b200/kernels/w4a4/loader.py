"""``load_extension()`` for the W4A4 operators (reference: ``kernels/w4a4/loader.py:13-67``).  Both
bit widths live in the same shared library."""
from __future__ import annotations

from functools import lru_cache

import torch

from ... import _lib


@lru_cache(maxsize=1)
def load_extension():
    if not torch.cuda.is_available():
        raise RuntimeError("The FastWAM W4A4 B200 backend requires CUDA.")
    return _lib.load_library()
