"""``load_extension()`` with the reference's contract (``kernels/w4a8/loader.py:13-35``): cached,
exposes ``.cache_info()`` (``runtime_profile.py:36-44`` inspects it), raises without CUDA.  Nothing is
JIT-compiled here: the handle is the prebuilt ``libsq_b200.so``."""
from __future__ import annotations

from functools import lru_cache

import torch

from ... import _lib


@lru_cache(maxsize=1)
def load_extension():
    if not torch.cuda.is_available():
        raise RuntimeError("The FastWAM W4A8 B200 backend requires CUDA.")
    return _lib.load_library()
