"""B200-native quantized-linear path of FastWAM SteerQuant.

The folder name carries a hyphen, so the package is imported under the alias
``fastwamjoint_quantization_b200`` (see ``load_package`` in the repository's
``__graft_entry__.py``).  Layout:

* ``csrc/``                   hand-written sm_100a CUDA + the C ABI (``include/sq_b200.h``)
* ``_lib.py`` / ``native.py`` ctypes binding and tensor-level wrappers
* ``kernels/w4a8/ops.py``, ``kernels/w4a4/wam_ops.py``  the reference's operator API
* ``runtime.py`` ...          ``WAMQuantLinear`` and friends, same names as the reference
"""
__all__ = ["native"]
