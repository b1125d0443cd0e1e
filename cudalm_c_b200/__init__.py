"""B200-native QLM hot path of Dsg2/cudalm-c behind a C ABI (libqlm_b200.so).

The package is a thin host-side mirror of the reference's operator interface
(names and argument meaning follow qlm.cuh / cudalm.cu); all arithmetic runs in
hand-written sm_100a kernels inside the shared library.  There is no CPU or
PyTorch fallback: importing works anywhere, but every compute call needs the
library built (python -m cudalm_c_b200.build) and a CUDA device.
"""
from ._lib import lib, check, QlmbError, SPAN_DTYPE, lib_path  # noqa: F401
from . import qlm, moe, linear, q4n  # noqa: F401
