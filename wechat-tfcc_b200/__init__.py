"""B200-native matmul backend for TFCC: the hot path only.

Python face of ``libtfcc_b200.so``.  It mirrors the reference's operator
surface for this path -- ``blas.matmul`` (tfcc/core/operations/tfcc_blas.cpp),
``quantization.matmul`` / ``quantization.reduce_sum``
(tfcc/mkl/operations/tfcc_mklquantization.h) -- on torch CUDA tensors, which
serve purely as device-memory handles.  All arithmetic happens in the CUDA
library; there is no CPU or eager fallback, and importing an operator without
the built library raises.
"""
from . import exceptions  # noqa: F401
from ._lib import lib, library_path, launch_count  # noqa: F401
from . import blas, nn, quantization, parallel, session  # noqa: F401

__all__ = ["blas", "nn", "quantization", "parallel", "exceptions", "lib", "library_path", "launch_count"]
