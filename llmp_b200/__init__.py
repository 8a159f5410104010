"""llmp_b200: B200 (sm_100a) kernels for llmp's quantized matrix products.

The product is the C-ABI shared library built from ``llmp_b200/csrc`` and
declared in ``include/llmp_b200.h``.  This package is its host-side mirror for
Python callers: the reference's operator builders (``QuantizeQ8``, ``VecQ``,
... of src/kernels/ggml/llmp_ops.h) restated over torch device tensors.
PyTorch provides device memory, streams and torch.distributed only.
"""
from . import _native  # noqa: F401
from .ops import *  # noqa: F401,F403
