"""B200-native SiHC hyper-connection read/write path.

Importing this package loads the in-tree CUDA library (``csrc/libsihc_b200.so``)
and registers the ``sihc_b200::*`` operators.  It raises if the library has not
been built; there is no fallback implementation.
"""

from . import _lib
from .ops import (blockwise_read, blockwise_triangular, blockwise_write, sihc_read, sihc_write, sihc_write_read,
                  sublayer_read, sublayer_triangular, sublayer_write)

__all__ = [
    "sublayer_read", "sublayer_write", "sublayer_triangular",
    "blockwise_read", "blockwise_write", "blockwise_triangular",
    "sihc_read", "sihc_write", "sihc_write_read",
]
