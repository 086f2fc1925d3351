"""B200-native build of the triton-rs LLM-decode kernel hot path.

The product is `libb200_kernels.so` (CUDA, sm_100a) behind the C ABI declared in
include/b200_kernels.h.  This package only loads it (`lib()`), mirrors the reference
prelude over torch-owned device memory (`prelude`), and holds the build recipe
(`build`).  It contains no arithmetic of its own and no fallback path.
"""
from ._lib import B200KError, Library, lib, parse_header  # noqa: F401
from . import prelude  # noqa: F401
from .layer import Comm, DecodeLayer, LayerShape, shard_columns, shard_layer_weights, shard_rows  # noqa: F401
