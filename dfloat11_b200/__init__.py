"""B200-native implementation of DFloat11's on-the-fly BF16 weight decompression path.

Importing the package loads ``libdf11.so`` (built in-tree by ``python -m dfloat11_b200.build``);
a missing or stale library is an ImportError -- there is no CPU or pure-PyTorch fallback.
"""
from . import _lib  # noqa: F401  (fails loudly when the native library is absent)
from .codec import UnrepresentableError, encode_weights, get_codec, get_luts, split_bf16, validate_unit
from .dfloat11 import (DFloat11Model, TensorManager, check_status, compress_in_place, compress_model, get_hook,
                       get_no_split_classes, load_and_replace_tensors, stats)
from . import ops  # noqa: F401
from .generation import GraphedGreedyDecoder
from .ops import (aux_bytes, decode, decode_prepared, decode_range_prepared, decode_rows_prepared, gemv_prepared,
                  prepare, seek_interval)

__all__ = [
    "DFloat11Model", "TensorManager", "compress_in_place", "compress_model", "get_hook", "get_no_split_classes",
    "load_and_replace_tensors", "check_status", "stats",
    "UnrepresentableError", "encode_weights", "get_codec", "get_luts", "split_bf16", "validate_unit",
    "aux_bytes", "decode", "decode_prepared", "decode_range_prepared", "decode_rows_prepared", "gemv_prepared",
    "prepare", "seek_interval", "ops",
    "GraphedGreedyDecoder",
]
