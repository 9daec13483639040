"""candy_b200 -- B200-native block-quantized (Q4_0 / Q8_0) matmul for gocnn/candy.

``libcandyq.so`` (CUDA, sm_100a, C ABI in ``include/candyq.h``) is the product; this
package is its Python binding plus a mirror of candy's device/storage interface used by
the tests and the benchmark.  Importing :mod:`candy_b200.backend` loads the library and
fails if it has not been built.
"""
from .abi import (ACT_F16, ACT_F32, ACT_Q8_1, ORDER_GGML_SPLIT, ORDER_GO_INTERLEAVED, Q4_0, Q8_0, CandyqError)

__all__ = ["ACT_F16", "ACT_F32", "ACT_Q8_1", "ORDER_GGML_SPLIT", "ORDER_GO_INTERLEAVED", "Q4_0", "Q8_0", "CandyqError"]
