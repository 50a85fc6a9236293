"""ferrum_b200: B200-native (sm_100a) K-quant dequantize-and-multiply behind Ferrum's quantized-linear
op surface.  All computation lives in ``libferrum_b200.so`` (CUDA); this package is the host-side
mirror of the reference interface over the C ABI."""
from ._lib import BF16, F32, Q4_K, Q6_K, Q8_0, LIB_PATH  # noqa: F401

__all__ = ["BF16", "F32", "Q4_K", "Q6_K", "Q8_0", "LIB_PATH", "surface", "build"]
