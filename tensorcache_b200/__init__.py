"""tensorcache_b200: the AMO-BQ feature-cache hot path of TensorCache on NVIDIA B200.

Drop-in for the reference's API on that path -- ``compress`` / ``decompress``,
``BlockwiseInt8Codec``, ``quantize_int8_amo_bq`` / ``dequantize_int8_amo_bq``, the symmetric
``quantize_int8_g32`` / ``quantize_int8_adaptive`` / ``dequantize_int8_g32``,
``FusedDequantLinear``, ``ZeroCopyTensorStreamer``, ``FeatureCacheWriter`` /
``FeatureCacheDataset`` -- on hand-written sm_100a CUDA kernels behind a C ABI
(``include/tcb200.h``, ``libtcb200.so``).  There is no Triton, no backend switch
and no CPU implementation: without the built library or a CUDA device the
compute calls raise.
"""
from .codec import (AMO_BQ_PRESETS, BlockwiseInt8Codec, dequantize_int8_amo_bq, dequantize_int8_g32,
                    quantize_int8_adaptive, quantize_int8_amo_bq, quantize_int8_g32)
from .feature_cache import FeatureCacheDataset, FeatureCacheWriter
from .fused_linear import FusedDequantLinear, fused_dequant_matmul
from .streamer import ZeroCopyTensorStreamer
from .utils import auto_select_mode, benchmark_tensor, compress, decompress, estimate_compression, selftest_sum_order

__version__ = "0.1.0"
__all__ = [
    "AMO_BQ_PRESETS", "BlockwiseInt8Codec", "quantize_int8_amo_bq", "dequantize_int8_amo_bq",
    "quantize_int8_g32", "quantize_int8_adaptive", "dequantize_int8_g32",
    "compress", "decompress", "estimate_compression", "benchmark_tensor", "auto_select_mode", "selftest_sum_order",
    "FusedDequantLinear", "fused_dequant_matmul",
    "FeatureCacheWriter", "FeatureCacheDataset", "ZeroCopyTensorStreamer",
]
