"""Quantization tools (the counterpart of onnxruntime/python/tools/quantization): dynamic and static (QDQ) int8 with
min-max / entropy / percentile calibration, block-wise 4-bit weights (MatMulNBits) and NF4 / FP4 weights (MatMulBnb4)."""
from .matmul_bnb4_quantizer import MatMulBnb4Quantizer, dequantize_bnb4, quantize_bnb4  # noqa: F401
from .matmul_nbits_quantizer import MatMulNBitsQuantizer, quantize_blockwise, quantize_blockwise_gptq, quantize_blockwise_hqq, dequantize_blockwise  # noqa: F401
from .quantize import (  # noqa: F401
    CalibrationDataReader, CalibrationMethod, EntropyCalibrator, HistogramCalibrator, MinMaxCalibrator, PercentileCalibrator, QuantFormat,
    QuantType, quantize_dynamic, quantize_static, quantize_weight,
)
