"""Weight-only quantization tools (the counterpart of onnxruntime/python/tools/quantization)."""
from .matmul_nbits_quantizer import MatMulNBitsQuantizer, quantize_blockwise, dequantize_blockwise  # noqa: F401
from .quantize import MinMaxCalibrator, quantize_dynamic, quantize_static, quantize_weight  # noqa: F401
