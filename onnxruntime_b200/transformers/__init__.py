"""Offline model tools (the counterpart of onnxruntime/python/tools/transformers): graph optimizer front end and
float16 conversion."""
from .float16 import convert_float_to_float16  # noqa: F401
from .optimizer import OptimizedModel, optimize_model  # noqa: F401
