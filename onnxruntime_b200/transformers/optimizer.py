"""Offline front end of the graph optimizer: ``optimize_model(path_or_bytes, ...)`` applies the runtime's own
fusion passes (Attention, EmbedLayerNorm, SkipLayerNorm, BiasGelu, FastGelu, LayerNorm, MatMulNBits, ...) and returns
the fused model, as ``onnxruntime/python/tools/transformers/optimizer.py:optimize_model`` does with its Python
fusion stack.  Also a CLI: ``python -m onnxruntime_b200.transformers.optimizer --input m.onnx --output m_opt.onnx``.
"""
from __future__ import annotations

import argparse
from typing import Dict, Iterable, Optional, Union

from .. import _core as C
from .. import onnx_lite as ol

_FUSED_OPS = ("Attention", "MultiHeadAttention", "GroupQueryAttention", "EmbedLayerNormalization", "SkipLayerNormalization",
              "SkipSimplifiedLayerNormalization", "LayerNormalization", "SimplifiedLayerNormalization", "BiasGelu", "FastGelu",
              "Gelu", "QuickGelu", "MatMulNBits", "RotaryEmbedding", "FusedGemm", "GemmSwiGLU", "FusedMatMul")


class OptimizedModel:
    def __init__(self, model_bytes: bytes):
        self.model_bytes = model_bytes
        self.applied_passes = {}  # pass name -> number of rewrites

    @property
    def model(self) -> ol.Model:
        return ol.load_model(self.model_bytes)

    def get_fused_operator_statistics(self) -> Dict[str, int]:
        counts: Dict[str, int] = {}
        for n in C.model_nodes(self.model_bytes):
            if n["op_type"] in _FUSED_OPS:
                counts[n["op_type"]] = counts.get(n["op_type"], 0) + 1
        return counts

    def get_operator_statistics(self) -> Dict[str, int]:
        counts: Dict[str, int] = {}
        for n in C.model_nodes(self.model_bytes):
            counts[n["op_type"]] = counts.get(n["op_type"], 0) + 1
        return counts

    def is_fully_optimized(self) -> bool:
        s = self.get_fused_operator_statistics()
        return s.get("Attention", 0) + s.get("MultiHeadAttention", 0) + s.get("GroupQueryAttention", 0) > 0

    def save_model_to_file(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.model_bytes)

    def convert_float_to_float16(self, keep_io_types: bool = True) -> None:
        from .float16 import convert_float_to_float16
        self.model_bytes = convert_float_to_float16(self.model_bytes, keep_io_types=keep_io_types).serialize()


def optimize_model(input: Union[str, bytes], model_type: str = "bert", num_heads: int = 0, hidden_size: int = 0,
                   opt_level: Optional[int] = None, use_gpu: bool = False, disabled_optimizers: Iterable[str] = ()) -> OptimizedModel:
    """``opt_level``: 0 none, 1 basic, 2 extended, 99 all (default).  ``model_type`` / ``num_heads`` / ``hidden_size`` are
    accepted for call compatibility; the pattern matchers read head counts from the graph itself.  ``use_gpu`` adds
    the GPU-only lowering passes (GEMM epilogue fusion, SwiGLU, MatMul + AllReduce)."""
    if isinstance(input, str):
        with open(input, "rb") as f:
            input = f.read()
    level = 99 if opt_level is None else int(opt_level)
    out, applied = C.optimize_model(bytes(input), level, list(disabled_optimizers), bool(use_gpu))
    m = OptimizedModel(bytes(out))
    m.applied_passes = dict(applied) if isinstance(applied, dict) else applied
    return m


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Fuse transformer subgraphs of an ONNX model")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--model_type", default="bert")
    ap.add_argument("--num_heads", type=int, default=0)
    ap.add_argument("--hidden_size", type=int, default=0)
    ap.add_argument("--opt_level", type=int, default=99, choices=[0, 1, 2, 99])
    ap.add_argument("--use_gpu", action="store_true")
    ap.add_argument("--float16", action="store_true")
    ap.add_argument("--disable", nargs="*", default=[], help="names of passes to skip")
    a = ap.parse_args(argv)
    m = optimize_model(a.input, a.model_type, a.num_heads, a.hidden_size, a.opt_level, a.use_gpu, a.disable)
    if a.float16:
        m.convert_float_to_float16()
    m.save_model_to_file(a.output)
    print("fused operators:", m.get_fused_operator_statistics())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
