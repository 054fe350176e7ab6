"""MatMul weights -> 4-bit NF4 / FP4 blocks (``com.microsoft.MatMulBnb4``).

Counterpart of the reference's onnxruntime/python/tools/quantization/matmul_bnb4_quantizer.py: every MatMul whose B is
a constant 2-D float matrix becomes a MatMulBnb4 node with the weight stored transposed ([N, K] flattened), two codes per
byte (first in the high nibble) and one absmax per block of ``block_size`` consecutive elements."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np

from .. import onnx_lite as ol

FP4, NF4 = 0, 1
_FP4_TABLE = np.array([0.0, 0.0052083333, 0.6666667, 1.0, 0.33333334, 0.5, 0.16666667, 0.25,
                       -0.0, -0.0052083333, -0.6666667, -1.0, -0.33333334, -0.5, -0.16666667, -0.25], np.float32)
_NF4_TABLE = np.array([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                       -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                       0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                       0.7229568362236023, 1.0], np.float32)


def quantize_bnb4(w_kn: np.ndarray, quant_type: int = NF4, block_size: int = 64):
    """[K, N] float weight -> (packed uint8 [ceil(N*K/2)], absmax float32 [ceil(N*K/block)]) of the transposed matrix."""
    table = _NF4_TABLE if quant_type == NF4 else _FP4_TABLE
    flat = np.ascontiguousarray(w_kn.T, dtype=np.float32).reshape(-1)
    n = flat.size
    blocks = -(-n // block_size)
    padded = np.zeros(blocks * block_size, np.float32)
    padded[:n] = flat
    padded = padded.reshape(blocks, block_size)
    absmax = np.abs(padded).max(1)
    scaled = padded / np.where(absmax > 0, absmax, 1.0)[:, None]
    codes = np.abs(scaled.reshape(-1, 1) - table[None, :]).argmin(1).astype(np.uint8)[:n]
    if n % 2:
        codes = np.append(codes, np.uint8(0))
    packed = (codes[0::2] << 4) | codes[1::2]
    return packed.astype(np.uint8), absmax.astype(np.float32)


def dequantize_bnb4(packed: np.ndarray, absmax: np.ndarray, K: int, N: int, quant_type: int = NF4, block_size: int = 64) -> np.ndarray:
    table = _NF4_TABLE if quant_type == NF4 else _FP4_TABLE
    codes = np.stack([packed >> 4, packed & 15], 1).reshape(-1)[:N * K]
    scale = np.repeat(absmax, block_size)[:N * K]
    return (table[codes] * scale).reshape(N, K).T


class MatMulBnb4Quantizer:
    def __init__(self, model: Union[str, bytes, ol.Model], quant_type: int = NF4, block_size: int = 64, nodes_to_exclude: Optional[Sequence[str]] = None):
        self.model = model if isinstance(model, ol.Model) else ol.load_model(model)
        self.quant_type, self.block_size = int(quant_type), int(block_size)
        self.nodes_to_exclude = set(nodes_to_exclude or [])
        if self.quant_type not in (FP4, NF4):
            raise ValueError("quant_type must be FP4 (0) or NF4 (1)")

    def process(self) -> ol.Model:
        g = self.model.graph
        inits = {t.name: t for t in g.initializers}
        new_nodes: List[ol.Node] = []
        for n in g.nodes:
            w_t = inits.get(n.inputs[1]) if n.op_type == "MatMul" and n.domain == "" and len(n.inputs) > 1 else None
            if w_t is None or n.name in self.nodes_to_exclude:
                new_nodes.append(n)
                continue
            w = ol.to_array(w_t)
            if w.ndim != 2 or w.dtype not in (np.float32, np.float16):
                new_nodes.append(n)
                continue
            K, N = w.shape
            packed, absmax = quantize_bnb4(w.astype(np.float32), self.quant_type, self.block_size)
            g.initializers += [ol.make_tensor(w_t.name + "_Bnb4", packed), ol.make_tensor(w_t.name + "_absmax", absmax.astype(w.dtype))]
            new_nodes.append(ol.make_node("MatMulBnb4", [n.inputs[0], w_t.name + "_Bnb4", w_t.name + "_absmax"], list(n.outputs), domain="com.microsoft",
                                          name=(n.name + "_Bnb4") if n.name else "", K=int(K), N=int(N), block_size=self.block_size, quant_type=self.quant_type))
        g.nodes = new_nodes
        used = {i for n in g.nodes for i in n.inputs} | {o.name for o in g.outputs}
        g.initializers = [t for t in g.initializers if t.name in used]
        self.model.opset_imports.setdefault("com.microsoft", 1)
        return self.model
