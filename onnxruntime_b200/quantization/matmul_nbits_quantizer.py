"""Round-to-nearest block quantisation of MatMul weights into ``com.microsoft.MatMulNBits``.

Mirrors what ``MatMulNBitsQuantizer`` with the default RTN algorithm does in the reference
(onnxruntime/python/tools/quantization/matmul_nbits_quantizer.py: ``DefaultWeightOnlyQuantizer.quantize_matmul``
and the native block quantiser behind ``quantize_matmul_4bits``): every ``MatMul`` whose second input is a constant
2-D ``[K, N]`` weight becomes ``MatMulNBits(A, B_packed, scales[, zero_points])`` with

* ``B_packed`` uint8 ``[N, n_blocks, block_size * bits / 8]`` (low nibble = even k),
* ``scales`` ``[N, n_blocks]`` in the weight's float type,
* ``zero_points`` packed uint8 ``[N, ceil(n_blocks * bits / 8)]`` when asymmetric (symmetric uses the implicit 2^(bits-1)).
"""
from __future__ import annotations

from typing import Iterable, Optional, Tuple, Union

import numpy as np

from .. import onnx_lite as ol

try:
    import torch
except ImportError:  # pragma: no cover
    torch = None


def quantize_blockwise(w_kn: np.ndarray, block_size: int = 32, bits: int = 4, symmetric: bool = True
                       ) -> Tuple[np.ndarray, np.ndarray, Optional[np.ndarray]]:
    """``w_kn`` float ``[K, N]`` -> (packed uint8 [N, n_blocks, blob], scales float32 [N, n_blocks], zero_points or None)."""
    assert bits in (4, 8) and block_size >= 16 and block_size & (block_size - 1) == 0
    K, N = w_kn.shape
    nb = (K + block_size - 1) // block_size
    w = np.zeros((N, nb * block_size), dtype=np.float32)
    w[:, :K] = np.asarray(w_kn, dtype=np.float32).T
    w = w.reshape(N, nb, block_size)
    qmax = (1 << bits) - 1
    mid = 1 << (bits - 1)
    if symmetric:
        # the value of largest magnitude maps to -mid (as in the reference's symmetric block quantiser)
        idx = np.abs(w).argmax(-1)
        vmax = np.take_along_axis(w, idx[..., None], -1)[..., 0]
        scales = vmax / -float(mid)
        inv = np.where(scales != 0, 1.0 / np.where(scales != 0, scales, 1.0), 0.0)
        q = np.clip(np.rint(w * inv[..., None]) + mid, 0, qmax).astype(np.uint8)
        zp = None
    else:
        lo = np.minimum(w.min(-1), 0.0)
        hi = np.maximum(w.max(-1), 0.0)
        scales = (hi - lo) / float(qmax)
        inv = np.where(scales != 0, 1.0 / np.where(scales != 0, scales, 1.0), 0.0)
        zp_vals = np.clip(np.rint(-lo * inv), 0, qmax).astype(np.uint8)
        q = np.clip(np.rint(w * inv[..., None]) + zp_vals[..., None], 0, qmax).astype(np.uint8)
        if bits == 4:
            z = np.zeros((N, (nb + 1) // 2 * 2), dtype=np.uint8)
            z[:, :nb] = zp_vals
            zp = (z[:, 0::2] | (z[:, 1::2] << 4)).astype(np.uint8)
        else:
            zp = zp_vals
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8) if bits == 4 else q
    return packed, scales.astype(np.float32), zp


def quantize_blockwise_hqq(w_kn: np.ndarray, block_size: int = 32, bits: int = 4, iters: int = 20, lp_norm: float = 0.7, beta: float = 10.0,
                           kappa: float = 1.01) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Half-quadratic quantisation (the HQQ option of the reference's quantizer, ``HQQWeightOnlyQuantizer``): starting from the
    min-max scale of every block, the zero point is re-fitted for a few iterations against an l_p (p < 1) shrinkage of the
    reconstruction error, which moves it away from what outliers dictate.  Zero points stay FLOAT (MatMulNBits takes zero
    points of the scales' type): returns (packed uint8, scales float32 [N, n_blocks], zero_points float32 [N, n_blocks])."""
    assert bits in (4, 8) and block_size >= 16 and block_size & (block_size - 1) == 0
    K, N = w_kn.shape
    nb = (K + block_size - 1) // block_size
    w = np.zeros((N, nb * block_size), dtype=np.float32)
    w[:, :K] = np.asarray(w_kn, dtype=np.float32).T
    w = w.reshape(N, nb, block_size)
    qmax = float((1 << bits) - 1)
    lo, hi = w.min(-1, keepdims=True), w.max(-1, keepdims=True)
    inv_scale = qmax / np.maximum(hi - lo, 1e-8)          # quantisation multiplies by this
    zero = -lo * inv_scale
    best_err, best_zero = None, zero
    for _ in range(iters):
        q = np.clip(np.rint(w * inv_scale + zero), 0, qmax)
        recon = (q - zero) / inv_scale
        resid = w - recon
        shrunk = np.sign(resid) * np.maximum(np.abs(resid) - (1.0 / beta) * np.power(np.abs(resid) + 1e-8, lp_norm - 1.0), 0.0)
        zero = np.mean(q - (w - shrunk) * inv_scale, -1, keepdims=True)
        beta *= kappa
        err = float(np.abs(w - recon).mean())
        if best_err is not None and err >= best_err:
            break
        best_err, best_zero = err, zero
    zero = best_zero
    q = np.clip(np.rint(w * inv_scale + zero), 0, qmax).astype(np.uint8)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8) if bits == 4 else q
    return packed, (1.0 / inv_scale)[..., 0].astype(np.float32), zero[..., 0].astype(np.float32)


def quantize_blockwise_gptq(w_kn: np.ndarray, hessian: np.ndarray, block_size: int = 32, bits: int = 4, percdamp: float = 0.01,
                            update_block: int = 128) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """GPTQ (the GPTQ option of the reference's quantizer, ``GPTQWeightOnlyQuantConfig``): the columns of the weight are
    rounded one after the other along K, and the rounding error of each is pushed onto the columns not yet rounded
    through the inverse of ``hessian`` = X^T X of calibration activations [K, K], so that the error of X W, not of W, is
    kept small.  Asymmetric min-max grid per block of ``block_size`` along K, fixed when the block is reached.  Same
    return layout as ``quantize_blockwise(..., symmetric=False)``."""
    assert bits in (4, 8) and block_size >= 16 and block_size & (block_size - 1) == 0
    K, N = w_kn.shape
    assert K % block_size == 0, "GPTQ needs K to be a multiple of the block size"
    nb = K // block_size
    qmax = float((1 << bits) - 1)
    W = np.asarray(w_kn, dtype=np.float64).T.copy()          # [N, K]
    H = np.asarray(hessian, dtype=np.float64).copy()
    dead = np.diag(H) == 0
    H[dead, dead] = 1.0
    W[:, dead] = 0.0
    H[np.diag_indices(K)] += percdamp * np.mean(np.diag(H))
    Hinv = np.linalg.cholesky(np.linalg.inv(H)).T             # upper factor of H^-1
    q_int = np.zeros((N, K), dtype=np.uint8)
    scales = np.zeros((N, nb), dtype=np.float64)
    zps = np.zeros((N, nb), dtype=np.float64)
    for i1 in range(0, K, update_block):
        i2 = min(i1 + update_block, K)
        W1 = W[:, i1:i2].copy()
        Err = np.zeros_like(W1)
        Hi = Hinv[i1:i2, i1:i2]
        for i in range(i2 - i1):
            col = i1 + i
            blk = col // block_size
            if col % block_size == 0:                           # fix the grid of this block from its present values
                seg = np.concatenate([W1[:, i:i + block_size], W[:, i2:col + block_size]], 1)[:, :block_size]
                lo, hi = np.minimum(seg.min(1), 0.0), np.maximum(seg.max(1), 0.0)
                sc = (hi - lo) / qmax
                sc[sc == 0] = 1.0
                scales[:, blk] = sc
                zps[:, blk] = np.clip(np.rint(-lo / sc), 0, qmax)
            w = W1[:, i]
            q = np.clip(np.rint(w / scales[:, blk] + zps[:, blk]), 0, qmax)
            q_int[:, col] = q.astype(np.uint8)
            err = (w - (q - zps[:, blk]) * scales[:, blk]) / Hi[i, i]
            W1[:, i:] -= np.outer(err, Hi[i, i:])
            Err[:, i] = err
        W[:, i2:] -= Err @ Hinv[i1:i2, i2:]
    q3 = q_int.reshape(N, nb, block_size)
    zp_vals = zps.astype(np.uint8)
    if bits == 4:
        z = np.zeros((N, (nb + 1) // 2 * 2), dtype=np.uint8)
        z[:, :nb] = zp_vals
        zp = (z[:, 0::2] | (z[:, 1::2] << 4)).astype(np.uint8)
        packed = (q3[..., 0::2] | (q3[..., 1::2] << 4)).astype(np.uint8)
    else:
        zp, packed = zp_vals, q3
    return packed, scales.astype(np.float32), zp


def dequantize_blockwise(packed: np.ndarray, scales: np.ndarray, zero_points: Optional[np.ndarray], K: int, bits: int = 4,
                         block_size: int = 32) -> np.ndarray:
    """Inverse of :func:`quantize_blockwise`: float32 ``[N, K]``."""
    N, nb = scales.shape
    if bits == 4:
        q = np.stack([packed & 0xF, packed >> 4], -1).reshape(N, nb, block_size).astype(np.float32)
    else:
        q = packed.reshape(N, nb, block_size).astype(np.float32)
    if zero_points is None:
        zp = np.full((N, nb), float(1 << (bits - 1)), dtype=np.float32)
    elif bits == 4 and zero_points.dtype == np.uint8:
        zp = np.stack([zero_points & 0xF, zero_points >> 4], -1).reshape(N, -1)[:, :nb].astype(np.float32)
    else:
        zp = zero_points.reshape(N, nb).astype(np.float32)
    return ((q - zp[..., None]) * scales.astype(np.float32)[..., None]).reshape(N, nb * block_size)[:, :K]


class MatMulNBitsQuantizer:
    """``MatMulNBitsQuantizer(model, block_size=32, is_symmetric=True, bits=4).process()`` then ``.model`` /
    ``.save(path)``.  ``model`` is ModelProto bytes, a path, or an ``onnx_lite.Model``."""

    def __init__(self, model: Union[str, bytes, ol.Model], block_size: int = 32, is_symmetric: bool = True, bits: int = 4,
                 nodes_to_exclude: Iterable[str] = (), nodes_to_include: Optional[Iterable[str]] = None, min_elements: int = 0,
                 algorithm: str = "rtn", calibration_data_reader=None):
        if algorithm not in ("rtn", "hqq", "gptq"):
            raise ValueError("algorithm must be 'rtn' (round to nearest), 'hqq' (half-quadratic, float zero points) or "
                             "'gptq' (error feedback through calibration activations; needs calibration_data_reader)")
        if algorithm == "gptq" and calibration_data_reader is None:
            raise ValueError("algorithm 'gptq' needs a calibration_data_reader (an object with get_next() -> feeds or None)")
        self.algorithm = algorithm
        self.calibration_data_reader = calibration_data_reader
        self._hessians = {}
        self.model = model if isinstance(model, ol.Model) else ol.load_model(model)
        self.block_size, self.symmetric, self.bits = block_size, is_symmetric, bits
        self.exclude = set(nodes_to_exclude)
        self.include = None if nodes_to_include is None else set(nodes_to_include)
        self.min_elements = min_elements
        self.quantized_nodes = []

    def _collect_hessians(self) -> None:
        """Runs the float model over the calibration feeds with the activation of every candidate MatMul as an extra
        output and accumulates X^T X (rows = all leading dimensions) per activation."""
        import copy

        from .. import capi
        g = self.model.graph
        inits = {t.name for t in g.initializers}
        acts = []
        for n in g.nodes:
            if n.op_type == "MatMul" and len(n.inputs) == 2 and n.inputs[1] in inits and n.inputs[0] not in acts:
                acts.append(n.inputs[0])
        probe = copy.deepcopy(self.model)
        have = {o.name for o in probe.graph.outputs}
        probe.graph.outputs.extend(ol.make_tensor_value_info(a, 0, None) for a in acts if a not in have)
        so = capi.SessionOptions()
        so.graph_optimization_level = capi.GraphOptimizationLevel.ORT_DISABLE_ALL
        sess = capi.InferenceSession(probe.serialize(), so, providers=["CPUExecutionProvider"])
        while True:
            feeds = self.calibration_data_reader.get_next()
            if feeds is None:
                break
            for a, x in zip(acts, sess.run(acts, feeds)):
                x2 = np.asarray(x, dtype=np.float64).reshape(-1, x.shape[-1])
                self._hessians[a] = self._hessians.get(a, 0.0) + x2.T @ x2

    def process(self) -> ol.Model:
        if self.algorithm == "gptq" and not self._hessians:
            self._collect_hessians()
        g = self.model.graph
        inits = {t.name: t for t in g.initializers}
        uses = {}
        for n in g.nodes:
            for i in n.inputs:
                uses[i] = uses.get(i, 0) + 1
        new_nodes = []
        for n in g.nodes:
            w = inits.get(n.inputs[1]) if n.op_type == "MatMul" and n.domain in ("", "ai.onnx") and len(n.inputs) == 2 else None
            ok = (w is not None and w.external is None and len(w.dims) == 2 and n.name not in self.exclude and
                  (self.include is None or n.name in self.include) and
                  w.data_type in (ol.TensorProto.FLOAT, ol.TensorProto.FLOAT16, ol.TensorProto.BFLOAT16) and
                  int(np.prod(w.dims)) >= self.min_elements)
            if not ok:
                new_nodes.append(n)
                continue
            arr = ol.to_array(w)
            is_torch = not isinstance(arr, np.ndarray)
            w32 = arr.float().numpy() if is_torch else arr.astype(np.float32)
            K, N = w32.shape
            if self.algorithm == "gptq" and n.inputs[0] in self._hessians:
                packed, scales, zp = quantize_blockwise_gptq(w32, self._hessians[n.inputs[0]], self.block_size, self.bits)
            elif self.algorithm == "hqq":
                packed, scales, zp = quantize_blockwise_hqq(w32, self.block_size, self.bits)
            else:
                packed, scales, zp = quantize_blockwise(w32, self.block_size, self.bits, self.symmetric)
            base = n.inputs[1]
            if is_torch:
                import torch  # noqa: F811
                scales_t = ol.make_tensor(base + "_scales", torch.from_numpy(scales).to(arr.dtype))
            else:
                scales_t = ol.make_tensor(base + "_scales", scales.astype(arr.dtype))
            g.initializers.append(ol.make_tensor(base + "_Q" + str(self.bits), packed))
            g.initializers.append(scales_t)
            ins = [n.inputs[0], base + "_Q" + str(self.bits), base + "_scales"]
            if zp is not None:
                if zp.dtype != np.uint8:   # float zero points take the type of the scales
                    zp = torch.from_numpy(zp).to(arr.dtype) if is_torch else zp.astype(arr.dtype)
                g.initializers.append(ol.make_tensor(base + "_zero_points", zp))
                ins.append(base + "_zero_points")
            new_nodes.append(ol.make_node("MatMulNBits", ins, list(n.outputs), name=(n.name + "_Q" + str(self.bits)) if n.name else "",
                                          domain="com.microsoft", K=K, N=N, bits=self.bits, block_size=self.block_size))
            self.quantized_nodes.append(n.name or n.outputs[0])
            uses[base] -= 1
        g.nodes = new_nodes
        g.initializers = [t for t in g.initializers if uses.get(t.name, 1) > 0 or t.name not in inits]
        self.model.opset_imports.setdefault("com.microsoft", 1)
        return self.model

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.model.serialize())
