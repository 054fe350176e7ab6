"""8-bit quantisation of ONNX models: dynamic (weights offline, activations at run time) and static (QDQ format
from calibration data).

Counterparts in the reference: ``quantize_dynamic`` / ``quantize_static`` / ``MinMaxCalibrater``
(onnxruntime/python/tools/quantization/quantize.py, onnx_quantizer.py, qdq_quantizer.py, calibrate.py).

* ``quantize_dynamic``: every ``MatMul`` with a constant 2-D weight becomes ``com.microsoft.DynamicQuantizeMatMul``
  (the activation is quantised to uint8 per call, the weight is stored as int8 / uint8 with a per-tensor or
  per-column scale).
* ``quantize_static``: activations of ``MatMul`` / ``Gemm`` / ``Conv`` are observed on calibration feeds (min / max),
  then ``QuantizeLinear -> DequantizeLinear`` pairs are inserted on their inputs and the constant weights are stored
  quantised behind a ``DequantizeLinear`` (QDQ format); the engine's optimizer or any QDQ-aware runtime can fuse them.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


def _load(model: Union[str, bytes, ol.Model]) -> ol.Model:
    return model if isinstance(model, ol.Model) else ol.load_model(model)


def _save(model: ol.Model, path: Optional[str]) -> ol.Model:
    if path:
        with open(path, "wb") as f:
            f.write(model.serialize())
    return model


def quantize_weight(w: np.ndarray, signed: bool = True, per_channel: bool = False, axis: int = -1, symmetric: bool = True):
    """float weight -> (q, scale, zero_point).  Per-channel scales run along ``axis``."""
    w = np.asarray(w, dtype=np.float32)
    qmin, qmax = (-127, 127) if signed else (0, 255)
    if per_channel:
        red = tuple(i for i in range(w.ndim) if i != axis % w.ndim)
        lo, hi = w.min(axis=red), w.max(axis=red)
        shape = [1] * w.ndim
        shape[axis % w.ndim] = -1
    else:
        lo, hi = np.float32(w.min()), np.float32(w.max())
        shape = []
    lo, hi = np.minimum(lo, 0), np.maximum(hi, 0)
    if symmetric and signed:
        scale = np.maximum(np.abs(lo), np.abs(hi)) / 127.0
        zp = np.zeros_like(scale)
    else:
        scale = (hi - lo) / float(qmax - qmin)
        zp = None
    scale = np.where(scale == 0, 1.0, scale).astype(np.float32)
    if zp is None:
        zp = np.clip(np.rint(qmin - lo / scale), qmin, qmax)
    s, z = (scale.reshape(shape), zp.reshape(shape)) if per_channel else (scale, zp)
    q = np.clip(np.rint(w / s) + z, qmin, qmax).astype(np.int8 if signed else np.uint8)
    return q, scale.astype(np.float32), zp.astype(np.int8 if signed else np.uint8)


def quantize_dynamic(model_input, model_output: Optional[str] = None, per_channel: bool = False, weight_signed: bool = True,
                     nodes_to_exclude: Iterable[str] = ()) -> ol.Model:
    model = _load(model_input)
    g = model.graph
    inits = {t.name: t for t in g.initializers}
    exclude = set(nodes_to_exclude)
    new_nodes: List[ol.Node] = []
    for n in g.nodes:
        w_t = inits.get(n.inputs[1]) if n.op_type == "MatMul" and n.domain == "" and len(n.inputs) == 2 else None
        if w_t is None or n.name in exclude or len(w_t.dims) != 2:
            new_nodes.append(n)
            continue
        w = ol.to_array(w_t)
        if w.dtype not in (np.float32, np.float16):
            new_nodes.append(n)
            continue
        q, scale, zp = quantize_weight(w, signed=weight_signed, per_channel=per_channel, axis=1)
        base = n.inputs[1]
        g.initializers += [ol.make_tensor(base + "_quantized", q), ol.make_tensor(base + "_scale", scale),
                           ol.make_tensor(base + "_zero_point", zp)]
        new_nodes.append(ol.make_node("DynamicQuantizeMatMul", [n.inputs[0], base + "_quantized", base + "_scale", base + "_zero_point"],
                                      list(n.outputs), name=(n.name + "_quant") if n.name else "", domain="com.microsoft"))
    g.nodes = new_nodes
    used = {i for n in g.nodes for i in n.inputs} | {o.name for o in g.outputs}
    g.initializers = [t for t in g.initializers if t.name in used]
    model.opset_imports.setdefault("com.microsoft", 1)
    return _save(model, model_output)


class MinMaxCalibrator:
    """Runs the float model on calibration feeds with the chosen tensors exposed as outputs and keeps their ranges."""

    def __init__(self, model: ol.Model, tensors: Sequence[str]):
        import copy

        import onnxruntime_b200 as ort
        m = copy.deepcopy(model)
        have = {o.name for o in m.graph.outputs}
        self.tensors = [t for t in dict.fromkeys(tensors)]
        for t in self.tensors:
            if t not in have:
                m.graph.outputs.append(ol.make_tensor_value_info(t, 0, None))
        so = ort.SessionOptions()
        so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
        self.sess = ort.InferenceSession(m.serialize(), so, providers=["CPUExecutionProvider"])
        self.ranges: Dict[str, List[float]] = {}

    def collect(self, feeds: Dict[str, np.ndarray]) -> None:
        graph_inputs = {i.name for i in self.sess.get_inputs()}
        outs = self.sess.run(self.tensors, {k: v for k, v in feeds.items() if k in graph_inputs})
        for name, v in zip(self.tensors, outs):
            v = np.asarray(v, dtype=np.float32)
            lo, hi = float(v.min()), float(v.max())
            r = self.ranges.setdefault(name, [lo, hi])
            r[0], r[1] = min(r[0], lo), max(r[1], hi)


class HistogramCalibrator(MinMaxCalibrator):
    """Keeps a histogram of |x| per tensor (2048 bins, range grown as needed) instead of the bare extremes; the entropy and
    percentile calibrators of the reference (onnxruntime/python/tools/quantization/calibrate.py) cut the range from it."""

    BINS = 2048

    def __init__(self, model: ol.Model, tensors: Sequence[str]):
        super().__init__(model, tensors)
        self.hist: Dict[str, np.ndarray] = {}
        self.limit: Dict[str, float] = {}

    def collect(self, feeds: Dict[str, np.ndarray]) -> None:
        graph_inputs = {i.name for i in self.sess.get_inputs()}
        outs = self.sess.run(self.tensors, {k: v for k, v in feeds.items() if k in graph_inputs})
        for name, v in zip(self.tensors, outs):
            a = np.abs(np.asarray(v, dtype=np.float32)).reshape(-1)
            top = float(a.max()) if a.size else 0.0
            if name not in self.hist:
                self.limit[name] = max(top, 1e-12)
                self.hist[name] = np.zeros(self.BINS, np.float64)
            elif top > self.limit[name]:
                # re-bin the old counts into the wider range
                old_edges = np.linspace(0, self.limit[name], self.BINS + 1)
                centres = (old_edges[:-1] + old_edges[1:]) / 2
                self.hist[name] = np.histogram(centres, bins=self.BINS, range=(0, top), weights=self.hist[name])[0]
                self.limit[name] = top
            self.hist[name] += np.histogram(a, bins=self.BINS, range=(0, self.limit[name]))[0]

    def _finish(self, pick) -> None:
        for name, h in self.hist.items():
            edge = pick(h, np.linspace(0, self.limit[name], self.BINS + 1))
            self.ranges[name] = [-edge, edge]


class PercentileCalibrator(HistogramCalibrator):
    """Symmetric range that keeps `percentile` percent of the observed |x| mass."""

    def __init__(self, model: ol.Model, tensors: Sequence[str], percentile: float = 99.999):
        super().__init__(model, tensors)
        self.percentile = float(percentile)

    def compute_ranges(self) -> Dict[str, List[float]]:
        def pick(h, edges):
            cdf = np.cumsum(h) / max(h.sum(), 1.0)
            return float(edges[min(int(np.searchsorted(cdf, self.percentile / 100.0)) + 1, len(edges) - 1)])
        self._finish(pick)
        return self.ranges


class EntropyCalibrator(HistogramCalibrator):
    """Symmetric range that minimises the KL divergence between the histogram and its 128-level quantisation."""

    def __init__(self, model: ol.Model, tensors: Sequence[str], num_quantized_bins: int = 128):
        super().__init__(model, tensors)
        self.levels = int(num_quantized_bins)

    def compute_ranges(self) -> Dict[str, List[float]]:
        levels = self.levels

        def pick(h, edges):
            best, best_i = None, len(h)
            for i in range(levels, len(h) + 1, 16):
                p = h[:i].copy()
                p[i - 1] += h[i:].sum()                      # the clipped tail lands in the last kept bin
                if p.sum() == 0:
                    continue
                # quantise the kept bins to `levels` levels and expand back over the non-empty bins
                chunks = np.array_split(np.arange(i), levels)
                q = np.zeros(i)
                for c in chunks:
                    mass, nz = h[c].sum(), (h[c] > 0).sum()
                    if nz:
                        q[c] = np.where(h[c] > 0, mass / nz, 0.0)
                pn, qn = p / p.sum(), q / max(q.sum(), 1e-30)
                mask = pn > 0
                kl = float(np.sum(pn[mask] * np.log(pn[mask] / np.maximum(qn[mask], 1e-30))))
                if best is None or kl < best:
                    best, best_i = kl, i
            return float(edges[best_i])
        self._finish(pick)
        return self.ranges


class CalibrationMethod:
    MinMax, Entropy, Percentile = 0, 1, 2


class QuantFormat:
    QOperator, QDQ = 0, 1


class QuantType:
    QInt8, QUInt8 = 0, 1


class CalibrationDataReader:
    """Iterator of feed dicts for quantize_static: subclass and implement get_next() (None when exhausted)."""

    def get_next(self) -> Optional[Dict[str, np.ndarray]]:
        raise NotImplementedError

    def __iter__(self):
        return self

    def __next__(self):
        feeds = self.get_next()
        if feeds is None:
            raise StopIteration
        return feeds


def quantize_static(model_input, calibration_feeds: Iterable[Dict[str, np.ndarray]], model_output: Optional[str] = None,
                    op_types: Sequence[str] = ("MatMul", "Gemm", "Conv"), per_channel: bool = False,
                    calibrate_method: int = CalibrationMethod.MinMax, percentile: float = 99.999,
                    quant_format: int = QuantFormat.QDQ) -> ol.Model:
    """QDQ format: uint8 asymmetric activations, int8 symmetric weights (per tensor, or per output channel).  The activation
    ranges come from the extremes (MinMax), or from a histogram cut by KL divergence (Entropy) or by mass (Percentile).
    quant_format = QuantFormat.QOperator writes MatMul nodes with a constant weight as QuantizeLinear -> QLinearMatMul ->
    DequantizeLinear (their output ranges are calibrated too); other operators keep the QDQ form."""
    model = _load(model_input)
    g = model.graph
    inits = {t.name: t for t in g.initializers}
    targets = [n for n in g.nodes if n.op_type in op_types and n.domain == ""]
    acts = [n.inputs[0] for n in targets if n.inputs[0] not in inits]
    if quant_format == QuantFormat.QOperator:
        acts += [n.outputs[0] for n in targets if n.op_type == "MatMul" and len(n.inputs) > 1 and n.inputs[1] in inits]
    if calibrate_method == CalibrationMethod.Entropy:
        calib = EntropyCalibrator(model, acts)
    elif calibrate_method == CalibrationMethod.Percentile:
        calib = PercentileCalibrator(model, acts, percentile)
    else:
        calib = MinMaxCalibrator(model, acts)
    for feeds in calibration_feeds:
        calib.collect(feeds)
    if calibrate_method != CalibrationMethod.MinMax:
        calib.compute_ranges()
    new_nodes: List[ol.Node] = []
    qdq_of: Dict[str, str] = {}
    for n in g.nodes:
        if n not in targets:
            new_nodes.append(n)
            continue
        ins = list(n.inputs)
        a = ins[0]
        w_t = inits.get(ins[1]) if len(ins) > 1 else None
        if (quant_format == QuantFormat.QOperator and n.op_type == "MatMul" and w_t is not None and ol.to_array(w_t).dtype == np.float32
                and ol.to_array(w_t).ndim == 2 and a in calib.ranges and n.outputs[0] in calib.ranges):
            def act_params(name):
                lo, hi = min(calib.ranges[name][0], 0.0), max(calib.ranges[name][1], 0.0)
                scale = np.float32((hi - lo) / 255.0) if hi > lo else np.float32(1.0)
                return scale, np.uint8(np.clip(np.rint(-lo / scale), 0, 255))
            (xs, xz), (ys, yz) = act_params(a), act_params(n.outputs[0])
            q, ws, wz = quantize_weight(ol.to_array(w_t), signed=True, per_channel=per_channel, axis=1)
            base, out = ins[1], n.outputs[0]
            tag = (n.name or out)
            g.initializers += [ol.make_tensor(tag + "_x_scale", np.array(xs, np.float32)), ol.make_tensor(tag + "_x_zp", np.array(xz, np.uint8)),
                               ol.make_tensor(tag + "_y_scale", np.array(ys, np.float32)), ol.make_tensor(tag + "_y_zp", np.array(yz, np.uint8)),
                               ol.make_tensor(base + "_quantized", q), ol.make_tensor(base + "_scale", ws), ol.make_tensor(base + "_zero_point", wz)]
            new_nodes.append(ol.make_node("QuantizeLinear", [a, tag + "_x_scale", tag + "_x_zp"], [tag + "_xq"], name=tag + "_QuantizeLinear"))
            new_nodes.append(ol.make_node("QLinearMatMul", [tag + "_xq", tag + "_x_scale", tag + "_x_zp", base + "_quantized", base + "_scale", base + "_zero_point",
                                                            tag + "_y_scale", tag + "_y_zp"], [tag + "_yq"], name=tag + "_QLinearMatMul"))
            new_nodes.append(ol.make_node("DequantizeLinear", [tag + "_yq", tag + "_y_scale", tag + "_y_zp"], [out], name=tag + "_DequantizeLinear"))
            continue
        if a in calib.ranges:
            if a not in qdq_of:
                lo, hi = min(calib.ranges[a][0], 0.0), max(calib.ranges[a][1], 0.0)
                scale = np.float32((hi - lo) / 255.0) if hi > lo else np.float32(1.0)
                zp = np.uint8(np.clip(np.rint(-lo / scale), 0, 255))
                g.initializers += [ol.make_tensor(a + "_scale", np.array(scale, np.float32)), ol.make_tensor(a + "_zero_point", np.array(zp, np.uint8))]
                new_nodes.append(ol.make_node("QuantizeLinear", [a, a + "_scale", a + "_zero_point"], [a + "_quantized"], name=a + "_QuantizeLinear"))
                new_nodes.append(ol.make_node("DequantizeLinear", [a + "_quantized", a + "_scale", a + "_zero_point"], [a + "_dequantized"],
                                              name=a + "_DequantizeLinear"))
                qdq_of[a] = a + "_dequantized"
            ins[0] = qdq_of[a]
        w_t = inits.get(ins[1]) if len(ins) > 1 else None
        if w_t is not None and ol.to_array(w_t).dtype == np.float32:
            w = ol.to_array(w_t)
            # output channels: rows of a Conv weight / transposed Gemm weight, columns of a MatMul weight
            trans_b = n.op_type == "Gemm" and any(a_.name == "transB" and ol.attr_value(a_) == 1 for a_ in n.attributes)
            axis = 0 if (n.op_type == "Conv" or trans_b) else w.ndim - 1
            q, scale, zp = quantize_weight(w, signed=True, per_channel=per_channel, axis=axis)
            base = ins[1]
            g.initializers += [ol.make_tensor(base + "_quantized", q), ol.make_tensor(base + "_scale", scale), ol.make_tensor(base + "_zero_point", zp)]
            dq = ol.make_node("DequantizeLinear", [base + "_quantized", base + "_scale", base + "_zero_point"], [base + "_dequantized"],
                              name=base + "_DequantizeLinear", **({"axis": axis} if per_channel else {}))
            new_nodes.append(dq)
            ins[1] = base + "_dequantized"
        n.inputs = ins
        new_nodes.append(n)
    g.nodes = new_nodes
    used = {i for n in g.nodes for i in n.inputs} | {o.name for o in g.outputs}
    g.initializers = [t for t in g.initializers if t.name in used]
    if per_channel and model.opset_imports.get("", 0) < 13:
        model.opset_imports[""] = 13
    return _save(model, model_output)
