"""Shape inference by tracing: fills ``graph.value_info`` with the type and shape of every intermediate tensor.

    python -m onnxruntime_b200.tools.shape_inference model.onnx out.onnx [--dim batch=2 --dim seq=8]

The reference ships ``symbolic_shape_infer.py`` (onnxruntime/python/tools/symbolic_shape_infer.py), a sympy-based
re-implementation of every operator's shape function, because ONNX's own inference gives up on data-dependent
shapes (Reshape with computed targets, Range, NonZero, ...) and on contrib operators.  Here the engine itself is the
shape function: the model runs on the CPU provider twice with two different assignments of the symbolic input
dimensions and every intermediate tensor is observed.  A dimension that is the same in both runs is static; one
that follows an input dimension gets that dimension's name; anything else gets a fresh symbol.  Operators need no
per-operator shape code, so contrib and custom operators are covered the day their kernel exists.
"""
from __future__ import annotations

import argparse
import copy
from typing import Dict, List, Optional, Sequence, Union

import numpy as np

from .. import onnx_lite as ol


def _feeds_for(model: ol.Model, dims: Dict[str, int], default: int, rng) -> Dict[str, np.ndarray]:
    inits = {t.name for t in model.graph.initializers}
    feeds = {}
    for vi in model.graph.inputs:
        if vi.name in inits:
            continue
        shape = [dims.get(d, default) if isinstance(d, str) else (int(d) if d is not None else default) for d in (vi.shape or [])]
        dt = ol.onnx_to_np_dtype(vi.elem_type) if vi.elem_type in (1, 2, 3, 5, 6, 7, 9, 10, 11, 12, 13) else np.float32
        if np.issubdtype(dt, np.floating):
            feeds[vi.name] = rng.standard_normal(shape).astype(dt)
        elif dt == np.bool_:
            feeds[vi.name] = np.ones(shape, dtype=dt)
        else:
            feeds[vi.name] = np.zeros(shape, dtype=dt)   # indices / lengths: zero is always in range
    return feeds


def _trace(model: ol.Model, feeds: Dict[str, np.ndarray], names: Sequence[str]):
    import onnxruntime_b200 as ort
    m = copy.deepcopy(model)
    have = {o.name for o in m.graph.outputs}
    for n in names:
        if n not in have:
            m.graph.outputs.append(ol.make_tensor_value_info(n, 0, None))
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    sess = ort.InferenceSession(m.serialize(), so, providers=["CPUExecutionProvider"])
    outs = sess.run(list(names), feeds)
    return {n: o for n, o in zip(names, outs)}


def infer_shapes(model: Union[str, bytes, ol.Model], dim_values: Optional[Dict[str, int]] = None,
                 feeds: Optional[Dict[str, np.ndarray]] = None) -> ol.Model:
    """Returns the model with ``value_info`` for every node output that is a tensor.  ``dim_values`` fixes symbolic
    input dimensions for the first trace (others default to 2); ``feeds`` supplies real inputs for models whose
    control flow or indexing needs meaningful values (then only one trace runs and every dimension is static)."""
    model = model if isinstance(model, ol.Model) else ol.load_model(model)
    model = copy.deepcopy(model)
    g = model.graph
    names: List[str] = [o for n in g.nodes for o in n.outputs if o]
    rng = np.random.default_rng(0)
    dim_values = dict(dim_values or {})
    sym_dims = sorted({d for vi in g.inputs for d in (vi.shape or []) if isinstance(d, str)})
    if feeds is not None:
        runs = [_trace(model, feeds, names)]
        assign = [{}]
    else:
        a = {d: dim_values.get(d, 2) for d in sym_dims}
        # distinct primes in the second run, so that a traced dimension identifies the input dimension it follows
        primes = [3, 5, 7, 11, 13, 17, 19, 23, 29, 31]
        b = {d: primes[i % len(primes)] + (a[d] if primes[i % len(primes)] == a[d] else 0) for i, d in enumerate(sym_dims)}
        assign = [a, b]
        runs = [_trace(model, _feeds_for(model, a, 2, rng), names), _trace(model, _feeds_for(model, b, 3, rng), names)]
    existing = {v.name for v in g.value_info} | {o.name for o in g.outputs}
    fresh = 0
    for name in names:
        v0 = runs[0].get(name)
        if v0 is None or not hasattr(v0, "shape"):
            continue
        s0 = list(np.shape(v0))
        shape: List[Union[int, str]] = []
        if len(runs) == 2 and hasattr(runs[1].get(name), "shape") and len(np.shape(runs[1][name])) == len(s0):
            s1 = list(np.shape(runs[1][name]))
            for d0, d1 in zip(s0, s1):
                if d0 == d1:
                    shape.append(int(d0))
                    continue
                match = [d for d in sym_dims if assign[0][d] == d0 and assign[1][d] == d1]
                if match:
                    shape.append(match[0])
                else:
                    shape.append(f"unk__{fresh}")
                    fresh += 1
        else:
            shape = [int(d) for d in s0]
        try:
            et = ol.np_dtype_to_onnx(np.asarray(v0).dtype) if not hasattr(v0, "dtype") or isinstance(v0, np.ndarray) else _torch_type(v0)
        except KeyError:
            continue
        if name in existing:
            for vi in list(g.value_info) + list(g.outputs):
                if vi.name == name and (vi.shape is None or not vi.elem_type):
                    vi.elem_type, vi.shape = et, shape
            continue
        g.value_info.append(ol.make_tensor_value_info(name, et, shape))
    return model


def infer_shapes_static(model: Union[str, bytes, ol.Model], strict: bool = False) -> ol.Model:
    """The same result without running anything: the runtime's per-operator shape functions (C++,
    ``csrc/core/shape_inference*.cc``) walk the graph symbolically.  Dimensions they cannot resolve get ``unk__N``
    names; operators without a shape function leave their outputs without a shape."""
    from .. import _core
    if isinstance(model, ol.Model):
        data = model.serialize()
    elif isinstance(model, (bytes, bytearray)):
        data = bytes(model)
    else:
        with open(model, "rb") as f:
            data = f.read()
    out, report = _core.infer_shapes(data, strict)
    m = ol.load_model(out)
    m.shape_inference_report = report
    return m


def _torch_type(t) -> int:
    import torch
    return {torch.bfloat16: 16, torch.float16: 10, torch.float32: 1, torch.float64: 11, torch.int64: 7, torch.int32: 6,
            torch.bool: 9, torch.uint8: 2, torch.int8: 3}[t.dtype]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("input")
    ap.add_argument("output")
    ap.add_argument("--dim", action="append", default=[], help="name=value for a symbolic input dimension")
    ap.add_argument("--static", action="store_true", help="use the per-operator shape functions instead of tracing two runs")
    a = ap.parse_args(argv)
    dims = {k: int(v) for k, v in (d.split("=") for d in a.dim)}
    m = infer_shapes_static(a.input) if a.static else infer_shapes(a.input, dims)
    with open(a.output, "wb") as f:
        f.write(m.serialize())
    print(f"{len(m.graph.value_info)} value_info entries")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
