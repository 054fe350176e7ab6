"""ORTModule: an ONNX graph as a trainable ``torch.nn.Module``.

The reference's ``ORTModule`` (``orttraining/orttraining/python/training/ortmodule/ortmodule.py``) exports a torch
module to ONNX, builds a gradient graph and runs both halves in its own session behind a ``torch.autograd.Function``.
Here the direction is the other one, because the generic kernels of the native session are compositions of
tensor-library calls: the float initializers of the graph become ``torch.nn.Parameter``s, each forward pass feeds them
to the session as overriding inputs, and autograd records through the kernels, so ``loss.backward()`` and every
``torch.optim`` optimizer work unchanged.  A session on the CUDA provider is created with ``ortb200.generic_kernels_only`` so that every node runs on the
differentiable tensor-library kernels (the hand-written sm_100a kernels are inference-only)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from .. import onnx_lite as ol


def _safe(name: str) -> str:
    return name.replace(".", "__").replace("/", "__").replace(":", "__")


def lift_initializers(model: ol.Model, names: Sequence[str]) -> ol.Model:
    """Turns the named initializers into graph inputs (so that nothing folds them into constants)."""
    g = model.graph
    chosen = set(names)
    kept = []
    for t in g.initializers:
        if t.name in chosen:
            if not any(v.name == t.name for v in g.inputs):
                g.inputs.append(ol.make_tensor_value_info(t.name, t.data_type, list(t.dims)))
        else:
            kept.append(t)
    g.initializers[:] = kept
    return model


class ORTModule(torch.nn.Module):
    def __init__(self, model: Union[str, bytes, ol.Model], trainable: Optional[Sequence[str]] = None,
                 providers: Sequence[str] = ("CPUExecutionProvider",), output_names: Optional[Sequence[str]] = None,
                 recompute: bool = False):
        """``recompute=True`` keeps no activations of the graph between the forward and the backward pass: the forward
        pass runs without recording and is run again, recording, when the gradients are asked for (the trade the
        reference's memory optimizer makes per subgraph, made here for the whole graph)."""
        super().__init__()
        self._recompute = bool(recompute)
        import copy
        from .. import capi
        m = copy.deepcopy(model) if isinstance(model, ol.Model) else ol.load_model(model)
        floats = (ol.TensorProto.FLOAT, ol.TensorProto.FLOAT16, ol.TensorProto.BFLOAT16, ol.TensorProto.DOUBLE)
        # by default every float initializer with more than one element: one-element floats are the constants of the
        # graph (an exponent, an epsilon, a scale), not weights
        names = [t.name for t in m.graph.initializers if t.data_type in floats and
                 ((trainable is None and int(np.prod(t.dims)) > 1) or (trainable is not None and t.name in trainable))]
        self._param_names: List[str] = names
        self._attr_of: Dict[str, str] = {}
        for t in m.graph.initializers:
            if t.name in names:
                arr = ol.to_array(t)
                value = arr if isinstance(arr, torch.Tensor) else torch.from_numpy(np.array(arr))
                attr = _safe(t.name)
                self._attr_of[t.name] = attr
                self.register_parameter(attr, torch.nn.Parameter(value.clone()))
        lift_initializers(m, names)
        self._input_names = [v.name for v in m.graph.inputs if v.name not in names]
        so = capi.SessionOptions()
        so.graph_optimization_level = capi.GraphOptimizationLevel.ORT_ENABLE_BASIC
        so.add_session_config_entry("ortb200.generic_kernels_only", "1")
        self._session = capi.InferenceSession(m.serialize(), so, providers=list(providers))
        self._outputs = list(output_names) if output_names else [o.name for o in self._session.get_outputs()]
        self._C = capi.C

    @property
    def input_names(self) -> List[str]:
        return list(self._input_names)

    def named_onnx_parameters(self):
        for name in self._param_names:
            yield name, getattr(self, self._attr_of[name])

    def forward(self, *inputs, **named):
        feeds = dict(zip(self._input_names, inputs))
        feeds.update(named)
        missing = [n for n in self._input_names if n not in feeds]
        if missing:
            raise ValueError(f"missing inputs {missing}")
        names = list(feeds) + self._param_names
        values = [v if isinstance(v, torch.Tensor) else torch.as_tensor(np.asarray(v)) for v in feeds.values()]
        values += [getattr(self, self._attr_of[n]) for n in self._param_names]
        def run(*tensors):
            outs = self._session._sess.run(self._C.RunOptions(), names, list(tensors), self._outputs)
            return outs[0] if len(outs) == 1 else tuple(outs)
        if self._recompute and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint, set_checkpoint_early_stop
            # no early stop: it works by raising a Python exception from a saved-tensor hook, which here would fire
            # in the middle of a native kernel
            with set_checkpoint_early_stop(False):
                return checkpoint(run, *values, use_reentrant=False)
        return run(*values)
