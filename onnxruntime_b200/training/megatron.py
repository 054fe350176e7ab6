"""Tensor-parallel training: the conjugate pair of collectives of a Megatron-style split and the graph rewrite that
inserts them.

``com.microsoft.MegatronF`` is the identity going forward and an all-reduce of the gradient going backward (it sits
where a replicated activation enters a column-parallel weight); ``com.microsoft.MegatronG`` is an all-reduce going
forward and the identity going backward (it sits after a row-parallel weight).  The reference defines the two operators
in ``orttraining/orttraining/core/graph/training_op_defs.cc`` and inserts them with
``orttraining/orttraining/core/optimizer/megatron_transformer.cc``.  Here both are autograd functions over
``torch.distributed`` registered as operators of the session, so they work on the tape of ``ORTModule``; the collectives
run on whatever backend the default process group has (NCCL over NVLink for GPU tensors, gloo on the CPU).
"""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np
import torch

from .. import onnx_lite as ol

MS = "com.microsoft"


def _all_reduce(t: torch.Tensor) -> torch.Tensor:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = t.contiguous().clone()
        dist.all_reduce(t)
    return t


class _F(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g)


class _G(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _all_reduce(x)

    @staticmethod
    def backward(ctx, g):
        return g


def _register() -> None:
    from .. import capi
    try:
        capi.C.register_python_op(MS, "MegatronF", lambda x, **_: _F.apply(x))
        capi.C.register_python_op(MS, "MegatronG", lambda x, **_: _G.apply(x))
    except Exception:  # pragma: no cover - a build without Python operators
        pass


_register()


def shard_mlp(model: ol.Model, column_weights: Sequence[str], row_weights: Sequence[str], rank: int, world: int,
              column_biases: Sequence[str] = ()) -> ol.Model:
    """Splits the named [K, N] weights of ``MatMul`` nodes over ``world`` ranks and keeps rank ``rank``'s shard:
    ``column_weights`` (and their biases) by columns, with ``MegatronF`` on the activation that enters them;
    ``row_weights`` by rows, with ``MegatronG`` on the product that leaves them."""
    g = model.graph
    col, row = set(column_weights), set(row_weights)
    for t in list(g.initializers):
        if t.name in col or t.name in row or t.name in column_biases:
            arr = np.array(ol.to_array(t))
            axis = (arr.ndim - 1) if (t.name in col or t.name in column_biases) else 0
            assert arr.shape[axis] % world == 0, f"{t.name}: {arr.shape[axis]} does not divide over {world} ranks"
            piece = np.ascontiguousarray(np.split(arr, world, axis)[rank])
            g.initializers[g.initializers.index(t)] = ol.make_tensor(t.name, piece)
    nodes = []
    entered: Dict[str, str] = {}
    for n in g.nodes:
        if n.op_type == "MatMul" and n.inputs[1] in col:
            src = n.inputs[0]
            if src not in entered:
                entered[src] = src + "_megatron_f"
                nodes.append(ol.make_node("MegatronF", [src], [entered[src]], name="MegatronF_" + src, domain=MS))
            n.inputs[0] = entered[src]
            nodes.append(n)
        elif n.op_type == "MatMul" and n.inputs[1] in row:
            out = n.outputs[0]
            n.outputs[0] = out + "_partial"
            nodes.append(n)
            nodes.append(ol.make_node("MegatronG", [n.outputs[0]], [out], name="MegatronG_" + out, domain=MS))
        else:
            nodes.append(n)
    g.nodes[:] = nodes
    model.opset_imports.setdefault(MS, 1)
    return model
