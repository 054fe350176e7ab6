"""``SymbolicShapeInference`` under the reference's name (onnxruntime/python/tools/symbolic_shape_infer.py).

``SymbolicShapeInference.infer_shapes(model, int_max, auto_merge, guess_output_rank, verbose)`` returns the model with
``value_info`` filled in for every intermediate value: first the schema-driven static pass (types and the shapes it can
prove), then, for values that pass leaves open, shapes observed by tracing the model on random inputs with the symbolic
input dimensions set to two different small values each, so that dimensions that follow an input dimension are
reported under its name.  The contrib operators the reference's tool special-cases (Attention, GroupQueryAttention,
MatMulNBits, SkipLayerNormalization ...) run through their kernels here, so they need no per-operator rule."""
from __future__ import annotations

import argparse
import sys
from typing import Union

from .. import onnx_lite as ol
from . import shape_inference as si


class SymbolicShapeInference:
    @staticmethod
    def infer_shapes(in_mp: Union[str, bytes, ol.Model], int_max: int = 2 ** 31 - 1, auto_merge: bool = False, guess_output_rank: bool = False,
                     verbose: int = 0) -> ol.Model:
        model = in_mp if isinstance(in_mp, ol.Model) else ol.load_model(in_mp)
        try:
            model = si.infer_shapes_static(model)
        except Exception as e:  # the static pass is best effort: tracing below still answers
            if verbose:
                print(f"static pass stopped: {e}", file=sys.stderr)
        known = {v.name for v in model.graph.value_info if v.elem_type and v.shape is not None}
        produced = {o for n in model.graph.nodes for o in n.outputs if o}
        if produced - known - {o.name for o in model.graph.outputs}:
            try:
                model = si.infer_shapes(model)
            except Exception as e:
                if verbose:
                    print(f"tracing pass stopped: {e}", file=sys.stderr)
        return model


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="symbolic_shape_infer")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--auto_merge", action="store_true")
    ap.add_argument("--int_max", type=int, default=2 ** 31 - 1)
    ap.add_argument("--guess_output_rank", action="store_true")
    ap.add_argument("--verbose", type=int, default=0)
    a = ap.parse_args(argv)
    out = SymbolicShapeInference.infer_shapes(a.input, a.int_max, a.auto_merge, a.guess_output_rank, a.verbose)
    with open(a.output, "wb") as f:
        f.write(out.serialize())
    return 0


if __name__ == "__main__":
    sys.exit(main())
