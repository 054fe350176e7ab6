"""Move TunableOp results between sessions and model files.

Counterpart of the reference's onnxruntime/python/tools/offline_tuning.py: ``extract`` reads the tuning results that a
session with tuning enabled wrote into the metadata of its optimized model (key ``tuning_results``) and writes them as
JSON; ``embed`` puts a JSON file into a model's metadata, so that a later session starts from it (with
``tunable_op_enable`` on and ``tunable_op_tuning_enable`` off)."""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, List, Optional

from .. import onnx_lite as ol

TUNING_RESULTS_KEY = "tuning_results"


def extract(model: ol.Model) -> Optional[List[Any]]:
    raw = model.metadata.get(TUNING_RESULTS_KEY)
    return None if raw is None else json.loads(raw)


def embed(model: ol.Model, tuning_results: List[Any], overwrite: bool = False) -> ol.Model:
    if TUNING_RESULTS_KEY in model.metadata and not overwrite:
        raise ValueError("the model already carries tuning results (pass overwrite=True / --force to replace them)")
    model.metadata[TUNING_RESULTS_KEY] = json.dumps(tuning_results)
    return model


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="offline_tuning")
    sub = ap.add_subparsers(dest="cmd", required=True)
    ex = sub.add_parser("extract", help="tuning results of a model -> JSON")
    ex.add_argument("input_onnx")
    ex.add_argument("output_json")
    em = sub.add_parser("embed", help="JSON tuning results -> model metadata")
    em.add_argument("--force", "-f", action="store_true")
    em.add_argument("output_onnx")
    em.add_argument("input_onnx")
    em.add_argument("input_json")
    pp = sub.add_parser("pprint", help="print the tuning results of a JSON file")
    pp.add_argument("json_path")
    args = ap.parse_args(argv)
    if args.cmd == "extract":
        res = extract(ol.load_model(args.input_onnx))
        if res is None:
            print("the model carries no tuning results", file=sys.stderr)
            return 1
        with open(args.output_json, "w") as f:
            json.dump(res, f, indent=1)
    elif args.cmd == "embed":
        with open(args.input_json) as f:
            res = json.load(f)
        model = embed(ol.load_model(args.input_onnx), res, overwrite=args.force)
        with open(args.output_onnx, "wb") as f:
            f.write(model.serialize())
    else:
        with open(args.json_path) as f:
            for entry in json.load(f):
                print(json.dumps(entry))
    return 0


if __name__ == "__main__":
    sys.exit(main())
