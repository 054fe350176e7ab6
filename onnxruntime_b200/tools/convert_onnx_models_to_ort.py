"""Convert ONNX models to the ORT format (``.ort``), optionally optimizing them first.

Counterpart of the reference's ``python -m onnxruntime.tools.convert_onnx_models_to_ort``
(tools/python/util/convert_onnx_models_to_ort.py): for every ``*.onnx`` file under the given path a ``.ort`` file is
written beside it (or into ``--output_dir``).

    python -m onnxruntime_b200.tools.convert_onnx_models_to_ort model_or_dir [--optimization_style Fixed|Runtime]
                                                                             [--optimization_level basic|extended|all|disable]
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List

LEVELS = {"disable": 0, "basic": 1, "extended": 2, "all": 99}


def convert(onnx_path: str, ort_path: str, level: str = "all") -> None:
    import onnxruntime_b200 as ort
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel(LEVELS[level]) if LEVELS[level] != 99 else ort.GraphOptimizationLevel.ORT_ENABLE_ALL
    so.optimized_model_filepath = ort_path
    so.add_session_config_entry("session.save_model_format", "ORT")
    ort.InferenceSession(onnx_path, so, providers=["CPUExecutionProvider"])


def main(argv: List[str] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("model_path_or_dir")
    ap.add_argument("--output_dir", default=None)
    ap.add_argument("--optimization_level", default="all", choices=sorted(LEVELS))
    ap.add_argument("--optimization_style", default="Fixed", choices=["Fixed", "Runtime"],
                    help="Runtime keeps the graph unoptimized so that a later session optimizes for its own device")
    args = ap.parse_args(argv)
    level = "disable" if args.optimization_style == "Runtime" else args.optimization_level
    paths = []
    if os.path.isdir(args.model_path_or_dir):
        for root, _, files in os.walk(args.model_path_or_dir):
            paths += [os.path.join(root, f) for f in sorted(files) if f.endswith(".onnx")]
    else:
        paths = [args.model_path_or_dir]
    for p in paths:
        base = os.path.splitext(os.path.basename(p))[0] + ".ort"
        out = os.path.join(args.output_dir or os.path.dirname(p) or ".", base)
        os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
        convert(p, out, level)
        print(f"{p} -> {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
