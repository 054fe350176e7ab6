"""``python -m onnxruntime_b200.tools.onnx_test_runner [-e cpu|cuda] [-j N] [--rtol R --atol A] <dir> [<dir> ...]``

Runs ONNX test-data directories: every directory that holds ``model.onnx`` (or a single ``*.onnx``) and
``test_data_set_*/input_k.pb`` + ``output_k.pb`` TensorProto files is loaded, run, and its outputs compared with the
expected ones - the layout and the job of the reference's ``onnx_test_runner`` (onnxruntime/test/onnx/main.cc,
TestCase.cc).  Exit code 0 when every case passes.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Tuple

import numpy as np

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol


def find_cases(roots: List[str]) -> List[Tuple[str, str]]:
    cases = []
    for root in roots:
        for d, _, files in os.walk(root):
            models = [f for f in files if f.endswith(".onnx")]
            if not models:
                continue
            model = "model.onnx" if "model.onnx" in models else models[0]
            if any(x.startswith("test_data_set_") for x in os.listdir(d)):
                cases.append((os.path.basename(d), os.path.join(d, model)))
    return sorted(cases)


def _as_np(x):
    if isinstance(x, np.ndarray):
        return x
    return x.float().numpy()  # torch tensor (bf16 / fp8 payloads)


def run_case(name: str, model_path: str, providers, rtol: float, atol: float) -> Tuple[int, int, List[str]]:
    errors: List[str] = []
    try:
        sess = ort.InferenceSession(model_path, providers=providers)
    except Exception as e:  # noqa: BLE001
        return 0, 1, [f"{name}: load failed: {e}"]
    in_names = [i.name for i in sess.get_inputs()]
    out_names = [o.name for o in sess.get_outputs()]
    base = os.path.dirname(model_path)
    passed = failed = 0
    for d in sorted(os.listdir(base)):
        full = os.path.join(base, d)
        if not (d.startswith("test_data_set_") and os.path.isdir(full)):
            continue
        feeds, expected = {}, {}
        for f in sorted(os.listdir(full)):
            if not f.endswith(".pb"):
                continue
            t = ol.load_tensor(os.path.join(full, f))
            idx = int(f.split("_")[1].split(".")[0])
            if f.startswith("input_"):
                feeds[t.name or in_names[idx]] = ol.to_array(t)
            elif f.startswith("output_"):
                expected[t.name or out_names[idx]] = ol.to_array(t)
        try:
            got = sess.run(list(expected.keys()), feeds)
            ok = True
            for (k, want), have in zip(expected.items(), got):
                w, h = _as_np(want), np.asarray(have)
                if w.shape != h.shape:
                    ok = False
                    errors.append(f"{name}/{d}: output {k} shape {h.shape}, expected {w.shape}")
                elif w.dtype.kind in "fc":
                    if not np.allclose(h.astype(np.float64), w.astype(np.float64), rtol=rtol, atol=atol, equal_nan=True):
                        ok = False
                        errors.append(f"{name}/{d}: output {k} max abs diff {np.abs(h.astype(np.float64) - w.astype(np.float64)).max():.3g}")
                elif not np.array_equal(h, w):
                    ok = False
                    errors.append(f"{name}/{d}: output {k} differs")
            passed += ok
            failed += not ok
        except Exception as e:  # noqa: BLE001
            failed += 1
            errors.append(f"{name}/{d}: run failed: {e}")
    return passed, failed, errors


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="onnx_test_runner")
    ap.add_argument("dirs", nargs="+")
    ap.add_argument("-e", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("-j", type=int, default=1, help="accepted for compatibility; cases run one after another")
    ap.add_argument("--rtol", type=float, default=1e-3)
    ap.add_argument("--atol", type=float, default=1e-5)
    a = ap.parse_args(argv)
    providers = ["CPUExecutionProvider"] if a.e == "cpu" else ["CUDAExecutionProvider", "CPUExecutionProvider"]
    cases = find_cases(a.dirs)
    total_p = total_f = 0
    for name, path in cases:
        p, f, errs = run_case(name, path, providers, a.rtol, a.atol)
        total_p += p
        total_f += f
        for e in errs:
            print("FAILED", e, file=sys.stderr)
    print(f"result: models {len(cases)}, data sets passed {total_p}, failed {total_f}")
    return 0 if total_f == 0 and cases else 1


if __name__ == "__main__":
    raise SystemExit(main())
