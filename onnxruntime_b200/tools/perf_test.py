"""``python -m onnxruntime_b200.tools.perf_test [options] model.onnx [result_file]``

Latency / throughput of a model through the public session API, with the flag names of the reference's
``onnxruntime_perf_test`` (onnxruntime/test/perftest/README.md, command_args_parser.cc):

  -e cpu|cuda      execution provider            -m duration|times   run for a time (-t) or a count (-r)
  -r N             repetitions (times mode)      -t S                seconds (duration mode)
  -o 0|1|2|99      graph optimization level      -c N                concurrent callers (threads sharing the session)
  -x N / -y N      intra / inter op threads      -P                  parallel executor
  -p FILE          write a chrome-trace profile  -u FILE             save the optimized model
  -C "k|v k|v"     session config entries        -f name:value       override a free dimension by name
  -I               generate inputs (the default when no test data directory is found)
  -q               capture the run into a CUDA graph (cuda provider; inputs bound with IOBinding)
  -w N             warm-up runs (default 1)      -s                  print per-run statistics
Reports the average and P50 / P90 / P95 / P99 / P999 latency and the throughput.
"""
from __future__ import annotations

import argparse
import json
import os
import threading
import time
from typing import Dict, List

import numpy as np

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol

_TYPE_TO_NP = {"tensor(float)": np.float32, "tensor(float16)": np.float16, "tensor(double)": np.float64, "tensor(int64)": np.int64,
               "tensor(int32)": np.int32, "tensor(int8)": np.int8, "tensor(uint8)": np.uint8, "tensor(bool)": np.bool_,
               "tensor(int16)": np.int16, "tensor(uint16)": np.uint16, "tensor(uint32)": np.uint32, "tensor(uint64)": np.uint64}


def generate_inputs(sess, free_dims: Dict[str, int], seed: int = 0) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    feeds = {}
    for i in sess.get_inputs():
        shape = [d if isinstance(d, int) and d > 0 else free_dims.get(d, 1) if isinstance(d, str) else 1 for d in (i.shape or [])]
        dt = _TYPE_TO_NP.get(i.type)
        if dt is None:
            raise SystemExit(f"cannot generate input {i.name!r} of type {i.type}")
        if np.issubdtype(dt, np.floating):
            feeds[i.name] = rng.rand(*shape).astype(dt)
        elif dt == np.bool_:
            feeds[i.name] = rng.rand(*shape) > 0.5
        else:
            feeds[i.name] = np.ones(shape, dtype=dt)
    return feeds


def load_test_data(model_path: str, sess) -> List[Dict[str, np.ndarray]]:
    """test_data_set_*/input_k.pb beside the model, in the model's input order."""
    base = os.path.dirname(os.path.abspath(model_path))
    sets = []
    names = [i.name for i in sess.get_inputs()]
    for d in sorted(os.listdir(base)):
        full = os.path.join(base, d)
        if not (d.startswith("test_data_set_") and os.path.isdir(full)):
            continue
        feeds = {}
        for k, name in enumerate(names):
            f = os.path.join(full, f"input_{k}.pb")
            if not os.path.exists(f):
                break
            t = ol.load_tensor(f)
            feeds[t.name or name] = ol.to_array(t)
        if len(feeds) == len(names):
            sets.append(feeds)
    return sets


def percentile(sorted_ms: List[float], p: float) -> float:
    if not sorted_ms:
        return float("nan")
    k = min(len(sorted_ms) - 1, max(0, int(round(p / 100.0 * len(sorted_ms) + 0.5)) - 1))
    return sorted_ms[k]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="perf_test", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model")
    ap.add_argument("result_file", nargs="?")
    ap.add_argument("-e", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("-m", default="times", choices=["duration", "times"])
    ap.add_argument("-r", type=int, default=100)
    ap.add_argument("-t", type=float, default=10.0)
    ap.add_argument("-o", type=int, default=99, choices=[0, 1, 2, 99])
    ap.add_argument("-c", type=int, default=1)
    ap.add_argument("-x", type=int, default=0)
    ap.add_argument("-y", type=int, default=0)
    ap.add_argument("-P", action="store_true")
    ap.add_argument("-p", default="")
    ap.add_argument("-u", default="")
    ap.add_argument("-C", default="")
    ap.add_argument("-f", action="append", default=[])
    ap.add_argument("-I", action="store_true")
    ap.add_argument("-q", action="store_true")
    ap.add_argument("-w", type=int, default=1)
    ap.add_argument("-s", action="store_true")
    a = ap.parse_args(argv)

    so = ort.SessionOptions()
    so.graph_optimization_level = {0: ort.GraphOptimizationLevel.ORT_DISABLE_ALL, 1: ort.GraphOptimizationLevel.ORT_ENABLE_BASIC,
                                   2: ort.GraphOptimizationLevel.ORT_ENABLE_EXTENDED, 99: ort.GraphOptimizationLevel.ORT_ENABLE_ALL}[a.o]
    if a.x:
        so.intra_op_num_threads = a.x
    if a.y:
        so.inter_op_num_threads = a.y
    if a.P:
        so.execution_mode = ort.ExecutionMode.ORT_PARALLEL
    if a.p:
        so.enable_profiling = True
        so.profile_file_prefix = a.p
    if a.u:
        so.optimized_model_filepath = a.u
    for kv in a.C.split():
        k, _, v = kv.partition("|")
        so.add_session_config_entry(k, v)
    free = {}
    for item in a.f:
        k, _, v = item.partition(":")
        free[k] = int(v)
        so.add_free_dimension_override_by_name(k, int(v))
    providers = ["CPUExecutionProvider"] if a.e == "cpu" else [("CUDAExecutionProvider", {"enable_cuda_graph": "1" if a.q else "0"}),
                                                               "CPUExecutionProvider"]
    t0 = time.perf_counter()
    sess = ort.InferenceSession(a.model, so, providers=providers)
    create_s = time.perf_counter() - t0

    data = [] if a.I else load_test_data(a.model, sess)
    if not data:
        data = [generate_inputs(sess, free)]

    binding = None
    if a.q and a.e == "cuda":
        import torch
        binding = sess.io_binding()
        for k, v in data[0].items():
            binding.bind_cpu_input(k, v)
        for o in sess.get_outputs():
            binding.bind_output(o.name, "cuda")
        run_one = lambda i: sess.run_with_iobinding(binding)  # noqa: E731
        sync = torch.cuda.synchronize
    else:
        run_one = lambda i: sess.run(None, data[i % len(data)])  # noqa: E731
        sync = (lambda: None)

    for i in range(max(a.w, 0)):
        run_one(i)
    sync()

    lat_ms: List[float] = []
    lock = threading.Lock()
    deadline = time.perf_counter() + a.t
    counter = [0]

    def worker():
        local = []
        while True:
            with lock:
                i = counter[0]
                if (a.m == "times" and i >= a.r) or (a.m == "duration" and time.perf_counter() >= deadline):
                    break
                counter[0] += 1
            s = time.perf_counter()
            run_one(i)
            sync()
            local.append((time.perf_counter() - s) * 1e3)
        with lock:
            lat_ms.extend(local)

    wall0 = time.perf_counter()
    threads = [threading.Thread(target=worker) for _ in range(max(a.c, 1))]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    wall = time.perf_counter() - wall0
    profile_file = sess.end_profiling() if a.p else ""

    lat_ms.sort()
    n = len(lat_ms)
    res = {"model": a.model, "provider": a.e, "runs": n, "session_creation_s": round(create_s, 4), "total_s": round(wall, 4),
           "avg_ms": round(sum(lat_ms) / max(n, 1), 4), "min_ms": round(lat_ms[0], 4) if n else None,
           "max_ms": round(lat_ms[-1], 4) if n else None, "p50_ms": round(percentile(lat_ms, 50), 4),
           "p90_ms": round(percentile(lat_ms, 90), 4), "p95_ms": round(percentile(lat_ms, 95), 4),
           "p99_ms": round(percentile(lat_ms, 99), 4), "p999_ms": round(percentile(lat_ms, 99.9), 4),
           "inferences_per_s": round(n / wall, 2) if wall > 0 else None, "concurrency": a.c}
    if profile_file:
        res["profile"] = profile_file
    print("Session creation time cost:", res["session_creation_s"], "s")
    print("Total inference time cost:", res["total_s"], "s")
    print("Total inference requests:", n)
    print("Average inference time cost:", res["avg_ms"], "ms")
    print("Number of inferences per second:", res["inferences_per_s"])
    print(f"P50 Latency: {res['p50_ms']} ms\nP90 Latency: {res['p90_ms']} ms\nP95 Latency: {res['p95_ms']} ms\n"
          f"P99 Latency: {res['p99_ms']} ms\nP999 Latency: {res['p999_ms']} ms")
    if a.s:
        print("latencies_ms:", [round(x, 3) for x in lat_ms])
    if a.result_file:
        with open(a.result_file, "w") as f:
            json.dump(res, f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
