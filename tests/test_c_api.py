"""The C API (csrc/core/ortb200_c_api.h, lib/libortb200.so): a C program with no Python in its process loads a
model, runs it and reads the result, the way a client of the reference's onnxruntime_c_api.h does."""
import os
import subprocess
import sys

import numpy as np
import pytest

import onnxruntime_b200
from onnxruntime_b200 import onnx_lite as ol

PKG = os.path.dirname(onnxruntime_b200.__file__)
LIB = os.path.join(PKG, "lib")
INC = os.path.join(PKG, "csrc", "core")

C_SOURCE = r"""
#include <stdio.h>
#include <string.h>
#include "ortb200_c_api.h"

#define CHECK(x) do { int rc_ = (x); if (rc_ != 0) { printf("ERR %d %s\n", rc_, ortb200_last_error()); return 1; } } while (0)

int main(int argc, char** argv) {
  ortb200_session* s = NULL;
  const char* config[] = {"graph_optimization_level", "99", "logid", "c-client", NULL};
  CHECK(ortb200_create_session(argv[1], NULL, 0, "CPUExecutionProvider", 0, config, &s));
  size_t n_in = 0, n_out = 0;
  CHECK(ortb200_session_input_count(s, &n_in));
  CHECK(ortb200_session_output_count(s, &n_out));
  const char *in0, *out0;
  CHECK(ortb200_session_input_name(s, 0, &in0));
  CHECK(ortb200_session_output_name(s, 0, &out0));
  printf("io %zu %zu %s %s\n", n_in, n_out, in0, out0);
  float x[6] = {-1.f, 2.f, -3.f, 4.f, -5.f, 6.f};
  ortb200_tensor_view v;
  memset(&v, 0, sizeof(v));
  v.data = x; v.elem_type = 1; v.ndim = 2; v.dims[0] = 2; v.dims[1] = 3;
  const char* names[] = {in0};
  ortb200_value* out = NULL;
  CHECK(ortb200_run(s, names, &v, 1, NULL, 1, &out));
  ortb200_tensor_view y;
  CHECK(ortb200_value_tensor(out, 1, &y));
  printf("out %d %d %lld %lld:", y.elem_type, y.ndim, (long long)y.dims[0], (long long)y.dims[1]);
  for (int i = 0; i < y.dims[0] * y.dims[1]; ++i) printf(" %g", ((float*)y.data)[i]);
  printf("\n");
  ortb200_release_value(out);
  /* an error path: unknown input name */
  const char* bad[] = {"nope"};
  int rc = ortb200_run(s, bad, &v, 1, NULL, 1, &out);
  printf("bad %d %s\n", rc != 0, ortb200_last_error());
  ortb200_release_session(s);
  rc = ortb200_create_session("/nonexistent/model.onnx", NULL, 0, NULL, 0, NULL, &s);
  printf("missing %d\n", rc != 0);
  return 0;
}
"""


@pytest.mark.skipif(not os.path.exists(os.path.join(LIB, "libortb200.so")), reason="libortb200.so not built")
def test_c_program_runs_a_model(tmp_path):
    T = ol.TensorProto
    w = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], np.float32)
    g = ol.make_graph([ol.make_node("Relu", ["x"], ["r"]), ol.make_node("MatMul", ["r", "w"], ["y"])], "g",
                      [ol.make_tensor_value_info("x", T.FLOAT, [2, 3])], [ol.make_tensor_value_info("y", T.FLOAT, [2, 2])],
                      [ol.make_tensor("w", w)])
    model = tmp_path / "m.onnx"
    model.write_bytes(ol.make_model(g, opset=17).serialize())
    src = tmp_path / "client.c"
    src.write_text(C_SOURCE)
    exe = tmp_path / "client"
    import torch
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["gcc", "-std=c99", "-o", str(exe), str(src), f"-I{INC}", f"-L{LIB}", "-lortb200", f"-Wl,-rpath,{LIB}",
           f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath-link,{torch_lib}", f"-Wl,-rpath-link,{LIB}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    run = subprocess.run([str(exe), str(model)], capture_output=True, text=True, env=env, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    lines = run.stdout.strip().splitlines()
    assert lines[0] == "io 1 1 x y"
    x = np.array([[-1, 2, -3], [4, -5, 6]], np.float32)
    want = np.maximum(x, 0) @ w
    assert lines[1] == "out 1 2 2 2: " + " ".join(f"{v:g}" for v in want.reshape(-1))
    assert lines[2].startswith("bad 1 ") and "nope" in lines[2]
    assert lines[3] == "missing 1"
