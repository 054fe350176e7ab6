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


C_SOURCE_WIDE = r"""
#include <stdio.h>
#include <string.h>
#include "ortb200_c_api.h"

#define CHECK(x) do { int rc_ = (x); if (rc_ != 0) { printf("ERR %d %s\n", rc_, ortb200_last_error()); return 1; } } while (0)

int main(int argc, char** argv) {
  ortb200_session_options* so = NULL;
  CHECK(ortb200_create_session_options(&so));
  CHECK(ortb200_session_options_set_graph_optimization_level(so, 1));
  CHECK(ortb200_session_options_set_intra_op_num_threads(so, 2));
  CHECK(ortb200_session_options_set_execution_mode(so, 0));
  CHECK(ortb200_session_options_set_log_id(so, "wide"));
  CHECK(ortb200_session_options_add_config_entry(so, "session.disable_prepacking", "1"));
  CHECK(ortb200_session_options_add_free_dimension_override_by_name(so, "batch", 2));
  CHECK(ortb200_session_options_append_execution_provider(so, "CPUExecutionProvider", NULL, NULL, 0));
  printf("badlevel %d\n", ortb200_session_options_set_graph_optimization_level(so, 7) != 0);
  ortb200_session* s = NULL;
  CHECK(ortb200_create_session_from_options(argv[1], NULL, 0, so, &s));
  ortb200_release_session_options(so);

  ortb200_type_info ti;
  CHECK(ortb200_session_input_type_info(s, 0, &ti));
  printf("in %d %d %d %lld %lld [%s]\n", ti.elem_type, ti.has_shape, ti.ndim, (long long)ti.dims[0], (long long)ti.dims[1], ti.dim_params[0]);
  CHECK(ortb200_session_output_type_info(s, 0, &ti));
  printf("out %d %d\n", ti.elem_type, ti.ndim);
  ortb200_model_metadata md;
  CHECK(ortb200_session_model_metadata(s, &md));
  const char* val = NULL;
  CHECK(ortb200_session_lookup_custom_metadata(s, "author", &val));
  const char* missing = "x";
  CHECK(ortb200_session_lookup_custom_metadata(s, "nope", &missing));
  const char* key0 = NULL;
  CHECK(ortb200_session_custom_metadata_key(s, 0, &key0));
  printf("meta %s %s %zu %s %s %d\n", md.producer_name, md.graph_name, md.num_custom_keys, key0, val, missing == NULL);
  size_t np_ = 0; const char* p0 = NULL;
  CHECK(ortb200_session_provider_count(s, &np_));
  CHECK(ortb200_session_provider_name(s, 0, &p0));
  printf("providers %zu %s\n", np_, p0);

  /* run with run options */
  float x[6] = {-1.f, 2.f, -3.f, 4.f, -5.f, 6.f};
  ortb200_tensor_view v; memset(&v, 0, sizeof(v));
  v.data = x; v.elem_type = 1; v.ndim = 2; v.dims[0] = 2; v.dims[1] = 3;
  const char* names[] = {"x"};
  ortb200_run_options* ro = NULL;
  CHECK(ortb200_create_run_options(&ro));
  CHECK(ortb200_run_options_set_tag(ro, "run-1"));
  ortb200_value* out = NULL;
  CHECK(ortb200_run_with_options(s, ro, names, &v, 1, NULL, 1, &out));
  float y[4]; size_t nbytes = 0;
  CHECK(ortb200_value_byte_size(out, &nbytes));
  CHECK(ortb200_value_copy_to_host(out, y, sizeof(y)));
  printf("run %zu %g %g %g %g\n", nbytes, y[0], y[1], y[2], y[3]);
  ortb200_release_value(out);
  CHECK(ortb200_run_options_set_terminate(ro, 1));
  printf("terminated %d\n", ortb200_run_with_options(s, ro, names, &v, 1, NULL, 1, &out) != 0);
  ortb200_release_run_options(ro);

  /* I/O binding with a runtime-owned input and a caller-owned output buffer */
  int64_t dims[2] = {2, 3};
  ortb200_value* xin = NULL;
  CHECK(ortb200_create_tensor(1, dims, 2, 0, 0, &xin));
  CHECK(ortb200_value_copy_from_host(xin, x, sizeof(x)));
  ortb200_tensor_view xv;
  CHECK(ortb200_value_tensor(xin, 0, &xv));
  float ybuf[4] = {0, 0, 0, 0};
  ortb200_tensor_view yv; memset(&yv, 0, sizeof(yv));
  yv.data = ybuf; yv.elem_type = 1; yv.ndim = 2; yv.dims[0] = 2; yv.dims[1] = 2;
  ortb200_io_binding* b = NULL;
  CHECK(ortb200_create_io_binding(s, &b));
  CHECK(ortb200_io_binding_bind_input(b, "x", &xv));
  CHECK(ortb200_io_binding_bind_output(b, "y", &yv));
  CHECK(ortb200_run_with_binding(s, NULL, b));
  CHECK(ortb200_io_binding_synchronize_outputs(b));
  size_t nout = 0; const char* oname = NULL;
  CHECK(ortb200_io_binding_output_count(b, &nout));
  CHECK(ortb200_io_binding_output_name(b, 0, &oname));
  printf("bound %zu %s %g %g %g %g\n", nout, oname, ybuf[0], ybuf[1], ybuf[2], ybuf[3]);
  CHECK(ortb200_io_binding_clear_outputs(b));
  CHECK(ortb200_io_binding_bind_output_to_device(b, "y", 0, 0));
  CHECK(ortb200_run_with_binding(s, NULL, b));
  ortb200_value* bound = NULL;
  CHECK(ortb200_io_binding_output_value(b, 0, &bound));
  ortb200_tensor_view bv;
  CHECK(ortb200_value_tensor(bound, 1, &bv));
  printf("bound2 %lld %lld %g\n", (long long)bv.dims[0], (long long)bv.dims[1], ((float*)bv.data)[3]);
  ortb200_release_value(bound);
  ortb200_release_io_binding(b);
  ortb200_release_value(xin);

  size_t navail = 0; const char* last = NULL;
  CHECK(ortb200_available_provider_count(&navail));
  CHECK(ortb200_available_provider_name(navail - 1, &last));
  printf("avail %d %s\n", navail >= 1, last);
  CHECK(ortb200_set_default_logger_severity(3));
  CHECK(ortb200_session_check_device_status(s));
  ortb200_release_session(s);
  return 0;
}
"""


@pytest.mark.skipif(not os.path.exists(os.path.join(LIB, "libortb200.so")), reason="libortb200.so not built")
def test_c_program_uses_options_metadata_and_io_binding(tmp_path):
    T = ol.TensorProto
    w = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], np.float32)
    g = ol.make_graph([ol.make_node("Relu", ["x"], ["r"]), ol.make_node("MatMul", ["r", "w"], ["y"])], "wide_graph",
                      [ol.make_tensor_value_info("x", T.FLOAT, ["batch", 3])], [ol.make_tensor_value_info("y", T.FLOAT, ["batch", 2])],
                      [ol.make_tensor("w", w)])
    m = ol.make_model(g, opset=17, producer_name="unit-test", metadata={"author": "someone"})
    model = tmp_path / "m.onnx"
    model.write_bytes(m.serialize())
    src = tmp_path / "wide.c"
    src.write_text(C_SOURCE_WIDE)
    exe = tmp_path / "wide"
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
    assert lines[0] == "badlevel 1"
    assert lines[1] == "in 1 1 2 2 3 []" or lines[1] == "in 1 1 2 -1 3 [batch]"   # the override pins the symbol
    assert lines[2] == "out 1 2"
    assert lines[3] == "meta unit-test wide_graph 1 author someone 1"
    assert lines[4] == "providers 1 CPUExecutionProvider"
    assert lines[5] == "run 16 0 2 10 6"
    assert lines[6] == "terminated 1"
    assert lines[7] == "bound 1 y 0 2 10 6"
    assert lines[8] == "bound2 2 2 6"
    assert lines[9] == "avail 1 CPUExecutionProvider"


C_SOURCE_STRINGS = r"""
#include <stdio.h>
#include <string.h>
#include "ortb200_c_api.h"

#define CHECK(x) do { int rc_ = (x); if (rc_ != 0) { printf("ERR %d %s\n", rc_, ortb200_last_error()); return 1; } } while (0)

int main(int argc, char** argv) {
  ortb200_session* s = NULL;
  CHECK(ortb200_create_session(argv[1], NULL, 0, "CPUExecutionProvider", 0, NULL, &s));
  const char* words[] = {"Monday", "tuesday", "WEDNESDAY", "monday"};
  int64_t dims[1] = {4};
  ortb200_value* in = NULL;
  CHECK(ortb200_create_string_tensor(words, dims, 1, &in));
  int is_str = 0;
  CHECK(ortb200_value_is_string(in, &is_str));
  const char* names[] = {"x"};
  ortb200_value* ins[] = {in};
  ortb200_value* outs[2] = {NULL, NULL};
  CHECK(ortb200_run_with_values(s, NULL, names, ins, 1, NULL, 2, outs));
  size_t n = 0;
  CHECK(ortb200_value_is_string(outs[0], &is_str));
  CHECK(ortb200_value_string_count(outs[0], &n));
  printf("strings %d %zu:", is_str, n);
  for (size_t i = 0; i < n; ++i) {
    const char* p; size_t len;
    CHECK(ortb200_value_string_element(outs[0], i, &p, &len));
    printf(" %s/%zu", p, len);
  }
  printf("\n");
  int64_t shape[8]; int32_t nd = 0;
  CHECK(ortb200_value_shape(outs[1], shape, &nd));
  CHECK(ortb200_value_is_string(outs[1], &is_str));
  ortb200_tensor_view v;
  CHECK(ortb200_value_tensor(outs[1], 1, &v));
  printf("ids %d %d %lld:", is_str, nd, (long long)shape[0]);
  for (int64_t i = 0; i < shape[0]; ++i) printf(" %lld", (long long)((int64_t*)v.data)[i]);
  printf("\n");
  int rc = ortb200_value_string_count(outs[1], &n);
  printf("not-strings %d\n", rc != 0);
  ortb200_release_value(in); ortb200_release_value(outs[0]); ortb200_release_value(outs[1]);
  ortb200_release_session(s);
  return 0;
}
"""


def test_c_program_feeds_and_reads_string_tensors(tmp_path):
    T = ol.TensorProto
    nodes = [ol.make_node("StringNormalizer", ["x"], ["y"], case_change_action="UPPER", stopwords=["monday"], is_case_sensitive=0),
             ol.make_node("LabelEncoder", ["y"], ["ids"], domain="ai.onnx.ml", keys_strings=["TUESDAY", "WEDNESDAY"], values_int64s=[2, 3], default_int64=-1)]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.STRING, ["n"])],
                      [ol.make_tensor_value_info("y", T.STRING, None), ol.make_tensor_value_info("ids", T.INT64, None)])
    m = ol.make_model(g, opset=17)
    m.opset_imports["ai.onnx.ml"] = 4
    model = tmp_path / "m.onnx"
    model.write_bytes(m.serialize())
    src = tmp_path / "client.c"
    src.write_text(C_SOURCE_STRINGS)
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
    assert lines[0] == "strings 1 2: TUESDAY/7 WEDNESDAY/9"
    assert lines[1] == "ids 0 1 2: 2 3"
    assert lines[2] == "not-strings 1"
