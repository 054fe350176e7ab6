// Python callables as operators (onnxruntime_b200.register_custom_op): the only part of the custom-operator support
// that needs the interpreter, kept apart so that the rest of the runtime links without Python.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "graph.h"
#include "kernel.h"

namespace py = pybind11;

namespace ortb {

namespace {
using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

py::dict AttrsToDict(const Node& n) {
  py::dict d;
  for (const auto& kv : n.attrs) {
    const pb::AttributeProto& a = kv.second;
    switch (a.type) {
      case 1: d[py::str(kv.first)] = a.f; break;
      case 2: d[py::str(kv.first)] = a.i; break;
      case 3: d[py::str(kv.first)] = py::bytes(a.s); break;
      case 4: d[py::str(kv.first)] = n.attr_tensor(kv.first); break;
      case 6: d[py::str(kv.first)] = a.floats; break;
      case 7: d[py::str(kv.first)] = a.ints; break;
      case 8: {
        py::list l;
        for (const auto& s : a.strings) l.append(py::bytes(s));
        d[py::str(kv.first)] = l;
        break;
      }
      default: break;
    }
  }
  return d;
}


}  // namespace

void RegisterPythonOp(const std::string& domain, const std::string& op, py::function fn) {
  EnsureKernelsRegistered();
  // the callable is leaked on purpose: the registry outlives the interpreter's teardown order
  auto* held = new py::function(std::move(fn));
  KernelRegistry::Generic().RegisterFn(domain, op, 1, kMax, [held, op](Ctx& ctx) {
    py::gil_scoped_acquire gil;
    py::list ins;
    for (int i = 0; i < ctx.InputCount(); ++i) {
      if (ctx.HasInput(i)) ins.append(py::cast(ctx.Input(i)));
      else ins.append(py::none());
    }
    py::object res;
    try {
      res = (*held)(*ins, **AttrsToDict(ctx.node()));
    } catch (py::error_already_set& e) {
      ORTB_THROW(FAIL, "custom op ", op, " raised: ", e.what());
    }
    auto set = [&](int i, const py::handle& h) {
      if (h.is_none()) return;
      ctx.SetOutput(i, h.cast<at::Tensor>());
    };
    if (py::isinstance<py::tuple>(res) || py::isinstance<py::list>(res)) {
      int i = 0;
      for (const py::handle& h : res) {
        if (i >= ctx.OutputCount()) break;
        set(i++, h);
      }
    } else {
      set(0, res);
    }
  });
}

}  // namespace ortb
