// pybind11 module `onnxruntime_b200._core`: the native runtime exposed to the
// Python API shell (reference: onnxruntime/python/onnxruntime_pybind_state.cc).
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "string_table.h"
#include "logging.h"
#include "executor.h"
#include "graph.h"
#include "kernel.h"
#include <c10/cuda/CUDACachingAllocator.h>

#include "session.h"
#include "shape_inference.h"
#include "cuda_ops.h"
#include "sharding_spec.h"

namespace py = pybind11;
using namespace ortb;

namespace ortb {
void RegisterPythonOp(const std::string& domain, const std::string& op, pybind11::function fn);
void LoadCustomOpLibrary(const std::string& path);
}  // namespace ortb

namespace {

struct PyOrtError {
  int code;
  std::string msg;
};

py::object g_error_factory;  // python callable (code:int, message:str) -> exception instance

void TranslateAndThrow(const OrtError& e) {
  if (g_error_factory && !g_error_factory.is_none()) {
    py::object exc = g_error_factory(static_cast<int>(e.code()), std::string(e.what()));
    PyErr_SetObject(reinterpret_cast<PyObject*>(Py_TYPE(exc.ptr())), exc.ptr());
    throw py::error_already_set();
  }
  throw std::runtime_error(e.what());
}

std::vector<Value> ToValues(const std::vector<py::object>& objs) {
  std::vector<Value> out;
  out.reserve(objs.size());
  for (auto& o : objs) {
    Value v;
    if (o.is_none()) {
    } else if (py::hasattr(o, "strings") && py::hasattr(o, "shape") && !py::hasattr(o, "dtype")) {
      // capi._StringTensor: strings + shape -> ids of the string table
      v.t = InternStrings(o.attr("strings").cast<std::vector<std::string>>(), o.attr("shape").cast<std::vector<int64_t>>());
      v.is_string = true;
    } else if (py::isinstance<py::dict>(o)) {
      // one map: int64 or string keys, numeric or string values (ai.onnx.ml CastMap / DictVectorizer inputs)
      py::dict d = o.cast<py::dict>();
      auto m = std::make_shared<MapRows>();
      std::vector<int64_t> keys;
      std::vector<double> vals;
      std::vector<int64_t> string_vals;
      bool values_are_strings = false;
      for (auto kv : d) {
        if (py::isinstance<py::str>(kv.first)) {
          m->string_keys = true;
          keys.push_back(InternString(kv.first.cast<std::string>()));
        } else {
          keys.push_back(kv.first.cast<int64_t>());
        }
        if (py::isinstance<py::str>(kv.second)) {
          values_are_strings = true;
          string_vals.push_back(InternString(kv.second.cast<std::string>()));
        } else {
          vals.push_back(kv.second.cast<double>());
        }
      }
      m->keys = at::tensor(keys, at::kLong);
      if (values_are_strings) {
        m->values = at::tensor(string_vals, at::kLong).reshape({1, -1});
        m->string_values = true;
      } else {
        m->values = at::tensor(vals, at::kDouble).reshape({1, -1});
      }
      v.maps = std::move(m);
    } else if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o)) {
      v.seq = std::make_shared<std::vector<at::Tensor>>(o.cast<std::vector<at::Tensor>>());
    } else {
      v.t = o.cast<at::Tensor>();
    }
    out.push_back(std::move(v));
  }
  return out;
}

py::object FromValue(const Value& v) {
  if (v.seq) return py::cast(*v.seq);
  if (v.maps) {
    // a list of dicts, one per row
    at::Tensor vals = v.maps->values.to(at::kCPU, at::kFloat).contiguous();
    at::Tensor keys = v.maps->keys.to(at::kCPU, at::kLong).contiguous();
    const int64_t N = vals.size(0), C = vals.size(1);
    std::vector<py::object> names;
    for (int64_t c = 0; c < C; ++c) {
      const int64_t k = keys.data_ptr<int64_t>()[c];
      names.push_back(v.maps->string_keys ? py::object(py::str(StringOfId(k))) : py::object(py::int_(k)));
    }
    py::list rows;
    for (int64_t i = 0; i < N; ++i) {
      py::dict d;
      for (int64_t c = 0; c < C; ++c) d[names[static_cast<size_t>(c)]] = py::float_(vals.data_ptr<float>()[i * C + c]);
      rows.append(d);
    }
    return rows;
  }
  if (v.t.defined() && v.is_string) return py::make_tuple(py::str("__strings__"), StringsOfTensor(v.t), v.t.sizes().vec());
  if (v.t.defined()) return py::cast(v.t);
  return py::none();
}

py::dict NodeToDict(const Node& n) {
  py::dict d;
  d["name"] = n.name;
  d["op_type"] = n.op_type;
  d["domain"] = n.domain;
  d["inputs"] = n.inputs;
  d["outputs"] = n.outputs;
  d["ep"] = n.ep;
  py::dict attrs;
  for (auto& kv : n.attrs) {
    const auto& a = kv.second;
    switch (a.type) {
      case pb::ATTR_INT: attrs[kv.first.c_str()] = a.i; break;
      case pb::ATTR_FLOAT: attrs[kv.first.c_str()] = a.f; break;
      case pb::ATTR_STRING: attrs[kv.first.c_str()] = py::bytes(a.s); break;
      case pb::ATTR_INTS: attrs[kv.first.c_str()] = a.ints; break;
      case pb::ATTR_FLOATS: attrs[kv.first.c_str()] = a.floats; break;
      case pb::ATTR_STRINGS: attrs[kv.first.c_str()] = a.strings; break;
      case pb::ATTR_TENSOR: attrs[kv.first.c_str()] = n.attr_tensor(kv.first); break;
      default: attrs[kv.first.c_str()] = py::none();
    }
  }
  d["attrs"] = attrs;
  return d;
}

template <typename F>
auto Guard(F&& f) -> decltype(f()) {
  try {
    return f();
  } catch (const OrtError& e) {
    TranslateAndThrow(e);
    throw;
  } catch (const c10::Error& e) {
    TranslateAndThrow(OrtError(StatusCode::RUNTIME_EXCEPTION, e.what_without_backtrace()));
    throw;
  }
}

}  // namespace

PYBIND11_MODULE(_core, m) {
  m.doc() = "onnxruntime_b200 native runtime";
  m.def("set_error_factory", [](py::object f) { g_error_factory = f; });
  m.def("set_default_logger_severity", [](int s) { logging::Manager::Get().set_default_severity(s); });
  m.def("set_default_logger_verbosity", [](int v) { logging::Manager::Get().set_default_verbosity(v); });
  // sink(severity, logger_id, formatted_line); None restores stderr
  m.def("set_log_sink", [](py::object fn) {
    if (fn.is_none()) {
      logging::Manager::Get().SetSink(nullptr);
      return;
    }
    auto holder = std::make_shared<py::object>(fn);
    logging::Manager::Get().SetSink([holder](const logging::Record& r) {
      py::gil_scoped_acquire gil;
      (*holder)(static_cast<int>(r.severity), r.logger_id, logging::Manager::Format(r));
    });
  });
  m.def("log_message", [](int severity, const std::string& id, const std::string& msg) {
    logging::Logger lg(id, -1, -1);
    if (lg.Enabled(static_cast<logging::Severity>(severity)))
      logging::Manager::Get().Emit({static_cast<logging::Severity>(severity), id, "python", "", msg, 0});
  });
  m.def("registered_ops", [](const std::string& which) {
    EnsureKernelsRegistered();
    return which == "cuda" ? KernelRegistry::Cuda().ListOps() : KernelRegistry::Generic().ListOps();
  });

  py::class_<SessionOptions>(m, "SessionOptions")
      .def(py::init<>())
      .def_readwrite("enable_cpu_mem_arena", &SessionOptions::enable_cpu_mem_arena)
      .def_readwrite("enable_mem_pattern", &SessionOptions::enable_mem_pattern)
      .def_readwrite("enable_mem_reuse", &SessionOptions::enable_mem_reuse)
      .def_readwrite("enable_profiling", &SessionOptions::enable_profiling)
      .def_readwrite("profile_file_prefix", &SessionOptions::profile_file_prefix)
      .def_readwrite("optimized_model_filepath", &SessionOptions::optimized_model_filepath)
      .def_readwrite("logid", &SessionOptions::logid)
      .def_readwrite("log_severity_level", &SessionOptions::log_severity_level)
      .def_readwrite("log_verbosity_level", &SessionOptions::log_verbosity_level)
      .def_readwrite("intra_op_num_threads", &SessionOptions::intra_op_num_threads)
      .def_readwrite("inter_op_num_threads", &SessionOptions::inter_op_num_threads)
      .def_readwrite("execution_mode", &SessionOptions::execution_mode)
      .def_readwrite("execution_order", &SessionOptions::execution_order)
      .def_readwrite("graph_optimization_level", &SessionOptions::graph_optimization_level)
      .def_readwrite("use_deterministic_compute", &SessionOptions::use_deterministic_compute)
      .def_readwrite("use_per_session_threads", &SessionOptions::use_per_session_threads)
      .def("add_config", [](SessionOptions& s, const std::string& k, const std::string& v) { s.config.entries[k] = v; })
      .def("get_config", [](SessionOptions& s, const std::string& k) -> py::object {
        auto it = s.config.entries.find(k);
        if (it == s.config.entries.end()) return py::none();
        return py::cast(it->second);
      })
      .def("config_entries", [](SessionOptions& s) { return s.config.entries; })
      .def("add_free_dim_by_name", [](SessionOptions& s, const std::string& k, int64_t v) { s.free_dim_by_name[k] = v; })
      .def("add_free_dim_by_denotation", [](SessionOptions& s, const std::string& k, int64_t v) { s.free_dim_by_denotation[k] = v; })
      .def("add_initializer", [](SessionOptions& s, const std::string& k, const at::Tensor& t) { s.initializers[k] = t; })
      .def("add_external_initializer", [](SessionOptions& s, const std::string& k, const at::Tensor& t) { s.external_initializers[k] = t; });

  py::class_<RunOptions>(m, "RunOptions")
      .def(py::init<>())
      .def_readwrite("log_severity_level", &RunOptions::log_severity_level)
      .def_readwrite("log_verbosity_level", &RunOptions::log_verbosity_level)
      .def_readwrite("logid", &RunOptions::logid)
      .def_readwrite("only_execute_path_to_fetches", &RunOptions::only_execute_path_to_fetches)
      .def_property("terminate", [](RunOptions& r) { return r.terminate->load(); },
                    [](RunOptions& r, bool v) { r.terminate->store(v); })
      .def("add_config", [](RunOptions& r, const std::string& k, const std::string& v) { r.config.entries[k] = v; })
      .def("get_config", [](RunOptions& r, const std::string& k) -> py::object {
        auto it = r.config.entries.find(k);
        if (it == r.config.entries.end()) return py::none();
        return py::cast(it->second);
      });

  py::class_<NodeArgMeta>(m, "NodeArgMeta")
      .def_readonly("name", &NodeArgMeta::name)
      .def_readonly("type", &NodeArgMeta::type)
      .def_readonly("has_shape", &NodeArgMeta::has_shape)
      .def_readonly("shape", &NodeArgMeta::shape)
      .def_readonly("sym", &NodeArgMeta::sym);

  py::class_<InferenceSession>(m, "InferenceSession")
      .def(py::init<const SessionOptions&>())
      .def("load", [](InferenceSession& s, const std::string& path) { Guard([&] { s.Load(path); return 0; }); })
      .def("load_bytes", [](InferenceSession& s, py::bytes b) {
        std::string bytes = b;
        Guard([&] { s.LoadFromBytes(bytes); return 0; });
      })
      .def("initialize",
           [](InferenceSession& s, const std::vector<std::pair<std::string, ProviderOptions>>& providers,
              const std::vector<std::string>& disabled) {
             py::gil_scoped_release rel;
             try {
               s.Initialize(providers, disabled);
             } catch (const OrtError& e) {
               py::gil_scoped_acquire acq;
               TranslateAndThrow(e);
             } catch (const c10::Error& e) {
               py::gil_scoped_acquire acq;
               TranslateAndThrow(OrtError(StatusCode::RUNTIME_EXCEPTION, e.what_without_backtrace()));
             }
           })
      .def("run",
           [](InferenceSession& s, const RunOptions& ro, const std::vector<std::string>& names,
              const std::vector<py::object>& feeds, const std::vector<std::string>& outputs) {
             std::vector<Value> vals = ToValues(feeds);
             std::vector<Value> res;
             {
               py::gil_scoped_release rel;
               try {
                 res = s.Run(ro, names, vals, outputs);
               } catch (const OrtError& e) {
                 py::gil_scoped_acquire acq;
                 TranslateAndThrow(e);
               } catch (const c10::Error& e) {
                 py::gil_scoped_acquire acq;
                 TranslateAndThrow(OrtError(StatusCode::RUNTIME_EXCEPTION, e.what_without_backtrace()));
               }
             }
             py::list out;
             for (auto& v : res) out.append(FromValue(v));
             return out;
           })
      .def("run_with_binding",
           [](InferenceSession& s, const RunOptions& ro, IOBinding& b) {
             py::gil_scoped_release rel;
             try {
               s.RunWithBinding(ro, b);
             } catch (const OrtError& e) {
               py::gil_scoped_acquire acq;
               TranslateAndThrow(e);
             } catch (const c10::Error& e) {
               py::gil_scoped_acquire acq;
               TranslateAndThrow(OrtError(StatusCode::RUNTIME_EXCEPTION, e.what_without_backtrace()));
             }
           })
      .def("inputs_meta", &InferenceSession::InputsMeta)
      .def("outputs_meta", &InferenceSession::OutputsMeta)
      .def("overridable_initializers_meta", &InferenceSession::OverridableInitializersMeta)
      .def("providers", &InferenceSession::Providers)
      .def("provider_options", &InferenceSession::ProviderOptionsMap)
      .def("end_profiling", &InferenceSession::EndProfiling)
      .def("profiling_start_time_ns", &InferenceSession::ProfilingStartTimeNs)
      .def("node_assignments", &InferenceSession::NodeAssignments)
      .def("num_captured_graphs", &InferenceSession::NumCapturedGraphs)
      .def("kernel_launch_count", &InferenceSession::KernelLaunchCount)
      .def("memory_plans", [](InferenceSession& s) {
        py::list out;
        for (auto& kv : s.MemoryPlans()) {
          const MemoryPlan& p = kv.second;
          py::dict d;
          d["pattern"] = p.pattern;
          d["host_peak_bytes"] = p.peak_bytes[0];
          d["host_total_bytes"] = p.total_bytes[0];
          d["host_live_peak_bytes"] = p.live_peak_bytes[0];
          d["host_values_reusing_memory"] = p.num_reused[0];
          d["device_peak_bytes"] = p.peak_bytes[1];
          d["device_total_bytes"] = p.total_bytes[1];
          d["device_live_peak_bytes"] = p.live_peak_bytes[1];
          d["device_values_reusing_memory"] = p.num_reused[1];
          std::string why;
          d["valid"] = PlanIsValid(p, &why);
          py::list bufs;
          for (auto& b : p.buffers) bufs.append(py::make_tuple(b.name, b.bytes, b.first_step, b.last_step, b.on_gpu, b.offset));
          d["buffers"] = bufs;
          out.append(d);
        }
        return out;
      })
      .def("tuning_results", [](InferenceSession& s) {
        py::dict d;
        for (auto& kv : s.tuning_results)
          d[py::str(kv.first)] = py::make_tuple(kv.second.force_splits, kv.second.force_bn, kv.second.force_tile_rows, kv.second.microseconds);
        return d;
      })
      .def("set_tuning_result", [](InferenceSession& s, const std::string& key, int splits, int bn, int rows) {
        InferenceSession::TunedGemm t;
        t.force_splits = splits;
        t.force_bn = bn;
        t.force_tile_rows = rows;
        s.tuning_results[key] = t;
      })
      .def("memory_stats", [](InferenceSession& s) {
        // arena statistics of the device allocator (the counterpart of the reference's BFCArena::GetStats)
        py::dict d;
        if (s.uses_gpu()) {
          const auto st = c10::cuda::CUDACachingAllocator::getDeviceStats(s.device().index());
          d["allocated_bytes"] = st.allocated_bytes[0].current;
          d["allocated_bytes_peak"] = st.allocated_bytes[0].peak;
          d["reserved_bytes"] = st.reserved_bytes[0].current;
          d["reserved_bytes_peak"] = st.reserved_bytes[0].peak;
          d["num_driver_allocations"] = st.segment[0].allocated;
          d["num_alloc_retries"] = st.num_alloc_retries;
          d["num_ooms"] = st.num_ooms;
        }
        return d;
      })
      .def("last_run_launch_count", &InferenceSession::LastRunLaunchCount)
      .def("check_device_status", [](InferenceSession& s) { Guard([&] { s.CheckDeviceStatus(); return 0; }); })
      .def("uses_gpu", &InferenceSession::uses_gpu)
      .def("set_symmetric_workspace", [](InferenceSession& s, const std::vector<int64_t>& ptrs, int64_t bytes, int64_t multicast_ptr) {
        s.symm_peers.clear();
        for (auto p : ptrs) s.symm_peers.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(p)));
        s.symm_bytes = bytes;
        s.symm_multicast = reinterpret_cast<void*>(static_cast<uintptr_t>(multicast_ptr));
      }, py::arg("ptrs"), py::arg("bytes"), py::arg("multicast_ptr") = 0)
      .def_readwrite("dist_group", &InferenceSession::dist_group)
      .def_readwrite("rank", &InferenceSession::rank)
      .def_readwrite("world_size", &InferenceSession::world_size)
      .def("serialize_model", [](InferenceSession& s) { return py::bytes(s.model().Serialize()); })
      .def("model_meta", [](InferenceSession& s) {
        const Model& mm = s.model();
        py::dict d;
        d["producer_name"] = mm.producer_name;
        d["graph_name"] = mm.graph_name;
        d["domain"] = mm.domain;
        d["description"] = mm.doc_string;
        d["graph_description"] = std::string();
        d["version"] = mm.model_version;
        d["custom_metadata_map"] = mm.metadata;
        return d;
      })
      .def("graph_nodes", [](InferenceSession& s) {
        py::list out;
        for (Node* n : s.model().MainGraph().TopologicalOrder()) out.append(NodeToDict(*n));
        return out;
      });

  py::class_<IOBinding>(m, "IOBinding")
      .def(py::init<InferenceSession*>(), py::keep_alive<1, 2>())
      .def("bind_input", [](IOBinding& b, const std::string& n, const at::Tensor& t) { Guard([&] { b.BindInput(n, t); return 0; }); })
      .def("bind_output", [](IOBinding& b, const std::string& n, const at::Tensor& t) { Guard([&] { b.BindOutput(n, t); return 0; }); })
      .def("bind_output_to_device", [](IOBinding& b, const std::string& n, const std::string& dev, int id) {
        Guard([&] {
          b.BindOutputToDevice(n, dev == "cuda" ? c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(id)) : c10::Device(c10::kCPU));
          return 0;
        });
      })
      .def("clear_inputs", &IOBinding::ClearInputs)
      .def("clear_outputs", &IOBinding::ClearOutputs)
      .def("synchronize_inputs", [](IOBinding& b) { Guard([&] { b.SynchronizeInputs(); return 0; }); })
      .def("synchronize_outputs", [](IOBinding& b) { Guard([&] { b.SynchronizeOutputs(); return 0; }); })
      .def("output_names", &IOBinding::OutputNames)
      .def("results", [](IOBinding& b) {
        py::list out;
        for (auto& v : b.Results()) out.append(FromValue(v));
        return out;
      });

  // ---- model / graph utilities (used by the Python tools and tests)
  m.def("register_python_op", [](const std::string& domain, const std::string& op, py::function fn) {
    Guard([&] { RegisterPythonOp(domain, op, std::move(fn)); return 0; });
  });
  m.def("load_custom_op_library", [](const std::string& path) { Guard([&] { LoadCustomOpLibrary(path); return 0; }); });
  m.def("nbits_build_blobs", [](const at::Tensor& B, const at::Tensor& scales, py::object zp, int64_t N, int64_t K, int64_t block) {
    return Guard([&] { return NbitsBuildBlobs(B, scales, zp.is_none() ? at::Tensor() : zp.cast<at::Tensor>(), N, K, block); });
  });
  m.def("model_roundtrip", [](py::bytes b) {
    std::string bytes = b;
    return Guard([&] {
      auto model = Model::LoadFromBytes(std::make_shared<std::string>(bytes), "");
      return py::bytes(model->Serialize());
    });
  });
  m.def("optimize_model", [](py::bytes b, int level, const std::vector<std::string>& disabled, bool gpu, int world_size) {
    std::string bytes = b;
    return Guard([&] {
      EnsureKernelsRegistered();
      auto model = Model::LoadFromBytes(std::make_shared<std::string>(bytes), "");
      std::set<std::string> dis(disabled.begin(), disabled.end());
      ConfigOptions cfg;
      OptimizerStats st = OptimizeGraph(model->MainGraph(), level, dis, gpu, cfg, world_size);
      return py::make_tuple(py::bytes(model->Serialize()), st.applied);
    });
  }, py::arg("model"), py::arg("level"), py::arg("disabled"), py::arg("gpu"), py::arg("world_size") = 1);
  m.def("infer_shapes", [](py::bytes b, bool strict) {
    std::string bytes = b;
    return Guard([&] {
      auto model = Model::LoadFromBytes(std::make_shared<std::string>(bytes), "");
      InferenceReport rep = InferShapes(model->MainGraph(), strict);
      py::dict d;
      d["nodes"] = rep.nodes;
      d["inferred"] = rep.inferred;
      d["problems"] = rep.problems;
      return py::make_tuple(py::bytes(model->Serialize()), d);
    });
  }, py::arg("model"), py::arg("strict") = false);
  m.def("op_schemas", [] {
    py::list out;
    for (const OpSchema* s : AllSchemas()) {
      py::dict d;
      d["domain"] = s->domain;
      d["op_type"] = s->op_type;
      d["min_inputs"] = s->min_inputs;
      d["max_inputs"] = s->max_inputs;
      d["has_shape_function"] = static_cast<bool>(s->infer);
      out.append(d);
    }
    return out;
  });
  m.def("model_nodes", [](py::bytes b) {
    std::string bytes = b;
    return Guard([&] {
      auto model = Model::LoadFromBytes(std::make_shared<std::string>(bytes), "");
      py::list out;
      for (Node* n : model->MainGraph().TopologicalOrder()) out.append(NodeToDict(*n));
      return out;
    });
  });
  m.def("tensor_from_proto", [](py::bytes b) {
    std::string bytes = b;
    return Guard([&] {
      pb::TensorProto t;
      pb::ParseTensor(bytes.data(), bytes.size(), &t);
      return TensorFromProto(t, "");
    });
  });
  m.def("tensor_to_proto", [](const at::Tensor& t, const std::string& name) {
    return Guard([&] { return py::bytes(pb::SerializeTensor(TensorToProto(t, name))); });
  });

  // ---- sharding-spec algebra of the Distributed* operators
  m.def("parse_shard_spec", [](const std::string& spec, const std::vector<int64_t>& mesh_elements,
                               const std::vector<int64_t>& mesh_shape) {
    return Guard([&] {
      TensorPartitionSpec s = TensorPartitionSpec::Parse(spec, DeviceMesh{mesh_elements, mesh_shape});
      py::dict d;
      d["spec"] = s.ToString();
      d["sharded_axis"] = s.ShardedAxis();
      d["num_shards"] = s.NumShards();
      return d;
    });
  });
  m.def("shard_shape", [](const std::vector<int64_t>& shape, const std::string& spec, const std::vector<int64_t>& mesh_elements,
                          const std::vector<int64_t>& mesh_shape) {
    return Guard([&] {
      return TensorPartitionSpec::Parse(spec, DeviceMesh{mesh_elements, mesh_shape}).ShardShape(shape);
    });
  });
}
