// Implementation of ortb200_c_api.h over the C++ session (no Python involved).
#include "string_table.h"
#include "ortb200_c_api.h"

#include <ATen/ATen.h>

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "graph.h"
#include "kernel.h"
#include "session.h"

#define ORTB200_EXPORT extern "C" __attribute__((visibility("default")))

struct ortb200_session {
  std::unique_ptr<ortb::InferenceSession> impl;
  std::vector<std::string> input_names, output_names;
  std::string profile_path;
};

struct ortb200_value {
  at::Tensor tensor;
  at::Tensor host;   // host copy made on request
  bool is_string = false;  // tensor holds ids of the string table
};

namespace {

thread_local std::string g_last_error;
void DropSessionExtras(const ortb200_session* s);

template <typename F>
int Guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const ortb::OrtError& e) {
    g_last_error = e.what();
    const int code = static_cast<int>(e.code());
    return code != 0 ? code : 1;
  } catch (const c10::Error& e) {
    g_last_error = e.what_without_backtrace();
    return 6;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return 6;
  }
}

at::Tensor WrapInput(const ortb200_tensor_view& v) {
  ORTB_ENFORCE_ARG(v.ndim >= 0 && v.ndim <= 8, "tensor rank must be in [0, 8]");
  std::vector<int64_t> dims(v.dims, v.dims + v.ndim);
  int64_t n = 1;
  for (int64_t d : dims) {
    ORTB_ENFORCE_ARG(d >= 0, "negative dimension");
    n *= d;
  }
  ORTB_ENFORCE_ARG(v.data != nullptr || n == 0, "tensor data is null");
  const at::ScalarType dt = ortb::ToTorchType(v.elem_type);
  const c10::Device dev = v.device_type == 1 ? c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(v.device_id)) : c10::Device(c10::kCPU);
  if (n == 0) return at::empty(dims, at::TensorOptions().dtype(dt).device(dev));
  return at::from_blob(v.data, dims, at::TensorOptions().dtype(dt).device(dev));
}

void FillView(const at::Tensor& t, ortb200_tensor_view* out) {
  std::memset(out, 0, sizeof(*out));
  out->data = t.data_ptr();
  out->elem_type = ortb::ToOnnxType(t.scalar_type());
  ORTB_ENFORCE_ARG(t.dim() <= 8, "tensor rank above 8");
  out->ndim = static_cast<int32_t>(t.dim());
  for (int64_t i = 0; i < t.dim(); ++i) out->dims[i] = t.size(i);
  out->device_type = t.is_cuda() ? 1 : 0;
  out->device_id = t.is_cuda() ? t.device().index() : 0;
}

}  // namespace

ORTB200_EXPORT const char* ortb200_last_error(void) { return g_last_error.c_str(); }
ORTB200_EXPORT const char* ortb200_version(void) { return "0.1.0"; }

ORTB200_EXPORT int ortb200_create_session(const char* model_path, const void* model_bytes, size_t model_size, const char* provider,
                                          int device_id, const char* const* config, ortb200_session** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    ORTB_ENFORCE_ARG(model_path != nullptr || (model_bytes != nullptr && model_size > 0), "no model given");
    ortb::EnsureKernelsRegistered();
    ortb::SessionOptions so;
    ortb::ProviderOptions popts;
    for (const char* const* kv = config; kv != nullptr && kv[0] != nullptr; kv += 2) {
      ORTB_ENFORCE_ARG(kv[1] != nullptr, "config key without a value: ", kv[0]);
      const std::string k = kv[0], v = kv[1];
      if (k == "graph_optimization_level") so.graph_optimization_level = std::stoi(v);
      else if (k == "enable_profiling") so.enable_profiling = v == "1" || v == "true";
      else if (k == "profile_file_prefix") so.profile_file_prefix = v;
      else if (k == "optimized_model_filepath") so.optimized_model_filepath = v;
      else if (k == "logid") so.logid = v;
      else if (k == "log_severity_level") so.log_severity_level = std::stoi(v);
      else if (k == "enable_cuda_graph") popts["enable_cuda_graph"] = v;
      else so.config.entries[k] = v;
    }
    auto s = std::make_unique<ortb200_session>();
    s->impl = std::make_unique<ortb::InferenceSession>(so);
    if (model_path != nullptr) s->impl->Load(model_path);
    else s->impl->LoadFromBytes(std::string(static_cast<const char*>(model_bytes), model_size));
    const std::string ep = provider != nullptr ? provider : ortb::kCpuEP;
    std::vector<std::pair<std::string, ortb::ProviderOptions>> providers;
    if (ep == ortb::kCudaEP) {
      popts["device_id"] = std::to_string(device_id);
      providers.emplace_back(ortb::kCudaEP, popts);
    }
    providers.emplace_back(ortb::kCpuEP, ortb::ProviderOptions{});
    s->impl->Initialize(providers, {});
    for (auto& m : s->impl->InputsMeta()) s->input_names.push_back(m.name);
    for (auto& m : s->impl->OutputsMeta()) s->output_names.push_back(m.name);
    *out = s.release();
  });
}

ORTB200_EXPORT void ortb200_release_session(ortb200_session* session) {
  if (session != nullptr) DropSessionExtras(session);
  delete session;
}

ORTB200_EXPORT int ortb200_session_input_count(const ortb200_session* session, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    *out = session->input_names.size();
  });
}

ORTB200_EXPORT int ortb200_session_output_count(const ortb200_session* session, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    *out = session->output_names.size();
  });
}

ORTB200_EXPORT int ortb200_session_input_name(const ortb200_session* session, size_t index, const char** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out && index < session->input_names.size(), "input index out of range");
    *out = session->input_names[index].c_str();
  });
}

ORTB200_EXPORT int ortb200_session_output_name(const ortb200_session* session, size_t index, const char** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out && index < session->output_names.size(), "output index out of range");
    *out = session->output_names[index].c_str();
  });
}

ORTB200_EXPORT int ortb200_run(ortb200_session* session, const char* const* input_names, const ortb200_tensor_view* inputs,
                               size_t num_inputs, const char* const* output_names, size_t num_outputs, ortb200_value** outputs) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && outputs && (num_inputs == 0 || (input_names && inputs)), "null argument");
    std::vector<std::string> in_names, out_names;
    std::vector<ortb::Value> feeds;
    for (size_t i = 0; i < num_inputs; ++i) {
      ORTB_ENFORCE_ARG(input_names[i] != nullptr, "input name ", i, " is null");
      in_names.emplace_back(input_names[i]);
      ortb::Value v;
      v.t = WrapInput(inputs[i]);
      feeds.push_back(std::move(v));
    }
    if (output_names != nullptr) {
      for (size_t i = 0; i < num_outputs; ++i) {
        ORTB_ENFORCE_ARG(output_names[i] != nullptr, "output name ", i, " is null");
        out_names.emplace_back(output_names[i]);
      }
    } else {
      ORTB_ENFORCE_ARG(num_outputs == session->output_names.size(), "num_outputs must equal the model's output count");
    }
    ortb::RunOptions ro;
    std::vector<ortb::Value> res = session->impl->Run(ro, in_names, feeds, out_names);
    ORTB_ENFORCE(res.size() == num_outputs, "unexpected number of outputs");
    for (size_t i = 0; i < num_outputs; ++i) outputs[i] = nullptr;
    for (size_t i = 0; i < num_outputs; ++i) {
      ORTB_ENFORCE_ARG(res[i].t.defined(), "output ", i, " is not a tensor (sequences are not exposed by the C API)");
      auto* v = new ortb200_value();
      // an output may alias caller memory (an input passed through): give the caller its own storage
      v->tensor = res[i].t.is_contiguous() ? res[i].t : res[i].t.contiguous();
      for (size_t k = 0; k < num_inputs; ++k)
        if (feeds[k].t.defined() && feeds[k].t.numel() > 0 && v->tensor.data_ptr() == feeds[k].t.data_ptr()) v->tensor = v->tensor.clone();
      outputs[i] = v;
    }
  });
}

ORTB200_EXPORT int ortb200_value_tensor(ortb200_value* value, int host, ortb200_tensor_view* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && out, "null argument");
    if (host && value->tensor.is_cuda()) {
      if (!value->host.defined()) value->host = value->tensor.cpu();
      FillView(value->host, out);
    } else {
      FillView(value->tensor, out);
    }
  });
}

ORTB200_EXPORT void ortb200_release_value(ortb200_value* value) { delete value; }

ORTB200_EXPORT int ortb200_end_profiling(ortb200_session* session, const char** out_path) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out_path, "null argument");
    session->profile_path = session->impl->EndProfiling();
    *out_path = session->profile_path.c_str();
  });
}

// ---------------------------------------------------------------------------------------------------------------
// Wider surface: option objects, type information, metadata, I/O binding, runtime-owned tensors, environment.
#include <cuda_runtime_api.h>

#include "logging.h"

namespace ortb {
void LoadCustomOpLibrary(const std::string& path);
}

struct ortb200_session_options {
  ortb::SessionOptions so;
  std::vector<std::pair<std::string, ortb::ProviderOptions>> providers;
};

struct ortb200_run_options {
  ortb::RunOptions ro;
};

struct ortb200_io_binding {
  explicit ortb200_io_binding(ortb::InferenceSession* s) : impl(s) {}
  ortb::IOBinding impl;
};

namespace {

struct SessionExtras {
  std::vector<ortb::NodeArgMeta> inputs, outputs, initializers;
  std::vector<std::string> providers, metadata_keys;
};
std::mutex g_extras_mu;
std::map<const ortb200_session*, std::shared_ptr<SessionExtras>> g_extras;

// type information is built on first use and kept for the strings' lifetime (dropped with the session)
std::shared_ptr<SessionExtras> Extras(const ortb200_session* s) {
  std::lock_guard<std::mutex> lock(g_extras_mu);
  auto it = g_extras.find(s);
  if (it != g_extras.end()) return it->second;
  auto e = std::make_shared<SessionExtras>();
  e->inputs = s->impl->InputsMeta();
  e->outputs = s->impl->OutputsMeta();
  e->initializers = s->impl->OverridableInitializersMeta();
  e->providers = s->impl->Providers();
  for (auto& kv : s->impl->model().metadata) e->metadata_keys.push_back(kv.first);
  g_extras[s] = e;
  return e;
}

void DropSessionExtras(const ortb200_session* s) {
  std::lock_guard<std::mutex> lock(g_extras_mu);
  g_extras.erase(s);
}

int32_t ElemTypeOfTypeString(const std::string& type) {  // "tensor(float16)" -> 10
  static const std::map<std::string, int32_t> table = {
      {"float", 1}, {"uint8", 2}, {"int8", 3}, {"uint16", 4}, {"int16", 5}, {"int32", 6}, {"int64", 7}, {"string", 8},
      {"bool", 9}, {"float16", 10}, {"double", 11}, {"uint32", 12}, {"uint64", 13}, {"bfloat16", 16},
      {"float8e4m3fn", 17}, {"float8e5m2", 19}};
  const size_t a = type.find('('), b = type.rfind(')');
  if (a == std::string::npos || b == std::string::npos || b <= a) return 0;
  auto it = table.find(type.substr(a + 1, b - a - 1));
  return it == table.end() ? 0 : it->second;
}

void FillTypeInfo(const ortb::NodeArgMeta& m, ortb200_type_info* out) {
  std::memset(out, 0, sizeof(*out));
  out->elem_type = ElemTypeOfTypeString(m.type);
  out->has_shape = m.has_shape ? 1 : 0;
  ORTB_ENFORCE_ARG(m.shape.size() <= 8, "rank above 8");
  out->ndim = static_cast<int32_t>(m.shape.size());
  for (size_t i = 0; i < m.shape.size(); ++i) {
    out->dims[i] = m.shape[i];
    out->dim_params[i] = i < m.sym.size() ? m.sym[i].c_str() : "";
  }
}

c10::Device DeviceOf(int device_type, int device_id) {
  return device_type == 1 ? c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device_id)) : c10::Device(c10::kCPU);
}

void RunCommon(ortb200_session* session, const ortb::RunOptions& ro, const char* const* input_names,
               const ortb200_tensor_view* inputs, size_t num_inputs, const char* const* output_names, size_t num_outputs,
               ortb200_value** outputs) {
  ORTB_ENFORCE_ARG(session && outputs && (num_inputs == 0 || (input_names && inputs)), "null argument");
  std::vector<std::string> in_names, out_names;
  std::vector<ortb::Value> feeds;
  for (size_t i = 0; i < num_inputs; ++i) {
    ORTB_ENFORCE_ARG(input_names[i] != nullptr, "input name ", i, " is null");
    in_names.emplace_back(input_names[i]);
    ortb::Value v;
    v.t = WrapInput(inputs[i]);
    feeds.push_back(std::move(v));
  }
  if (output_names != nullptr) {
    for (size_t i = 0; i < num_outputs; ++i) {
      ORTB_ENFORCE_ARG(output_names[i] != nullptr, "output name ", i, " is null");
      out_names.emplace_back(output_names[i]);
    }
  } else {
    ORTB_ENFORCE_ARG(num_outputs == session->output_names.size(), "num_outputs must equal the model's output count");
  }
  std::vector<ortb::Value> res = session->impl->Run(ro, in_names, feeds, out_names);
  ORTB_ENFORCE(res.size() == num_outputs, "unexpected number of outputs");
  for (size_t i = 0; i < num_outputs; ++i) outputs[i] = nullptr;
  for (size_t i = 0; i < num_outputs; ++i) {
    ORTB_ENFORCE_ARG(res[i].t.defined(), "output ", i, " is not a tensor (sequences are not exposed by the C API)");
    auto* v = new ortb200_value();
    v->tensor = res[i].t.is_contiguous() ? res[i].t : res[i].t.contiguous();
    v->is_string = res[i].is_string;
    for (size_t k = 0; k < num_inputs; ++k)
      if (feeds[k].t.defined() && feeds[k].t.numel() > 0 && v->tensor.data_ptr() == feeds[k].t.data_ptr()) v->tensor = v->tensor.clone();
    outputs[i] = v;
  }
}

}  // namespace

#define ORTB200_SETTER(name, arg_decl, body)                                                      \
  ORTB200_EXPORT int name(ortb200_session_options* options, arg_decl) {                           \
    return Guarded([&] {                                                                          \
      ORTB_ENFORCE_ARG(options != nullptr, "options is null");                                    \
      body;                                                                                       \
    });                                                                                           \
  }

ORTB200_EXPORT int ortb200_create_session_options(ortb200_session_options** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    *out = new ortb200_session_options();
  });
}
ORTB200_EXPORT void ortb200_release_session_options(ortb200_session_options* options) { delete options; }
ORTB200_SETTER(ortb200_session_options_set_graph_optimization_level, int level, {
  ORTB_ENFORCE_ARG(level == 0 || level == 1 || level == 2 || level == 3 || level == 99, "unknown optimization level ", level);
  options->so.graph_optimization_level = level;
})
ORTB200_SETTER(ortb200_session_options_set_intra_op_num_threads, int n, {
  ORTB_ENFORCE_ARG(n >= 0, "thread count must not be negative");
  options->so.intra_op_num_threads = n;
})
ORTB200_SETTER(ortb200_session_options_set_inter_op_num_threads, int n, {
  ORTB_ENFORCE_ARG(n >= 0, "thread count must not be negative");
  options->so.inter_op_num_threads = n;
})
ORTB200_SETTER(ortb200_session_options_set_execution_mode, int mode, {
  ORTB_ENFORCE_ARG(mode == 0 || mode == 1, "execution mode must be 0 (sequential) or 1 (parallel)");
  options->so.execution_mode = mode;
})
ORTB200_SETTER(ortb200_session_options_set_log_id, const char* logid, { options->so.logid = logid ? logid : ""; })
ORTB200_SETTER(ortb200_session_options_set_log_severity_level, int level, { options->so.log_severity_level = level; })
ORTB200_SETTER(ortb200_session_options_enable_profiling, const char* file_prefix, {
  options->so.enable_profiling = true;
  if (file_prefix != nullptr) options->so.profile_file_prefix = file_prefix;
})
ORTB200_SETTER(ortb200_session_options_set_optimized_model_filepath, const char* path, {
  options->so.optimized_model_filepath = path ? path : "";
})
ORTB200_SETTER(ortb200_session_options_register_custom_ops_library, const char* path, {
  ORTB_ENFORCE_ARG(path != nullptr, "path is null");
  ortb::LoadCustomOpLibrary(path);
})

ORTB200_EXPORT int ortb200_session_options_add_config_entry(ortb200_session_options* options, const char* key, const char* value) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options && key && value, "null argument");
    options->so.config.entries[key] = value;
  });
}

ORTB200_EXPORT int ortb200_session_options_add_free_dimension_override_by_name(ortb200_session_options* options, const char* name,
                                                                               int64_t value) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options && name, "null argument");
    options->so.free_dim_by_name[name] = value;
  });
}

ORTB200_EXPORT int ortb200_session_options_append_execution_provider(ortb200_session_options* options, const char* provider,
                                                                     const char* const* keys, const char* const* values,
                                                                     size_t num_options) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options && provider, "null argument");
    const std::string ep = provider;
    ORTB_ENFORCE_ARG(ep == ortb::kCudaEP || ep == ortb::kCpuEP, "unknown execution provider '", ep, "'");
    ortb::ProviderOptions po;
    for (size_t i = 0; i < num_options; ++i) {
      ORTB_ENFORCE_ARG(keys && values && keys[i] && values[i], "provider option ", i, " is null");
      po[keys[i]] = values[i];
    }
    options->providers.emplace_back(ep, po);
  });
}

ORTB200_EXPORT int ortb200_create_session_from_options(const char* model_path, const void* model_bytes, size_t model_size,
                                                       const ortb200_session_options* options, ortb200_session** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    ORTB_ENFORCE_ARG(model_path != nullptr || (model_bytes != nullptr && model_size > 0), "no model given");
    ortb::EnsureKernelsRegistered();
    ortb200_session_options defaults;
    const ortb200_session_options& o = options != nullptr ? *options : defaults;
    auto s = std::make_unique<ortb200_session>();
    s->impl = std::make_unique<ortb::InferenceSession>(o.so);
    if (model_path != nullptr) s->impl->Load(model_path);
    else s->impl->LoadFromBytes(std::string(static_cast<const char*>(model_bytes), model_size));
    std::vector<std::pair<std::string, ortb::ProviderOptions>> providers;
    bool has_cpu = false;
    for (auto& p : o.providers) {
      providers.push_back(p);
      has_cpu = has_cpu || p.first == ortb::kCpuEP;
    }
    if (!has_cpu) providers.emplace_back(ortb::kCpuEP, ortb::ProviderOptions{});
    s->impl->Initialize(providers, {});
    for (auto& m : s->impl->InputsMeta()) s->input_names.push_back(m.name);
    for (auto& m : s->impl->OutputsMeta()) s->output_names.push_back(m.name);
    *out = s.release();
  });
}

ORTB200_EXPORT int ortb200_create_run_options(ortb200_run_options** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    *out = new ortb200_run_options();
  });
}
ORTB200_EXPORT void ortb200_release_run_options(ortb200_run_options* options) { delete options; }
ORTB200_EXPORT int ortb200_run_options_set_tag(ortb200_run_options* options, const char* tag) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options != nullptr, "options is null");
    options->ro.logid = tag ? tag : "";
  });
}
ORTB200_EXPORT int ortb200_run_options_set_log_severity_level(ortb200_run_options* options, int level) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options != nullptr, "options is null");
    options->ro.log_severity_level = level;
  });
}
ORTB200_EXPORT int ortb200_run_options_add_config_entry(ortb200_run_options* options, const char* key, const char* value) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options && key && value, "null argument");
    options->ro.config.entries[key] = value;
  });
}
ORTB200_EXPORT int ortb200_run_options_set_terminate(ortb200_run_options* options, int terminate) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(options != nullptr, "options is null");
    options->ro.terminate->store(terminate != 0);
  });
}
ORTB200_EXPORT int ortb200_run_with_options(ortb200_session* session, const ortb200_run_options* options,
                                            const char* const* input_names, const ortb200_tensor_view* inputs, size_t num_inputs,
                                            const char* const* output_names, size_t num_outputs, ortb200_value** outputs) {
  return Guarded([&] {
    ortb::RunOptions defaults;
    RunCommon(session, options ? options->ro : defaults, input_names, inputs, num_inputs, output_names, num_outputs, outputs);
  });
}

ORTB200_EXPORT int ortb200_session_input_type_info(const ortb200_session* session, size_t index, ortb200_type_info* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    auto e = Extras(session);
    ORTB_ENFORCE_ARG(index < e->inputs.size(), "input index out of range");
    FillTypeInfo(e->inputs[index], out);
  });
}
ORTB200_EXPORT int ortb200_session_output_type_info(const ortb200_session* session, size_t index, ortb200_type_info* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    auto e = Extras(session);
    ORTB_ENFORCE_ARG(index < e->outputs.size(), "output index out of range");
    FillTypeInfo(e->outputs[index], out);
  });
}
ORTB200_EXPORT int ortb200_session_overridable_initializer_count(const ortb200_session* session, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    *out = Extras(session)->initializers.size();
  });
}
ORTB200_EXPORT int ortb200_session_overridable_initializer_name(const ortb200_session* session, size_t index, const char** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    auto e = Extras(session);
    ORTB_ENFORCE_ARG(index < e->initializers.size(), "initializer index out of range");
    *out = e->initializers[index].name.c_str();
  });
}

ORTB200_EXPORT int ortb200_session_model_metadata(const ortb200_session* session, ortb200_model_metadata* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    const ortb::Model& m = session->impl->model();
    out->producer_name = m.producer_name.c_str();
    out->graph_name = m.graph_name.c_str();
    out->domain = m.domain.c_str();
    out->description = m.doc_string.c_str();
    out->version = m.model_version;
    out->num_custom_keys = Extras(session)->metadata_keys.size();
  });
}
ORTB200_EXPORT int ortb200_session_custom_metadata_key(const ortb200_session* session, size_t index, const char** key) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && key, "null argument");
    auto e = Extras(session);
    ORTB_ENFORCE_ARG(index < e->metadata_keys.size(), "metadata index out of range");
    *key = e->metadata_keys[index].c_str();
  });
}
ORTB200_EXPORT int ortb200_session_lookup_custom_metadata(const ortb200_session* session, const char* key, const char** value) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && key && value, "null argument");
    const auto& md = session->impl->model().metadata;
    auto it = md.find(key);
    *value = it == md.end() ? nullptr : it->second.c_str();
  });
}
ORTB200_EXPORT int ortb200_session_provider_count(const ortb200_session* session, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    *out = Extras(session)->providers.size();
  });
}
ORTB200_EXPORT int ortb200_session_provider_name(const ortb200_session* session, size_t index, const char** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    auto e = Extras(session);
    ORTB_ENFORCE_ARG(index < e->providers.size(), "provider index out of range");
    *out = e->providers[index].c_str();
  });
}
ORTB200_EXPORT int ortb200_session_profiling_start_time_ns(const ortb200_session* session, int64_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    *out = session->impl->ProfilingStartTimeNs();
  });
}
ORTB200_EXPORT int ortb200_session_check_device_status(ortb200_session* session) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session != nullptr, "session is null");
    session->impl->CheckDeviceStatus();
  });
}

ORTB200_EXPORT int ortb200_create_io_binding(ortb200_session* session, ortb200_io_binding** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && out, "null argument");
    *out = new ortb200_io_binding(session->impl.get());
  });
}
ORTB200_EXPORT void ortb200_release_io_binding(ortb200_io_binding* binding) { delete binding; }
ORTB200_EXPORT int ortb200_io_binding_bind_input(ortb200_io_binding* binding, const char* name, const ortb200_tensor_view* tensor) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(binding && name && tensor, "null argument");
    binding->impl.BindInput(name, WrapInput(*tensor));
  });
}
ORTB200_EXPORT int ortb200_io_binding_bind_output(ortb200_io_binding* binding, const char* name, const ortb200_tensor_view* tensor) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(binding && name && tensor, "null argument");
    binding->impl.BindOutput(name, WrapInput(*tensor));
  });
}
ORTB200_EXPORT int ortb200_io_binding_bind_output_to_device(ortb200_io_binding* binding, const char* name, int device_type, int device_id) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(binding && name, "null argument");
    binding->impl.BindOutputToDevice(name, DeviceOf(device_type, device_id));
  });
}
#define ORTB200_BINDING_CALL(name, call)                        \
  ORTB200_EXPORT int name(ortb200_io_binding* binding) {        \
    return Guarded([&] {                                        \
      ORTB_ENFORCE_ARG(binding != nullptr, "binding is null");  \
      binding->impl.call();                                     \
    });                                                         \
  }
ORTB200_BINDING_CALL(ortb200_io_binding_clear_inputs, ClearInputs)
ORTB200_BINDING_CALL(ortb200_io_binding_clear_outputs, ClearOutputs)
ORTB200_BINDING_CALL(ortb200_io_binding_synchronize_inputs, SynchronizeInputs)
ORTB200_BINDING_CALL(ortb200_io_binding_synchronize_outputs, SynchronizeOutputs)

ORTB200_EXPORT int ortb200_run_with_binding(ortb200_session* session, const ortb200_run_options* options, ortb200_io_binding* binding) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && binding, "null argument");
    ortb::RunOptions defaults;
    session->impl->RunWithBinding(options ? options->ro : defaults, binding->impl);
  });
}
ORTB200_EXPORT int ortb200_io_binding_output_count(const ortb200_io_binding* binding, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(binding && out, "null argument");
    *out = binding->impl.OutputNames().size();
  });
}
ORTB200_EXPORT int ortb200_io_binding_output_name(const ortb200_io_binding* binding, size_t index, const char** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(binding && out && index < binding->impl.OutputNames().size(), "output index out of range");
    *out = binding->impl.OutputNames()[index].c_str();
  });
}
ORTB200_EXPORT int ortb200_io_binding_output_value(ortb200_io_binding* binding, size_t index, ortb200_value** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(binding && out, "null argument");
    const auto& res = binding->impl.Results();
    ORTB_ENFORCE_ARG(index < res.size(), "no result for output ", index, " (run the binding first)");
    ORTB_ENFORCE_ARG(res[index].t.defined(), "output ", index, " is not a tensor");
    auto* v = new ortb200_value();
    v->tensor = res[index].t;
    *out = v;
  });
}

ORTB200_EXPORT int ortb200_create_tensor(int32_t elem_type, const int64_t* dims, int32_t ndim, int device_type, int device_id,
                                         ortb200_value** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr && ndim >= 0 && ndim <= 8 && (ndim == 0 || dims != nullptr), "bad shape arguments");
    std::vector<int64_t> shape(dims, dims + ndim);
    for (int64_t d : shape) ORTB_ENFORCE_ARG(d >= 0, "negative dimension");
    auto opt = at::TensorOptions().dtype(ortb::ToTorchType(elem_type));
    auto* v = new ortb200_value();
    if (device_type == 2) v->tensor = at::empty(shape, opt.pinned_memory(true));
    else v->tensor = at::empty(shape, opt.device(DeviceOf(device_type, device_id)));
    *out = v;
  });
}
// ---- tensors of strings (reference: CreateTensorAsOrtValue with ONNX_TENSOR_ELEMENT_DATA_TYPE_STRING, FillStringTensor,
// GetStringTensorDataLength / GetStringTensorContent / GetStringTensorElement)
ORTB200_EXPORT int ortb200_create_string_tensor(const char* const* strings, const int64_t* dims, int32_t ndim, ortb200_value** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr && ndim >= 0 && ndim <= 8 && (ndim == 0 || dims != nullptr), "bad shape arguments");
    std::vector<int64_t> shape(dims, dims + ndim);
    int64_t n = 1;
    for (int64_t d : shape) {
      ORTB_ENFORCE_ARG(d >= 0, "negative dimension");
      n *= d;
    }
    ORTB_ENFORCE_ARG(n == 0 || strings != nullptr, "strings is null");
    std::vector<std::string> items;
    for (int64_t i = 0; i < n; ++i) {
      ORTB_ENFORCE_ARG(strings[i] != nullptr, "string ", i, " is null");
      items.emplace_back(strings[i]);
    }
    auto* v = new ortb200_value();
    v->tensor = ortb::InternStrings(items, shape);
    v->is_string = true;
    *out = v;
  });
}
ORTB200_EXPORT int ortb200_value_is_string(const ortb200_value* value, int* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && out, "null argument");
    *out = value->is_string ? 1 : 0;
  });
}
ORTB200_EXPORT int ortb200_value_string_count(const ortb200_value* value, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && out && value->is_string, "not a tensor of strings");
    *out = static_cast<size_t>(value->tensor.numel());
  });
}
ORTB200_EXPORT int ortb200_value_string_element(const ortb200_value* value, size_t index, const char** out, size_t* length) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && out && value->is_string, "not a tensor of strings");
    ORTB_ENFORCE_ARG(index < static_cast<size_t>(value->tensor.numel()), "string index out of range");
    at::Tensor ids = value->tensor.to(at::kCPU, at::kLong).contiguous().reshape({-1});
    const std::string& s = ortb::StringOfId(ids.data_ptr<int64_t>()[index]);  // the table never frees or moves a string
    *out = s.c_str();
    if (length) *length = s.size();
  });
}
ORTB200_EXPORT int ortb200_value_shape(const ortb200_value* value, int64_t* dims, int32_t* ndim) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && dims && ndim && value->tensor.defined(), "null argument");
    ORTB_ENFORCE_ARG(value->tensor.dim() <= 8, "more than 8 dimensions");
    *ndim = static_cast<int32_t>(value->tensor.dim());
    for (int64_t i = 0; i < value->tensor.dim(); ++i) dims[i] = value->tensor.size(i);
  });
}
// Run with runtime-owned values as inputs (tensors of strings can only be fed this way).
ORTB200_EXPORT int ortb200_run_with_values(ortb200_session* session, const ortb200_run_options* options, const char* const* input_names,
                                           ortb200_value* const* inputs, size_t num_inputs, const char* const* output_names, size_t num_outputs,
                                           ortb200_value** outputs) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(session && outputs && (num_inputs == 0 || (input_names && inputs)), "null argument");
    std::vector<std::string> in_names, out_names;
    std::vector<ortb::Value> feeds;
    for (size_t i = 0; i < num_inputs; ++i) {
      ORTB_ENFORCE_ARG(input_names[i] && inputs[i], "input ", i, " is null");
      in_names.emplace_back(input_names[i]);
      ortb::Value v;
      v.t = inputs[i]->tensor;
      v.is_string = inputs[i]->is_string;
      feeds.push_back(std::move(v));
    }
    if (output_names != nullptr) {
      for (size_t i = 0; i < num_outputs; ++i) out_names.emplace_back(output_names[i]);
    } else {
      ORTB_ENFORCE_ARG(num_outputs == session->output_names.size(), "num_outputs must equal the model's output count");
    }
    ortb::RunOptions defaults;
    std::vector<ortb::Value> res = session->impl->Run(options ? options->ro : defaults, in_names, feeds, out_names);
    ORTB_ENFORCE(res.size() == num_outputs, "unexpected number of outputs");
    for (size_t i = 0; i < num_outputs; ++i) outputs[i] = nullptr;
    for (size_t i = 0; i < num_outputs; ++i) {
      ORTB_ENFORCE_ARG(res[i].t.defined(), "output ", i, " is not a tensor (sequences and maps are not exposed by the C API)");
      auto* v = new ortb200_value();
      v->tensor = res[i].t.contiguous();
      v->is_string = res[i].is_string;
      for (size_t k = 0; k < num_inputs; ++k)
        if (v->tensor.numel() > 0 && v->tensor.data_ptr() == inputs[k]->tensor.data_ptr()) v->tensor = v->tensor.clone();
      outputs[i] = v;
    }
  });
}

ORTB200_EXPORT int ortb200_value_byte_size(const ortb200_value* value, size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && out, "null argument");
    *out = static_cast<size_t>(value->tensor.numel()) * value->tensor.element_size();
  });
}
ORTB200_EXPORT int ortb200_value_copy_from_host(ortb200_value* value, const void* src, size_t bytes) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && (src || bytes == 0), "null argument");
    at::Tensor& t = value->tensor;
    ORTB_ENFORCE_ARG(bytes == static_cast<size_t>(t.numel()) * t.element_size(), "byte count does not match the tensor");
    if (bytes == 0) return;
    at::Tensor host = at::from_blob(const_cast<void*>(src), t.sizes(), at::TensorOptions().dtype(t.scalar_type()));
    t.copy_(host);
    value->host = at::Tensor();
  });
}
ORTB200_EXPORT int ortb200_value_copy_to_host(ortb200_value* value, void* dst, size_t bytes) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(value && (dst || bytes == 0), "null argument");
    const at::Tensor& t = value->tensor;
    ORTB_ENFORCE_ARG(bytes == static_cast<size_t>(t.numel()) * t.element_size(), "byte count does not match the tensor");
    if (bytes == 0) return;
    at::Tensor host = at::from_blob(dst, t.sizes(), at::TensorOptions().dtype(t.scalar_type()));
    host.copy_(t);
  });
}

ORTB200_EXPORT int ortb200_cuda_device_count(int* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
    *out = n;
  });
}
ORTB200_EXPORT int ortb200_cuda_memory_info(int device_id, size_t* free_bytes, size_t* total_bytes) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(free_bytes && total_bytes, "null argument");
    int prev = 0;
    ORTB_ENFORCE(cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(device_id) == cudaSuccess, "no such CUDA device: ", device_id);
    const cudaError_t rc = cudaMemGetInfo(free_bytes, total_bytes);
    cudaSetDevice(prev);
    ORTB_ENFORCE(rc == cudaSuccess, "cudaMemGetInfo failed: ", cudaGetErrorString(rc));
  });
}
ORTB200_EXPORT int ortb200_available_provider_count(size_t* out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    int n = 0;
    ortb200_cuda_device_count(&n);
    *out = n > 0 ? 2 : 1;
  });
}
ORTB200_EXPORT int ortb200_available_provider_name(size_t index, const char** out) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(out != nullptr, "out is null");
    size_t n = 0;
    ortb200_available_provider_count(&n);
    ORTB_ENFORCE_ARG(index < n, "provider index out of range");
    *out = (n == 2 && index == 0) ? ortb::kCudaEP : ortb::kCpuEP;
  });
}
ORTB200_EXPORT int ortb200_set_default_logger_severity(int level) {
  return Guarded([&] {
    ORTB_ENFORCE_ARG(level >= 0 && level <= 4, "severity must be in [0, 4]");
    ortb::logging::Manager::Get().set_default_severity(level);
  });
}
