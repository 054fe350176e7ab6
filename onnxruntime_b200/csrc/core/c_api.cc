// Implementation of ortb200_c_api.h over the C++ session (no Python involved).
#include "ortb200_c_api.h"

#include <ATen/ATen.h>

#include <cstring>
#include <memory>
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
};

namespace {

thread_local std::string g_last_error;

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

ORTB200_EXPORT void ortb200_release_session(ortb200_session* session) { delete session; }

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
