// Custom operators: Python callables and shared libraries speaking the C ABI of custom_op_api.h.
// Both register into the generic kernel registry under (domain, op_type); the partitioner then treats them like
// any other operator (they run where their first input lives).
#include <dlfcn.h>
#include <ATen/ATen.h>

#include <mutex>

#include "custom_op_api.h"
#include "graph.h"
#include "kernel.h"
#include "session.h"


struct ortb200_kernel_context {
  ortb::OpKernelContext* ctx;
  std::string error;
};

namespace ortb {
namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

int OnnxTypeOf(at::ScalarType t) { return static_cast<int>(ToOnnxType(t)); }

void FillTensor(const at::Tensor& t, ortb200_tensor* o) {
  *o = ortb200_tensor{};
  if (!t.defined()) return;
  o->present = 1;
  o->data = t.data_ptr();
  o->ndim = static_cast<int32_t>(t.dim());
  for (int i = 0; i < t.dim() && i < 8; ++i) o->dims[i] = t.size(i);
  o->elem_type = OnnxTypeOf(t.scalar_type());
  o->on_gpu = t.is_cuda() ? 1 : 0;
}

// ---- C ABI callbacks
int ApiAttrInt(const ortb200_kernel_context* c, const char* name, int64_t* out) {
  const Node& n = c->ctx->node();
  if (!n.has_attr(name)) return 1;
  *out = n.attr_i(name, 0);
  return 0;
}
int ApiAttrFloat(const ortb200_kernel_context* c, const char* name, float* out) {
  const Node& n = c->ctx->node();
  if (!n.has_attr(name)) return 1;
  *out = n.attr_f(name, 0.f);
  return 0;
}
int ApiAttrString(const ortb200_kernel_context* c, const char* name, char* out, int64_t capacity) {
  const Node& n = c->ctx->node();
  if (!n.has_attr(name)) return 1;
  const std::string s = n.attr_s(name);
  if (static_cast<int64_t>(s.size()) + 1 > capacity) return 2;
  std::memcpy(out, s.c_str(), s.size() + 1);
  return 0;
}
int ApiAllocateOutput(ortb200_kernel_context* c, int index, const int64_t* dims, int ndim, int32_t elem_type, ortb200_tensor* out) {
  if (index < 0 || index >= c->ctx->OutputCount() || ndim < 0 || ndim > 8) return 1;
  at::TensorOptions opt = at::TensorOptions().dtype(ToTorchType(elem_type));
  if (c->ctx->InputCount() > 0 && c->ctx->HasInput(0)) opt = opt.device(c->ctx->Input(0).device());
  at::Tensor t = at::empty(std::vector<int64_t>(dims, dims + ndim), opt);
  c->ctx->SetOutput(index, t);
  FillTensor(t, out);
  return 0;
}
void* ApiCudaStream(const ortb200_kernel_context* c) {
  InferenceSession* s = c->ctx->session();
  return (s && s->uses_gpu()) ? c->ctx->cuda_stream() : nullptr;
}
void ApiSetError(ortb200_kernel_context* c, const char* message) { c->error = message ? message : ""; }

using ComputeFn = int (*)(const ortb200_custom_op_api*, ortb200_kernel_context*, const ortb200_tensor*, int, int, void*);
int ApiRegisterOp(const char* domain, const char* op_type, ComputeFn compute, void* user);

const ortb200_custom_op_api kApi = {ORTB200_CUSTOM_OP_API_VERSION, ApiAttrInt, ApiAttrFloat, ApiAttrString, ApiAllocateOutput,
                                   ApiCudaStream, ApiSetError, ApiRegisterOp};

int ApiRegisterOp(const char* domain, const char* op_type, ComputeFn compute, void* user) {
  if (!domain || !op_type || !compute) return 1;
  EnsureKernelsRegistered();
  const std::string op = op_type;
  KernelRegistry::Generic().RegisterFn(domain, op, 1, kMax, [compute, user, op](Ctx& ctx) {
    std::vector<at::Tensor> keep;
    std::vector<ortb200_tensor> ins(static_cast<size_t>(ctx.InputCount()));
    for (int i = 0; i < ctx.InputCount(); ++i) {
      at::Tensor t = ctx.HasInput(i) ? ctx.Input(i).contiguous() : at::Tensor();
      keep.push_back(t);
      FillTensor(t, &ins[static_cast<size_t>(i)]);
    }
    ortb200_kernel_context kc{&ctx, ""};
    const int rc = compute(&kApi, &kc, ins.data(), ctx.InputCount(), ctx.OutputCount(), user);
    if (rc != 0) ORTB_THROW(FAIL, "custom op ", op, " failed (code ", rc, ")", kc.error.empty() ? "" : ": ", kc.error);
  });
  return 0;
}

std::mutex g_lib_mu;
std::vector<void*> g_libs;  // handles stay open for the life of the process: kernels point into them

}  // namespace

void LoadCustomOpLibrary(const std::string& path) {
  std::lock_guard<std::mutex> lock(g_lib_mu);
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) ORTB_THROW(FAIL, "cannot load custom op library ", path, ": ", dlerror());
  using RegFn = int (*)(const ortb200_custom_op_api*);
  RegFn fn = reinterpret_cast<RegFn>(dlsym(h, "ortb200_register_custom_ops"));
  if (!fn) {
    dlclose(h);
    ORTB_THROW(FAIL, "custom op library ", path, " does not export ortb200_register_custom_ops");
  }
  const int rc = fn(&kApi);
  if (rc != 0) ORTB_THROW(FAIL, "ortb200_register_custom_ops of ", path, " returned ", rc);
  g_libs.push_back(h);
}

}  // namespace ortb
