#include <mutex>

#include "kernel.h"

namespace ortb {

namespace {
class FnKernel final : public OpKernel {
 public:
  FnKernel(const OpKernelInfo& info, KernelFn fn) : OpKernel(info), fn_(std::move(fn)) {}
  void Compute(OpKernelContext& ctx) const override { fn_(ctx); }

 private:
  KernelFn fn_;
};
}  // namespace

KernelRegistry& KernelRegistry::Generic() {
  static KernelRegistry r;
  return r;
}

KernelRegistry& KernelRegistry::Cuda() {
  static KernelRegistry r;
  return r;
}

void KernelRegistry::Register(KernelDef def) {
  defs_[{def.domain, def.op_type}].push_back(std::move(def));
}

void KernelRegistry::RegisterFn(const std::string& domain, const std::string& op, int since_min, int since_max,
                                KernelFn fn, std::vector<int> host_inputs) {
  KernelDef d;
  d.domain = domain;
  d.op_type = op;
  d.since_min = since_min;
  d.since_max = since_max;
  d.host_inputs = std::move(host_inputs);
  d.factory = [fn](const OpKernelInfo& info) { return std::make_unique<FnKernel>(info, fn); };
  Register(std::move(d));
}

void KernelRegistry::RegisterAlias(const std::string& from_domain, const std::string& op, const std::string& to_domain) {
  auto it = defs_.find({from_domain, op});
  if (it == defs_.end() || it->second.empty()) return;
  const KernelDef* newest = &it->second.front();
  for (auto& d : it->second)
    if (d.since_max > newest->since_max || (d.since_max == newest->since_max && d.since_min > newest->since_min)) newest = &d;
  KernelDef copy = *newest;
  copy.domain = to_domain;
  copy.since_min = 1;
  copy.since_max = 1 << 30;
  Register(std::move(copy));
}

const KernelDef* KernelRegistry::Find(const Node& node, const Graph& graph) const {
  auto it = defs_.find({node.domain, node.op_type});
  if (it == defs_.end()) return nullptr;
  const int v = node.since_version > 0 ? node.since_version : static_cast<int>(graph.Opset(node.domain));
  for (auto& d : it->second) {
    if (v < d.since_min || v > d.since_max) continue;
    if (d.supports && !d.supports(node, graph)) continue;
    return &d;
  }
  return nullptr;
}

bool KernelRegistry::HasOp(const std::string& domain, const std::string& op) const {
  return defs_.count({domain, op}) != 0;
}

std::vector<std::string> KernelRegistry::ListOps() const {
  std::vector<std::string> out;
  for (auto& kv : defs_) out.push_back(kv.first.first.empty() ? kv.first.second : kv.first.first + "." + kv.first.second);
  return out;
}

void EnsureKernelsRegistered() {
  static std::once_flag once;
  std::call_once(once, [] {
    KernelRegistry& g = KernelRegistry::Generic();
    RegisterElementwiseKernels(g);
    RegisterTensorKernels(g);
    RegisterNnKernels(g);
    RegisterContribKernels(g);
    RegisterContribKernels2(g);
    RegisterContribKernels3(g);
    RegisterContribKernels4(g);
    RegisterContribKernels5(g);
    RegisterContribKernels6(g);
    RegisterTrainingKernels(g);
    RegisterOnnxExtraKernels(g);
    RegisterOnnxExtraKernels2(g);
    RegisterOnnxExtraKernels3(g);
    RegisterMlKernels(g);
    RegisterQOrderedKernels(g);
    RegisterStringKernels(g);
    RegisterControlFlowKernels(g);
    RegisterCollectiveKernels(g);
    // com.microsoft operators that are early forms of ONNX operators with the same semantics (contrib_ops/cpu_contrib_kernels.cc)
    for (const char* op : {"GatherND", "GridSample", "Pad", "QLinearConv", "Range"}) g.RegisterAlias("", op, "com.microsoft");
    RegisterCudaKernels(KernelRegistry::Cuda());
  });
}

std::vector<int> HostInputsOf(const Node& node, const Graph& graph) {
  EnsureKernelsRegistered();
  if (node.ep == kCudaEP || node.ep.empty()) {
    const KernelDef* c = KernelRegistry::Cuda().Find(node, graph);
    if (c) return c->host_inputs;
  }
  const KernelDef* d = KernelRegistry::Generic().Find(node, graph);
  return d ? d->host_inputs : std::vector<int>{};
}

}  // namespace ortb
