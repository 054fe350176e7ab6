// Operator kernel interface and registry.
//
// Counterpart of the reference's OpKernel / OpKernelInfo / OpKernelContext
// (include/onnxruntime/core/framework/op_kernel.h:40-144) and KernelRegistry
// (onnxruntime/core/framework/kernel_registry.cc:146-226).  Kernels are created
// once per node at session initialisation (attributes parsed there, constant
// weights pre-packed there) and called with a light context at run time.
//
// Two registries exist: "generic" kernels are written against ATen and run on
// whichever device their inputs live on (they are the CPU execution provider
// and the long tail of the GPU one); "cuda" kernels are the hand-written
// sm_100a kernels and win the lookup for GPU nodes.
#pragma once
#include <ATen/ATen.h>

#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "graph.h"

namespace ortb {

class InferenceSession;
struct RunOptions;
using RunOptionsRef = RunOptions;

// A run-time value: a tensor, or a sequence of tensors (ONNX sequence type), or absent.
// A sequence of maps that share one key set (what ai.onnx.ml ZipMap produces): row i maps keys[c] -> values[i, c].
struct MapRows {
  at::Tensor keys;           // [C] int64 (ids of the string table when string_keys)
  bool string_keys = false;
  at::Tensor values;         // [N, C] float (ids of the string table when string_values)
  bool string_values = false;
};

struct Value {
  at::Tensor t;
  std::shared_ptr<std::vector<at::Tensor>> seq;
  std::shared_ptr<MapRows> maps;
  bool is_string = false;  // t holds ids of the string table (string_table.h): a tensor of strings
  bool defined() const { return t.defined() || seq != nullptr || maps != nullptr; }
};

struct ConfigOptions {
  std::map<std::string, std::string> entries;
  std::string Get(const std::string& k, const std::string& dflt = "") const {
    auto it = entries.find(k);
    return it == entries.end() ? dflt : it->second;
  }
};

struct OpKernelInfo {
  const Node& node;
  const Graph& graph;
  InferenceSession* session;
  c10::Device device;
  const ConfigOptions* config;
  // Constant initializer feeding input `idx`, already on `device` (nullptr when not constant).
  std::function<const at::Tensor*(int)> constant_input;
};

class OpKernelContext {
 public:
  OpKernelContext(const Node& node, InferenceSession* session, c10::Device device, std::vector<Value>& in,
                  std::vector<Value>& out, const std::vector<bool>& out_needed)
      : node_(node), session_(session), device_(device), in_(in), out_(out), out_needed_(out_needed) {}

  const Node& node() const { return node_; }
  InferenceSession* session() const { return session_; }
  c10::Device device() const { return device_; }
  int InputCount() const { return static_cast<int>(in_.size()); }
  int OutputCount() const { return static_cast<int>(out_.size()); }
  bool HasInput(int i) const { return i < static_cast<int>(in_.size()) && in_[i].t.defined(); }
  const at::Tensor& Input(int i) const {
    static const at::Tensor undefined;
    return i < static_cast<int>(in_.size()) ? in_[i].t : undefined;
  }
  const at::Tensor& RequiredInput(int i) const {
    if (!HasInput(i)) ORTB_THROW(INVALID_ARGUMENT, "node '", node_.name, "' (", node_.op_type, ") is missing input ", i);
    return in_[i].t;
  }
  const Value& InputValue(int i) const { return in_[i]; }
  const MapRows* InputMaps(int i) const { return i < static_cast<int>(in_.size()) ? in_[i].maps.get() : nullptr; }
  bool InputIsString(int i) const { return i < static_cast<int>(in_.size()) && in_[i].is_string; }
  // output i is a tensor of strings: `ids` index the string table
  void SetOutputStrings(int i, at::Tensor ids) {
    if (i < static_cast<int>(out_.size())) {
      out_[i].t = std::move(ids);
      out_[i].is_string = true;
    }
  }
  bool OutputNeeded(int i) const { return i < static_cast<int>(out_needed_.size()) && out_needed_[i]; }
  void SetOutput(int i, at::Tensor t) {
    if (i < static_cast<int>(out_.size())) out_[i].t = std::move(t);
  }
  void SetOutputMaps(int i, MapRows m) {
    if (i < static_cast<int>(out_.size())) out_[i].maps = std::make_shared<MapRows>(std::move(m));
  }
  void SetOutputSeq(int i, std::vector<at::Tensor> s) {
    if (i < static_cast<int>(out_.size())) out_[i].seq = std::make_shared<std::vector<at::Tensor>>(std::move(s));
  }
  // Output buffer bound by the caller (IOBinding) or planned by the session, if any.
  at::Tensor& Preallocated(int i) { return out_[i].t; }
  void* cuda_stream() const;  // cudaStream_t of the current torch stream on device()
  // Resolve a value of the enclosing scope by name (control-flow bodies read captured values).
  using Lookup = std::function<Value(const std::string&)>;
  void set_lookup(const Lookup* l) { lookup_ = l; }
  Value LookupValue(const std::string& name) const {
    if (!lookup_) ORTB_THROW(FAIL, "no scope available to resolve '", name, "'");
    return (*lookup_)(name);
  }
  const RunOptionsRef* run_options = nullptr;

 private:
  const Lookup* lookup_ = nullptr;
  const Node& node_;
  InferenceSession* session_;
  c10::Device device_;
  std::vector<Value>& in_;
  std::vector<Value>& out_;
  const std::vector<bool>& out_needed_;
};

class OpKernel {
 public:
  explicit OpKernel(const OpKernelInfo& info) : node_(info.node) {}
  virtual ~OpKernel() = default;
  virtual void Compute(OpKernelContext& ctx) const = 0;
  // Inputs (by index) this kernel reads on the host even when the node runs on the GPU.
  virtual bool InputOnHost(int /*idx*/) const { return false; }
  // Constant inputs the kernel re-packed into its own storage at construction; Compute() never reads them,
  // so the session may drop the original copy.
  virtual std::vector<int> PrepackedInputs() const { return {}; }
  const Node& node() const { return node_; }

 protected:
  const Node& node_;
};

using KernelFactory = std::function<std::unique_ptr<OpKernel>(const OpKernelInfo&)>;
using KernelFn = std::function<void(OpKernelContext&)>;

struct KernelDef {
  std::string domain, op_type;
  int since_min = 1, since_max = 1 << 30;
  KernelFactory factory;
  // indices of inputs that must stay in host memory (shape-like operands)
  std::vector<int> host_inputs;
  // optional predicate: can this kernel handle the node (dtype / attribute checks)?
  std::function<bool(const Node&, const Graph&)> supports;
};

class KernelRegistry {
 public:
  static KernelRegistry& Generic();  // ATen-backed, device-agnostic
  static KernelRegistry& Cuda();     // hand-written sm_100a kernels
  void Register(KernelDef def);
  void RegisterFn(const std::string& domain, const std::string& op, int since_min, int since_max, KernelFn fn,
                  std::vector<int> host_inputs = {});
  // the newest kernel of (from_domain, op) also serves (to_domain, op), any version
  void RegisterAlias(const std::string& from_domain, const std::string& op, const std::string& to_domain);
  const KernelDef* Find(const Node& node, const Graph& graph) const;
  bool HasOp(const std::string& domain, const std::string& op) const;
  std::vector<std::string> ListOps() const;

 private:
  std::map<std::pair<std::string, std::string>, std::vector<KernelDef>> defs_;
};

// Registration entry points (each defined in its own translation unit).
void RegisterElementwiseKernels(KernelRegistry& r);
void RegisterTensorKernels(KernelRegistry& r);
void RegisterNnKernels(KernelRegistry& r);
void RegisterContribKernels(KernelRegistry& r);
void RegisterContribKernels2(KernelRegistry& r);
void RegisterContribKernels3(KernelRegistry& r);
void RegisterContribKernels4(KernelRegistry& r);
void RegisterContribKernels5(KernelRegistry& r);
void RegisterContribKernels6(KernelRegistry& r);
void RegisterTrainingKernels(KernelRegistry& r);
// convolution / pooling with the attributes of `node` (kernels_nn.cc)
at::Tensor ConvWithNodeAttrs(const Node& node, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias);
at::Tensor ConvTransposeWithNodeAttrs(const Node& node, const at::Tensor& x, const at::Tensor& w,
                                      const c10::optional<at::Tensor>& bias, const std::vector<int64_t>* pads_override = nullptr);
at::Tensor PoolWithNodeAttrs(const Node& node, at::Tensor x, bool is_max);
void RegisterOnnxExtraKernels(KernelRegistry& r);
void RegisterOnnxExtraKernels2(KernelRegistry& r);
void RegisterOnnxExtraKernels3(KernelRegistry& r);
void RegisterMlKernels(KernelRegistry& r);
void RegisterQOrderedKernels(KernelRegistry& r);
void RegisterStringKernels(KernelRegistry& r);
// Cast with a string on either side (kernels_string.cc); false when neither side is a string
bool CastWithStrings(OpKernelContext& ctx, int32_t to);
void RegisterControlFlowKernels(KernelRegistry& r);
void RegisterCollectiveKernels(KernelRegistry& r);
void RegisterCudaKernels(KernelRegistry& r);
void EnsureKernelsRegistered();

// Indices of inputs that are shape-like (read on the host) for a node, from its generic kernel definition.
std::vector<int> HostInputsOf(const Node& node, const Graph& graph);

}  // namespace ortb
