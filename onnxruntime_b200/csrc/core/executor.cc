#include "executor.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <set>
#include <sstream>
#include <cuda_runtime_api.h>
#include <nvtx3/nvToolsExt.h>

#include "threadpool.h"

namespace ortb {

namespace {
// NVTX range around one node (reference: onnxruntime/core/providers/cuda/nvtx_profile.h:100-139, used at
// sequential_executor.cc:413,517).  Without a profiler attached the calls are a few nanoseconds.
struct NvtxRange {
  explicit NvtxRange(const char* name) : on_(name != nullptr) {
    if (on_) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (on_) nvtxRangePop();
  }
  bool on_;
};
}  // namespace

namespace {
bool IsShapeOnlyOp(const Node& n) { return n.domain.empty() && (n.op_type == "Shape" || n.op_type == "Size"); }
bool IsControlFlow(const Node& n) {
  return n.domain.empty() && (n.op_type == "If" || n.op_type == "Loop" || n.op_type == "Scan" || n.op_type == "SequenceMap");
}
bool Contains(const std::vector<int>& v, int x) { return std::find(v.begin(), v.end(), x) != v.end(); }
const char* kGpuSuffix = "\x01gpu";
}  // namespace

void* OpKernelContext::cuda_stream() const {
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(device_.index()).stream());
}

GraphExecutor::GraphExecutor(InferenceSession* session, Graph* graph, const std::map<std::string, bool>* outer_on_gpu)
    : session_(session), graph_(graph) {
  if (outer_on_gpu) outer_on_gpu_ = *outer_on_gpu;
}

bool GraphExecutor::ValueOnGpu(const std::string& name) const {
  auto it = on_gpu_.find(name);
  if (it != on_gpu_.end()) return it->second;
  auto ot = outer_on_gpu_.find(name);
  return ot != outer_on_gpu_.end() ? ot->second : false;
}

int GraphExecutor::SlotOf(const std::string& name) const {
  auto it = slot_of_.find(name);
  return it == slot_of_.end() ? -1 : it->second;
}

int GraphExecutor::NewSlot(const std::string& name) {
  auto it = slot_of_.find(name);
  if (it != slot_of_.end()) return it->second;
  const int s = static_cast<int>(slot_names_.size());
  slot_of_[name] = s;
  slot_names_.push_back(name);
  constant_slots_.emplace_back();
  return s;
}

void GraphExecutor::Partition() {
  const bool gpu = session_->uses_gpu();
  on_gpu_.clear();
  for (auto& kv : outer_on_gpu_) on_gpu_[kv.first] = kv.second;

  // Runtime inputs live on the GPU when some consumer reads them there.
  for (const ValueInfo& vi : graph_->Inputs()) {
    const ValueInfo* v = &vi;
    if (graph_->IsConstant(v->name)) continue;
    bool dev_use = false;
    for (Node* n : graph_->Consumers(v->name)) {
      if (IsShapeOnlyOp(*n)) continue;
      if (IsControlFlow(*n)) {
        const std::vector<int> host = HostInputsOf(*n, *graph_);
        bool direct = false;
        for (size_t i = 0; i < n->inputs.size(); ++i)
          if (n->inputs[i] == v->name) {
            direct = true;
            if (!Contains(host, static_cast<int>(i))) dev_use = true;
          }
        if (!direct) dev_use = true;
        continue;
      }
      const std::vector<int> host = HostInputsOf(*n, *graph_);
      for (size_t i = 0; i < n->inputs.size(); ++i)
        if (n->inputs[i] == v->name && !Contains(host, static_cast<int>(i))) dev_use = true;
    }
    if (graph_->Parent() != nullptr) {
      // body inputs arrive wherever the control-flow op has them; decided by the caller
      auto it = outer_on_gpu_.find("\x02input:" + v->name);
      on_gpu_[v->name] = it != outer_on_gpu_.end() ? it->second : (gpu && dev_use);
    } else {
      on_gpu_[v->name] = gpu && dev_use;
    }
  }

  for (Node* n : graph_->TopologicalOrder()) {
    bool node_gpu = gpu;
    if (gpu) {
      if (IsShapeOnlyOp(*n) || IsControlFlow(*n)) {
        node_gpu = false;
      } else {
        bool has_dyn = false, all_cpu = true;
        for (auto& i : n->inputs) {
          if (i.empty() || graph_->IsConstant(i)) continue;
          if (!graph_->IsInitializer(i) || graph_->IsGraphInput(i)) {
            has_dyn = true;
            if (ValueOnGpu(i)) all_cpu = false;
          }
        }
        if (has_dyn && all_cpu) node_gpu = false;  // host-side shape arithmetic stays on the host
        if (!has_dyn) {
          // constant-only producers (Constant, ConstantOfShape, Range ...): keep small integer results on the host
          bool all_host_use = true;
          const std::vector<int> none;
          for (auto& o : n->outputs) {
            if (o.empty()) continue;
            if (graph_->IsGraphOutput(o)) all_host_use = false;
            for (Node* c : graph_->Consumers(o)) {
              if (IsShapeOnlyOp(*c)) continue;
              const std::vector<int> host = HostInputsOf(*c, *graph_);
              for (size_t k = 0; k < c->inputs.size(); ++k)
                if (c->inputs[k] == o && !Contains(host, static_cast<int>(k))) all_host_use = false;
            }
          }
          if (all_host_use) node_gpu = false;
        }
      }
    }
    n->ep = node_gpu ? kCudaEP : kCpuEP;
    bool out_gpu = node_gpu;
    if (gpu && IsControlFlow(*n)) out_gpu = true;  // control-flow kernels hand their results over on the GPU
    for (auto& o : n->outputs)
      if (!o.empty()) on_gpu_[o] = out_gpu;
  }
}

void GraphExecutor::InsertCopies() {
  if (!session_->uses_gpu()) return;
  std::map<std::pair<std::string, bool>, std::string> copies;  // (value, want_gpu) -> copy name
  for (Node* n : graph_->TopologicalOrder()) {
    if (IsShapeOnlyOp(*n)) continue;
    if (n->op_type == "MemcpyToHost" || n->op_type == "MemcpyFromHost") continue;
    const bool node_gpu = n->ep == kCudaEP;
    const std::vector<int> host = HostInputsOf(*n, *graph_);
    const bool cf = IsControlFlow(*n);
    for (size_t i = 0; i < n->inputs.size(); ++i) {
      const std::string v = n->inputs[i];
      if (v.empty() || graph_->IsConstant(v)) continue;
      bool want_gpu;
      if (cf) {
        if (!Contains(host, static_cast<int>(i))) continue;  // bodies take values wherever they are
        want_gpu = false;
      } else {
        want_gpu = node_gpu && !Contains(host, static_cast<int>(i));
      }
      const bool have_gpu = ValueOnGpu(v);
      if (have_gpu == want_gpu) continue;
      auto key = std::make_pair(v, want_gpu);
      auto it = copies.find(key);
      if (it == copies.end()) {
        const std::string cname = graph_->UniqueName(v + (want_gpu ? "_to_device" : "_to_host"));
        Node* c = graph_->AddNode(want_gpu ? "MemcpyFromHost" : "MemcpyToHost", {v}, {cname}, "");
        c->ep = want_gpu ? kCudaEP : kCpuEP;
        on_gpu_[cname] = want_gpu;
        it = copies.emplace(key, cname).first;
      }
      n->inputs[i] = it->second;
    }
  }
  graph_->Invalidate();
}

void GraphExecutor::Build() {
  Partition();
  InsertCopies();
  const bool gpu = session_->uses_gpu();
  const c10::Device dev = session_->device();
  const c10::Device cpu(c10::kCPU);

  steps_.clear();
  slot_of_.clear();
  slot_names_.clear();
  constant_slots_.clear();
  input_names_.clear();
  input_slot_.clear();
  input_device_.clear();

  std::vector<Node*> order = graph_->TopologicalOrder();

  // runtime inputs (overridable initializers are optional inputs with a default)
  for (auto& v : graph_->Inputs()) {
    const bool is_init = graph_->IsInitializer(v.name);
    if (is_init && graph_->IsConstant(v.name)) continue;
    const int s = NewSlot(v.name);
    input_names_.push_back(v.name);
    input_slot_.push_back(s);
    const bool g = ValueOnGpu(v.name);
    input_device_.push_back(g ? dev : cpu);
    if (is_init) {
      const at::Tensor* t = graph_->GetInitializer(v.name);
      constant_slots_[s].t = g ? t->to(dev) : *t;
      constant_slots_[s].is_string = graph_->IsStringValue(v.name);
    }
  }

  // values captured from enclosing graphs
  outer_names_.clear();
  outer_slot_.clear();
  auto outer_slot = [&](const std::string& name) {
    auto it = slot_of_.find(name);
    if (it != slot_of_.end()) return it->second;
    const int s = NewSlot(name);
    outer_names_.push_back(name);
    outer_slot_.push_back(s);
    return s;
  };

  auto const_slot = [&](const std::string& name, bool want_gpu) {
    const std::string key = want_gpu ? name + kGpuSuffix : name;
    auto it = slot_of_.find(key);
    if (it != slot_of_.end()) return it->second;
    const int s = NewSlot(key);
    const at::Tensor* t = graph_->GetInitializer(name);
    ORTB_ENFORCE(t != nullptr, "missing initializer ", name);
    if (graph_->PendingExternal().count(name) && t->numel() == 0)
      ORTB_THROW(INVALID_ARGUMENT, "initializer '", name,
                 "' is marked as supplied by the session but no value was given (add_external_initializers)");
    if (want_gpu) constant_slots_[s].t = t->is_cuda() ? *t : t->to(dev);
    else constant_slots_[s].t = t->is_cuda() ? t->cpu() : *t;
    constant_slots_[s].is_string = graph_->IsStringValue(name);
    return s;
  };

  std::map<std::string, int> produced;
  for (Node* n : order) {
    Step st;
    st.node = n;
    st.on_gpu = gpu && n->ep == kCudaEP;
    st.device = st.on_gpu ? dev : cpu;
    const std::vector<int> host = HostInputsOf(*n, *graph_);
    std::vector<at::Tensor> const_inputs(n->inputs.size());  // handles, not pointers: the slot vector may grow
    for (size_t i = 0; i < n->inputs.size(); ++i) {
      const std::string& v = n->inputs[i];
      if (v.empty()) {
        st.in_slots.push_back(-1);
        continue;
      }
      if (graph_->IsConstant(v)) {
        const bool want_gpu = st.on_gpu && !Contains(host, static_cast<int>(i));
        const int s = const_slot(v, want_gpu);
        st.in_slots.push_back(s);
        const_inputs[i] = constant_slots_[s].t;
        continue;
      }
      auto it = slot_of_.find(v);
      if (it != slot_of_.end()) {
        st.in_slots.push_back(it->second);
      } else if (graph_->Parent() != nullptr) {
        // constant in an enclosing graph, or a value computed there
        const Graph* g = graph_->Parent();
        const at::Tensor* outer_const = nullptr;
        for (; g; g = g->Parent())
          if (g->IsConstant(v)) {
            outer_const = g->GetInitializer(v);
            break;
          }
        if (outer_const) {
          const bool want_gpu = st.on_gpu && !Contains(host, static_cast<int>(i));
          const std::string key = want_gpu ? v + kGpuSuffix : v;
          int s;
          auto kt = slot_of_.find(key);
          if (kt != slot_of_.end()) s = kt->second;
          else {
            s = NewSlot(key);
            constant_slots_[s].t = want_gpu ? outer_const->to(dev) : outer_const->cpu();
          }
          st.in_slots.push_back(s);
          const_inputs[i] = constant_slots_[s].t;
        } else {
          st.in_slots.push_back(outer_slot(v));
        }
      } else {
        ORTB_THROW(INVALID_GRAPH, "node '", n->name, "' (", n->op_type, ") reads undefined value '", v, "'");
      }
    }
    for (auto& o : n->outputs) {
      if (o.empty()) {
        st.out_slots.push_back(-1);
        st.out_needed.push_back(false);
      } else {
        st.out_slots.push_back(NewSlot(o));
        st.out_needed.push_back(graph_->NumConsumers(o) > 0);
      }
    }
    // implicit inputs of control-flow bodies must be alive in this executor too
    if (!n->subgraphs.empty()) {
      for (auto& v : graph_->ImplicitInputs(*n)) {
        if (graph_->IsConstant(v) || slot_of_.count(v)) continue;
        if (graph_->Parent() != nullptr) outer_slot(v);
      }
    }

    // kernel lookup: hand-written sm_100a kernel first for GPU nodes, then the ATen-backed one
    // ("ortb200.generic_kernels_only" = "1" keeps a session on the differentiable tensor-library set: training)
    const KernelDef* def = nullptr;
    if (st.on_gpu && session_->config().Get("ortb200.generic_kernels_only", "0") != "1") def = KernelRegistry::Cuda().Find(*n, *graph_);
    if (!def) def = KernelRegistry::Generic().Find(*n, *graph_);
    if (!def)
      ORTB_THROW(NOT_IMPLEMENTED, "Could not find an implementation for ", n->op_type, "(", n->since_version,
                 ") node with name '", n->name, "' (domain '", n->domain, "')");
    OpKernelInfo info{*n, *graph_, session_, st.device, &session_->config(),
                      [&const_inputs](int idx) -> const at::Tensor* {
                        return idx >= 0 && idx < static_cast<int>(const_inputs.size()) && const_inputs[idx].defined()
                                   ? &const_inputs[idx]
                                   : nullptr;
                      }};
    st.kernel = def->factory(info);
    for (int idx : st.kernel->PrepackedInputs())
      if (idx >= 0 && idx < static_cast<int>(st.in_slots.size())) st.in_slots[idx] = -1;
    steps_.push_back(std::move(st));
  }

  output_names_.clear();
  for (auto& o : graph_->Outputs()) {
    output_names_.push_back(o.name);
    if (!slot_of_.count(o.name)) {
      if (graph_->IsConstant(o.name)) const_slot(o.name, false);
      else if (graph_->Parent() != nullptr) outer_slot(o.name);
      else ORTB_THROW(INVALID_GRAPH, "graph output '", o.name, "' is not produced by any node");
    }
  }

  // constants that only pre-packing kernels consumed are no longer needed in their original layout
  {
    std::vector<bool> used(slot_names_.size(), false);
    for (auto& st : steps_)
      for (int s : st.in_slots)
        if (s >= 0) used[s] = true;
    for (auto& o : output_names_) used[slot_of_[o]] = true;
    for (int s : input_slot_) used[s] = true;
    for (int s : outer_slot_) used[s] = true;
    for (size_t s = 0; s < constant_slots_.size(); ++s) {
      if (used[s] || !constant_slots_[s].t.defined()) continue;
      constant_slots_[s] = Value();
      std::string name = slot_names_[s];
      const size_t suffix = name.find(kGpuSuffix);
      if (suffix != std::string::npos) name = name.substr(0, suffix);
      bool other_copy_used = false;
      for (const std::string& alt : {name, name + kGpuSuffix}) {
        auto it = slot_of_.find(alt);
        if (it != slot_of_.end() && used[it->second]) other_copy_used = true;
      }
      if (!other_copy_used && graph_->IsConstant(name) && graph_->Parent() == nullptr && graph_->Consumers(name).size() > 0) {
        bool subgraph_reader = false;
        for (Node* c : graph_->Consumers(name))
          if (!c->subgraphs.empty()) subgraph_reader = true;
        const at::Tensor* t = graph_->GetInitializer(name);
        if (!subgraph_reader && t && t->numel() > 4096)
          graph_->AddInitializer(name, at::empty({0}, t->options().device(c10::kCPU)));  // free the storage, keep the name
      }
    }
  }

  // release plan: a slot is dropped after the last step that reads it
  std::vector<int> last_use(slot_names_.size(), -1);
  for (size_t si = 0; si < steps_.size(); ++si) {
    for (int s : steps_[si].in_slots)
      if (s >= 0) last_use[s] = static_cast<int>(si);
    // bodies read captured values by name
    if (!steps_[si].node->subgraphs.empty())
      for (auto& v : graph_->ImplicitInputs(*steps_[si].node)) {
        auto it = slot_of_.find(v);
        if (it != slot_of_.end()) last_use[it->second] = static_cast<int>(si);
      }
  }
  std::vector<bool> keep(slot_names_.size(), false);
  for (size_t s = 0; s < constant_slots_.size(); ++s)
    if (constant_slots_[s].t.defined()) keep[s] = true;
  for (auto& o : output_names_) keep[slot_of_[o]] = true;
  for (int s : outer_slot_) keep[s] = true;
  for (size_t si = 0; si < steps_.size(); ++si) {
    for (int s : steps_[si].out_slots)
      if (s >= 0 && last_use[s] < 0 && !keep[s]) steps_[si].release.push_back(s);  // never read
  }
  for (size_t s = 0; s < last_use.size(); ++s)
    if (last_use[s] >= 0 && !keep[s]) steps_[last_use[s]].release.push_back(static_cast<int>(s));

  capturable_ = gpu;
  for (auto& st : steps_) {
    if (!st.on_gpu && !IsShapeOnlyOp(*st.node)) capturable_ = false;
    if (st.node->op_type == "MemcpyToHost") capturable_ = false;
  }
  BuildStepGraph();
  nvtx_ = session_->config().Get("ortb200.nvtx", "1") == "1";
}

namespace {
bool MovesElementsOnly(const Node& n) {
  static const std::set<std::string> ops = {"Identity", "Reshape", "Squeeze", "Unsqueeze", "Flatten", "Transpose", "Gather", "GatherElements",
                                            "GatherND", "Concat", "Slice", "Split", "Expand", "Tile", "Where", "Compress", "Pad",
                                            "DepthToSpace", "SpaceToDepth", "ReverseSequence", "ScatterElements", "ScatterND", "Unique",
                                            "MemcpyToHost", "MemcpyFromHost", "Optional", "OptionalGetElement"};
  return n.domain.empty() && ops.count(n.op_type) != 0;
}
}  // namespace

// One node: gather its inputs from the slots, run the kernel, put the outputs back.
void GraphExecutor::RunStep(const RunOptions& ro, const Step& st, std::vector<Value>& slots, OpKernelContext::Lookup* lookup, int node_index) {
  Profiler* prof = session_->profiler().enabled() ? &session_->profiler() : nullptr;
  std::vector<Value> in(st.in_slots.size()), out(st.out_slots.size());
  for (size_t i = 0; i < st.in_slots.size(); ++i)
    if (st.in_slots[i] >= 0) in[i] = slots[st.in_slots[i]];
  for (size_t i = 0; i < st.out_slots.size(); ++i)
    if (st.out_slots[i] >= 0) out[i] = slots[st.out_slots[i]];  // caller-bound output buffer, if any
  OpKernelContext ctx(*st.node, session_, st.device, in, out, st.out_needed);
  ctx.set_lookup(lookup);
  ctx.run_options = &ro;
  const int64_t t_node0 = prof ? prof->NowUs() : 0;
  NvtxRange range(nvtx_ ? st.node->name.c_str() : nullptr);  // one range per node: profiler timelines carry node names
  try {
    st.kernel->Compute(ctx);
    if (prof) {
      // per-node durations need the node's GPU work to have finished (profiling mode only)
      if (st.on_gpu && at::cuda::currentStreamCaptureStatusMayInitCtx() == c10::cuda::CaptureStatus::None) cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(st.device.index()).stream());
      std::map<std::string, std::string> args;
      args["op_name"] = st.node->op_type;
      args["provider"] = st.node->ep.empty() ? kCpuEP : st.node->ep;
      args["node_index"] = std::to_string(node_index);
      std::string shapes;
      for (auto& v : in)
        if (v.t.defined()) {
          std::ostringstream ss;
          ss << v.t.sizes();
          shapes += ss.str() + " ";
        }
      args["input_type_shape"] = shapes;
      prof->Record("Node", st.node->name + "_kernel_time", t_node0, prof->NowUs() - t_node0, std::move(args));
    }
  } catch (const OrtError&) {
    throw;
  } catch (const std::exception& e) {
    ORTB_THROW(RUNTIME_EXCEPTION, "Non-zero status code returned while running ", st.node->op_type, " node. Name:'",
               st.node->name, "' Status Message: ", e.what());
  }
  // operators that only move elements hand the string-ness of their data input on to their outputs
  if (!in.empty() && MovesElementsOnly(*st.node)) {
    bool strings = in[0].is_string;
    if (st.node->op_type == "Where" && in.size() > 1) strings = in[1].is_string;
    if (st.node->op_type == "Concat")
      for (auto& v : in) strings = strings || v.is_string;
    if (strings)
      for (auto& v : out) v.is_string = v.t.defined();
  }
  if (dump_.any) DumpNodeIO(dump_, *st.node, in, out);
  for (size_t i = 0; i < st.out_slots.size(); ++i) {
    const int s = st.out_slots[i];
    if (s < 0) continue;
    Value& bound = slots[s];
    if (bound.t.defined() && out[i].t.defined() && !bound.t.is_same(out[i].t) &&
        bound.t.data_ptr() != out[i].t.data_ptr()) {
      ORTB_ENFORCE_ARG(bound.t.sizes() == out[i].t.sizes(), "bound output '", slot_names_[s], "' has shape ",
                       bound.t.sizes(), " but the model produced ", out[i].t.sizes());
      bound.t.copy_(out[i].t, /*non_blocking=*/true);
    } else {
      slots[s] = std::move(out[i]);
    }
    if (tracing_ && slots[s].t.defined()) {
      const at::Tensor& t = slots[s].t;
      // a view of an input (Reshape, Squeeze, Identity ...) allocates nothing
      bool alias = false;
      for (auto& v : in)
        if (v.t.defined() && v.t.has_storage() && t.has_storage() && v.t.storage().data() == t.storage().data()) alias = true;
      SlotTrace& tr = trace_[static_cast<size_t>(s)];
      tr.bytes = alias || !t.has_storage() ? 0 : static_cast<int64_t>(t.storage().nbytes());
      tr.step = node_index;
      tr.on_gpu = t.is_cuda();
    }
  }
}

void GraphExecutor::BeginMemoryTrace() {
  trace_.assign(slot_names_.size(), SlotTrace());
  tracing_ = true;
}

std::vector<PlannedBuffer> GraphExecutor::EndMemoryTrace() {
  tracing_ = false;
  const int n = static_cast<int>(steps_.size());
  std::vector<int> last(slot_names_.size(), n - 1);  // values nobody releases (graph outputs) live to the end
  for (int i = 0; i < n; ++i)
    for (int s : steps_[static_cast<size_t>(i)].release) last[static_cast<size_t>(s)] = i;
  std::vector<PlannedBuffer> out;
  for (size_t s = 0; s < trace_.size(); ++s) {
    if (trace_[s].bytes < 0) continue;
    PlannedBuffer b;
    b.name = slot_names_[s];
    b.bytes = trace_[s].bytes;
    b.first_step = trace_[s].step;
    b.last_step = std::max(last[s], trace_[s].step);
    b.on_gpu = trace_[s].on_gpu;
    out.push_back(std::move(b));
  }
  trace_.clear();
  return out;
}

void GraphExecutor::ExecuteSteps(const RunOptions& ro, std::vector<Value>& slots) {
  const std::map<std::string, Value>* outer = current_outer_;
  OpKernelContext::Lookup lookup = [this, &slots, outer](const std::string& name) -> Value {
    auto it = slot_of_.find(name);
    if (it != slot_of_.end() && slots[it->second].defined()) return slots[it->second];
    if (graph_->IsInitializer(name)) {
      Value v;
      v.t = *graph_->GetInitializer(name);
      v.is_string = graph_->IsStringValue(name);
      return v;
    }
    if (outer) {
      auto ot = outer->find(name);
      if (ot != outer->end()) return ot->second;
    }
    ORTB_THROW(FAIL, "value '", name, "' is not available in the enclosing scope");
  };
  ThreadPool* pool = session_->InterOpPool();
  if (pool != nullptr && pool->NumThreads() > 0 && parallel_ok_ && steps_.size() > 1) {
    ExecuteStepsParallel(ro, slots, &lookup, pool);
    return;
  }
  int node_index = 0;
  for (auto& st : steps_) {
    if (ro.terminate && ro.terminate->load(std::memory_order_relaxed))
      ORTB_THROW(FAIL, "Exiting due to terminate flag being set to true.");
    RunStep(ro, st, slots, &lookup, node_index++);
    for (int s : st.release) slots[s] = Value();
  }
}

// ExecutionMode::ORT_PARALLEL (host graphs): a node is queued on the inter-op pool as soon as the nodes that produce
// its inputs have finished; the calling thread helps until the graph is done.  Nodes with control-flow bodies read
// values by name, so they wait for everything before them and everything after them waits for them.  Values are
// released when the run ends (a release list assumes program order).  The reference's counterpart is the parallel
// branch of onnxruntime/core/framework/sequential_executor.cc:526-771 (one task per logic stream).
void GraphExecutor::ExecuteStepsParallel(const RunOptions& ro, std::vector<Value>& slots, OpKernelContext::Lookup* lookup, ThreadPool* pool) {
  const size_t n = steps_.size();
  std::vector<std::atomic<int>> pending(n);
  for (size_t i = 0; i < n; ++i) pending[i].store(static_cast<int>(step_deps_[i].size()), std::memory_order_relaxed);
  std::atomic<size_t> finished{0};
  std::atomic<bool> failed{false};
  std::exception_ptr first_error;
  std::mutex err_mu;
  std::function<void(size_t)> run = [&](size_t i) {
    if (!failed.load(std::memory_order_acquire) && !(ro.terminate && ro.terminate->load(std::memory_order_relaxed))) {
      try {
        RunStep(ro, steps_[i], slots, lookup, static_cast<int>(i));
      } catch (...) {
        std::lock_guard<std::mutex> lk(err_mu);
        if (!first_error) first_error = std::current_exception();
        failed.store(true, std::memory_order_release);
      }
    }
    for (int succ : step_succ_[i])
      if (pending[static_cast<size_t>(succ)].fetch_sub(1, std::memory_order_acq_rel) == 1) pool->Schedule([&run, succ] { run(static_cast<size_t>(succ)); });
    finished.fetch_add(1, std::memory_order_acq_rel);
  };
  for (size_t i = 0; i < n; ++i)
    if (step_deps_[i].empty()) pool->Schedule([&run, i] { run(i); });
  pool->HelpUntil([&] { return finished.load(std::memory_order_acquire) == n; });
  if (first_error) std::rethrow_exception(first_error);
  if (ro.terminate && ro.terminate->load(std::memory_order_relaxed)) ORTB_THROW(FAIL, "Exiting due to terminate flag being set to true.");
}

// Dependencies between steps, from the slots they read and write.
void GraphExecutor::BuildStepGraph() {
  const size_t n = steps_.size();
  step_deps_.assign(n, {});
  step_succ_.assign(n, {});
  std::map<int, int> producer;  // slot -> step
  int last_barrier = -1;
  parallel_ok_ = true;
  for (size_t i = 0; i < n; ++i) {
    const Step& st = steps_[i];
    std::set<int> deps;
    const bool barrier = !st.node->subgraphs.empty();
    if (barrier) {
      for (size_t j = 0; j < i; ++j) deps.insert(static_cast<int>(j));
    } else {
      if (last_barrier >= 0) deps.insert(last_barrier);
      for (int s : st.in_slots) {
        auto it = s >= 0 ? producer.find(s) : producer.end();
        if (it != producer.end()) deps.insert(it->second);
      }
    }
    for (int s : st.out_slots) {
      if (s < 0) continue;
      auto it = producer.find(s);
      if (it != producer.end()) deps.insert(it->second);  // two writers of one slot keep their order
      producer[s] = static_cast<int>(i);
    }
    if (barrier) last_barrier = static_cast<int>(i);
    if (st.on_gpu) parallel_ok_ = false;  // device work is ordered by its stream: nothing to gain, a lot to break
    step_deps_[i].assign(deps.begin(), deps.end());
    for (int d : deps) step_succ_[static_cast<size_t>(d)].push_back(static_cast<int>(i));
  }
}

std::vector<Value> GraphExecutor::Run(const RunOptions& ro, const std::vector<Value>& inputs,
                                      const std::map<std::string, Value>* outer,
                                      const std::vector<std::string>& output_names) {
  std::vector<Value> slots = constant_slots_;
  ORTB_ENFORCE(inputs.size() == input_slot_.size(), "executor expected ", input_slot_.size(), " inputs, got ",
               inputs.size());
  for (size_t i = 0; i < inputs.size(); ++i)
    if (inputs[i].defined()) slots[input_slot_[i]] = inputs[i];
  for (size_t i = 0; i < outer_names_.size(); ++i) {
    ORTB_ENFORCE(outer != nullptr, "subgraph needs outer-scope values");
    auto it = outer->find(outer_names_[i]);
    ORTB_ENFORCE(it != outer->end(), "outer-scope value '", outer_names_[i], "' not available");
    slots[outer_slot_[i]] = it->second;
  }
  current_outer_ = outer;
  ExecuteSteps(ro, slots);
  current_outer_ = nullptr;
  std::vector<Value> result;
  result.reserve(output_names.size());
  for (auto& n : output_names) {
    auto it = slot_of_.find(n);
    ORTB_ENFORCE_ARG(it != slot_of_.end(), "unknown output '", n, "'");
    result.push_back(slots[it->second]);
  }
  return result;
}

}  // namespace ortb
