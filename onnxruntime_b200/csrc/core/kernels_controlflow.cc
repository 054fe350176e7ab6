// If / Loop / Scan.  Each body graph gets its own GraphExecutor, built on first
// use when the devices of the captured values and body inputs are known
// (reference: onnxruntime/core/providers/cpu/controlflow/{if,loop,scan_9}.cc,
// which create a sub-SessionState per body).
#include <ATen/ATen.h>

#include <mutex>

#include "executor.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

struct Body {
  std::shared_ptr<Graph> graph;
  std::unique_ptr<GraphExecutor> exec;
  std::vector<std::string> implicit;  // captured value names
};

class ControlFlowBase : public OpKernel {
 public:
  explicit ControlFlowBase(const OpKernelInfo& info) : OpKernel(info), session_(info.session), parent_graph_(&info.graph) {}

 protected:
  void Prepare(Body& body, Ctx& ctx, const std::vector<Value>& body_inputs) const {
    if (body.exec) return;
    std::map<std::string, bool> outer_on_gpu;
    for (auto& name : body.implicit) {
      Value v = ctx.LookupValue(name);
      outer_on_gpu[name] = v.t.defined() && v.t.is_cuda();
    }
    const auto& ins = body.graph->Inputs();
    for (size_t i = 0; i < ins.size() && i < body_inputs.size(); ++i)
      outer_on_gpu["\x02input:" + ins[i].name] = body_inputs[i].t.defined() && body_inputs[i].t.is_cuda();
    auto ex = std::make_unique<GraphExecutor>(session_, body.graph.get(), &outer_on_gpu);
    ex->Build();
    body.exec = std::move(ex);
  }

  std::vector<Value> RunBody(Body& body, Ctx& ctx, const std::vector<Value>& inputs) const {
    Prepare(body, ctx, inputs);
    std::map<std::string, Value> outer;
    for (auto& name : body.exec->outer_names()) outer[name] = ctx.LookupValue(name);
    std::vector<Value> ordered(body.exec->input_names().size());
    const auto& gi = body.graph->Inputs();
    // executor inputs follow graph input order minus constant initializers
    size_t k = 0;
    for (size_t i = 0; i < gi.size() && k < ordered.size(); ++i) {
      if (body.exec->input_names()[k] != gi[i].name) continue;
      if (i < inputs.size()) ordered[k] = inputs[i];
      ++k;
    }
    static const RunOptions default_ro;
    const RunOptions& ro = ctx.run_options ? *ctx.run_options : default_ro;
    return body.exec->Run(ro, ordered, &outer, body.exec->output_names());
  }

  Body MakeBody(const std::string& attr) const {
    auto it = node_.subgraphs.find(attr);
    if (it == node_.subgraphs.end()) ORTB_THROW(INVALID_GRAPH, node_.op_type, " node '", node_.name, "' has no ", attr);
    Body b;
    b.graph = it->second;
    Node probe;
    probe.subgraphs[attr] = it->second;
    b.implicit = parent_graph_->ImplicitInputs(probe);
    return b;
  }

  at::Tensor ToSessionDevice(const at::Tensor& t) const {
    if (!t.defined() || !session_ || !session_->uses_gpu() || t.is_cuda()) return t;
    return t.to(session_->device());
  }

  InferenceSession* session_;
  const Graph* parent_graph_;
  mutable std::mutex mu_;
};

class IfKernel final : public ControlFlowBase {
 public:
  explicit IfKernel(const OpKernelInfo& info) : ControlFlowBase(info) {
    then_ = MakeBody("then_branch");
    else_ = MakeBody("else_branch");
  }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    const bool cond = ctx.RequiredInput(0).cpu().reshape({-1})[0].item<bool>();
    Body& b = cond ? then_ : else_;
    std::vector<Value> outs = RunBody(b, ctx, {});
    for (int i = 0; i < ctx.OutputCount() && i < static_cast<int>(outs.size()); ++i) {
      if (outs[i].seq) ctx.SetOutputSeq(i, *outs[i].seq);
      else ctx.SetOutput(i, ToSessionDevice(outs[i].t));
    }
  }

 private:
  mutable Body then_, else_;
};

class LoopKernel final : public ControlFlowBase {
 public:
  explicit LoopKernel(const OpKernelInfo& info) : ControlFlowBase(info) { body_ = MakeBody("body"); }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    int64_t max_trip = std::numeric_limits<int64_t>::max();
    if (ctx.HasInput(0)) max_trip = ctx.Input(0).cpu().reshape({-1})[0].item<int64_t>();
    bool cond = true;
    if (ctx.HasInput(1)) cond = ctx.Input(1).cpu().reshape({-1})[0].item<bool>();
    const int n_carried = ctx.InputCount() - 2;
    std::vector<Value> carried;
    for (int i = 0; i < n_carried; ++i) carried.push_back(ctx.InputValue(2 + i));
    const int n_body_out = static_cast<int>(body_.graph->Outputs().size());
    const int n_scan = n_body_out - 1 - n_carried;
    ORTB_ENFORCE(n_scan >= 0, "Loop body has too few outputs");
    std::vector<std::vector<at::Tensor>> scans(n_scan);
    for (int64_t it = 0; it < max_trip && cond; ++it) {
      std::vector<Value> in(2 + n_carried);
      in[0].t = at::scalar_tensor(it, at::kLong);
      in[1].t = at::scalar_tensor(cond, at::kBool);
      for (int i = 0; i < n_carried; ++i) in[2 + i] = carried[i];
      std::vector<Value> out = RunBody(body_, ctx, in);
      cond = out[0].t.cpu().reshape({-1})[0].item<bool>();
      for (int i = 0; i < n_carried; ++i) carried[i] = out[1 + i];
      for (int i = 0; i < n_scan; ++i) scans[i].push_back(out[1 + n_carried + i].t);
    }
    for (int i = 0; i < n_carried; ++i) {
      if (carried[i].seq) ctx.SetOutputSeq(i, *carried[i].seq);
      else ctx.SetOutput(i, ToSessionDevice(carried[i].t));
    }
    for (int i = 0; i < n_scan; ++i) {
      if (scans[i].empty()) {
        ctx.SetOutput(n_carried + i, at::empty({0}, at::TensorOptions().device(ctx.device())));
      } else {
        ctx.SetOutput(n_carried + i, ToSessionDevice(at::stack(scans[i], 0)));
      }
    }
  }

 private:
  mutable Body body_;
};

class ScanKernel final : public ControlFlowBase {
 public:
  explicit ScanKernel(const OpKernelInfo& info) : ControlFlowBase(info) { body_ = MakeBody("body"); }
  void Compute(Ctx& ctx) const override {
    std::lock_guard<std::mutex> lk(mu_);
    const Node& n = ctx.node();
    const int64_t m = n.attr_i("num_scan_inputs", 0);
    const int total_in = ctx.InputCount();
    const int n_state = total_in - static_cast<int>(m);
    std::vector<int64_t> in_axes = n.attr_ints("scan_input_axes"), in_dirs = n.attr_ints("scan_input_directions");
    std::vector<int64_t> out_axes = n.attr_ints("scan_output_axes"), out_dirs = n.attr_ints("scan_output_directions");
    in_axes.resize(m, 0);
    in_dirs.resize(m, 0);
    const int n_body_out = static_cast<int>(body_.graph->Outputs().size());
    const int k = n_body_out - n_state;
    out_axes.resize(k, 0);
    out_dirs.resize(k, 0);
    std::vector<Value> state;
    for (int i = 0; i < n_state; ++i) state.push_back(ctx.InputValue(i));
    std::vector<at::Tensor> scan_in;
    int64_t len = -1;
    for (int64_t i = 0; i < m; ++i) {
      at::Tensor t = ctx.RequiredInput(n_state + static_cast<int>(i));
      int64_t ax = in_axes[i] < 0 ? in_axes[i] + t.dim() : in_axes[i];
      in_axes[i] = ax;
      if (len < 0) len = t.size(ax);
      ORTB_ENFORCE_ARG(t.size(ax) == len, "Scan inputs disagree on sequence length");
      scan_in.push_back(t);
    }
    std::vector<std::vector<at::Tensor>> outs(k);
    for (int64_t s = 0; s < len; ++s) {
      std::vector<Value> in(n_state + m);
      for (int i = 0; i < n_state; ++i) in[i] = state[i];
      for (int64_t i = 0; i < m; ++i) {
        const int64_t idx = in_dirs[i] ? len - 1 - s : s;
        in[n_state + i].t = scan_in[i].select(in_axes[i], idx).contiguous();
      }
      std::vector<Value> out = RunBody(body_, ctx, in);
      for (int i = 0; i < n_state; ++i) state[i] = out[i];
      for (int i = 0; i < k; ++i) outs[i].push_back(out[n_state + i].t);
    }
    for (int i = 0; i < n_state; ++i) ctx.SetOutput(i, ToSessionDevice(state[i].t));
    for (int i = 0; i < k; ++i) {
      if (outs[i].empty()) continue;
      if (out_dirs[i]) std::reverse(outs[i].begin(), outs[i].end());
      int64_t ax = out_axes[i];
      if (ax < 0) ax += outs[i][0].dim() + 1;
      ctx.SetOutput(n_state + i, ToSessionDevice(at::stack(outs[i], ax)));
    }
  }

 private:
  mutable Body body_;
};

template <typename K>
void RegisterClass(KernelRegistry& r, const std::string& op, int since, std::vector<int> host) {
  KernelDef d;
  d.domain = "";
  d.op_type = op;
  d.since_min = since;
  d.since_max = kMax;
  d.host_inputs = std::move(host);
  d.factory = [](const OpKernelInfo& info) { return std::make_unique<K>(info); };
  r.Register(std::move(d));
}

}  // namespace

void RegisterControlFlowKernels(KernelRegistry& r) {
  RegisterClass<IfKernel>(r, "If", 1, {0});
  RegisterClass<LoopKernel>(r, "Loop", 1, {0, 1});
  RegisterClass<ScanKernel>(r, "Scan", 9, {});
}

}  // namespace ortb
