#include "optimizer.h"
#include "shape_inference.h"

#include <cmath>

#include "kernel.h"

namespace ortb {
namespace opt {

Pat V(const std::string& name) {
  Pat p;
  p.kind = Pat::VAR;
  p.name = name;
  return p;
}
Pat C(double value) {
  Pat p;
  p.kind = Pat::CONST;
  p.cval = value;
  return p;
}
Pat K(const std::string& name) {
  Pat p;
  p.kind = Pat::ANYCONST;
  p.name = name;
  return p;
}
Pat Op(const std::string& op, std::vector<Pat> args, const std::string& bind) { return OpD("", op, std::move(args), bind); }
Pat OpD(const std::string& domain, const std::string& op, std::vector<Pat> args, const std::string& bind) {
  Pat p;
  p.kind = Pat::OP;
  p.op = op;
  p.domain = domain;
  p.args = std::move(args);
  p.name = bind;
  p.commutative = (op == "Add" || op == "Mul") && p.args.size() == 2;
  return p;
}

bool ScalarConst(const Graph& g, const std::string& value, double* out) {
  const at::Tensor* t = g.GetConstant(value);
  if (!t) {
    // a Constant node that has not been folded yet
    Node* n = g.Producer(value);
    if (n && n->op_type == "Constant" && n->domain.empty() && n->has_attr("value")) {
      at::Tensor v = n->attr_tensor("value");
      if (v.numel() != 1) return false;
      *out = v.to(at::kDouble).reshape({-1})[0].item<double>();
      return true;
    }
    return false;
  }
  if (t->numel() != 1) return false;
  *out = t->to(at::kCPU, at::kDouble).reshape({-1})[0].item<double>();
  return true;
}

bool IsConst1D(const Graph& g, const std::string& value, int64_t* len) {
  const at::Tensor* t = g.GetConstant(value);
  if (!t || t->dim() != 1) return false;
  if (len) *len = t->size(0);
  return true;
}

namespace {

bool MatchRec(const Graph& g, const std::string& value, const Pat& p, Match* m, bool through_casts) {
  switch (p.kind) {
    case Pat::VAR: {
      auto it = m->values.find(p.name);
      if (it != m->values.end()) return it->second == value;
      m->values[p.name] = value;
      return true;
    }
    case Pat::CONST: {
      double v;
      if (!ScalarConst(g, value, &v)) return false;
      const double tol = std::max(std::abs(p.cval) * p.tol, 1e-6);
      return std::abs(v - p.cval) <= tol;
    }
    case Pat::ANYCONST: {
      if (!g.GetConstant(value)) return false;
      auto it = m->values.find(p.name);
      if (it != m->values.end()) return it->second == value;
      m->values[p.name] = value;
      return true;
    }
    case Pat::OP: {
      if (!p.name.empty()) {
        auto it = m->values.find(p.name);
        if (it != m->values.end() && it->second == value) return true;  // same sub-expression seen before
      }
      Node* n = g.Producer(value);
      if (!n) return false;
      if (through_casts && n->op_type == "Cast" && n->domain.empty() && p.op != "Cast") {
        Match save = *m;
        m->matched.push_back(n);
        if (MatchRec(g, n->inputs[0], p, m, through_casts)) return true;
        *m = save;
        return false;
      }
      if (n->op_type != p.op || n->domain != p.domain) return false;
      size_t present = 0;
      for (auto& i : n->inputs)
        if (!i.empty()) ++present;
      if (present < p.args.size()) return false;
      if (present > p.args.size() && !p.allow_extra_inputs) return false;
      auto try_order = [&](bool swap) {
        Match save = *m;
        m->matched.push_back(n);
        bool ok = true;
        for (size_t i = 0; i < p.args.size() && ok; ++i) {
          const size_t src = (swap && p.args.size() == 2) ? 1 - i : i;
          ok = MatchRec(g, n->inputs[src], p.args[i], m, through_casts);
        }
        if (!ok) *m = save;
        return ok;
      };
      bool ok = try_order(false);
      if (!ok && p.commutative) ok = try_order(true);
      if (ok && !p.name.empty()) {
        if (!m->values.count(p.name)) m->values[p.name] = value;
        m->nodes[p.name] = n;
      }
      return ok;
    }
  }
  return false;
}

}  // namespace

bool MatchExpr(const Graph& g, const std::string& value, const Pat& p, Match* m, bool through_casts) {
  m->values.clear();
  m->nodes.clear();
  m->matched.clear();
  if (!MatchRec(g, value, p, m, through_casts)) return false;
  // de-duplicate matched nodes, keep order
  std::vector<Node*> uniq;
  std::set<Node*> seen;
  for (Node* n : m->matched)
    if (seen.insert(n).second) uniq.push_back(n);
  m->matched = uniq;
  return true;
}

bool IsClosed(const Graph& g, const Match& m, const Node* root, const std::set<std::string>& allowed_escapes) {
  std::set<const Node*> inside(m.matched.begin(), m.matched.end());
  for (Node* n : m.matched) {
    if (n == root) continue;
    for (auto& o : n->outputs) {
      if (o.empty()) continue;
      if (allowed_escapes.count(o)) continue;
      if (g.IsGraphOutput(o)) return false;
      for (Node* c : g.Consumers(o))
        if (!inside.count(c)) return false;
    }
  }
  return true;
}

void RemoveMatched(Graph& g, const Match& m) {
  for (Node* n : m.matched) g.RemoveNode(n);
}

const std::vector<Pass>& AllPasses() {
  static std::vector<Pass> passes = [] {
    std::vector<Pass> v;
    AddBasicPasses(v);
    AddFusionPasses(v);
    AddMorePasses(v);
    AddQdqPrepPasses(v);  // every quantised node unit gets its own DequantizeLinear before the QDQ fusions look
    AddQdqPasses(v);  // after the transformer fusions: those match the un-simplified MatMul / Add / Softmax forms
    AddMorePasses2(v);  // MatMul scale / transpose folding and the conv fusions come last for the same reason
    AddMorePasses3(v);
    AddGpuPasses(v);
    return v;
  }();
  return passes;
}

}  // namespace opt

// Evaluate one node with the generic (ATen) kernels on whatever device its inputs live on.
std::vector<at::Tensor> EvaluateNodeOnCpu(const Node& node, const Graph& g, const std::vector<at::Tensor>& inputs) {
  EnsureKernelsRegistered();
  const KernelDef* d = KernelRegistry::Generic().Find(node, g);
  if (!d) ORTB_THROW(NOT_IMPLEMENTED, "no kernel for ", node.op_type);
  c10::Device dev(c10::kCPU);
  for (auto& t : inputs)
    if (t.defined() && t.is_cuda()) dev = t.device();
  static const ConfigOptions empty_cfg;
  OpKernelInfo info{node, g, nullptr, dev, &empty_cfg, [&inputs](int i) -> const at::Tensor* {
                      return i >= 0 && i < static_cast<int>(inputs.size()) && inputs[i].defined() ? &inputs[i] : nullptr;
                    }};
  std::unique_ptr<OpKernel> k = d->factory(info);
  std::vector<Value> in(inputs.size()), out(node.outputs.size());
  for (size_t i = 0; i < inputs.size(); ++i) {
    in[i].t = inputs[i];
    // shape-like operands are read on the host
    if (in[i].t.defined() && in[i].t.is_cuda() &&
        std::find(d->host_inputs.begin(), d->host_inputs.end(), static_cast<int>(i)) != d->host_inputs.end())
      in[i].t = in[i].t.cpu();
  }
  std::vector<bool> needed(node.outputs.size(), true);
  OpKernelContext ctx(node, nullptr, dev, in, out, needed);
  k->Compute(ctx);
  std::vector<at::Tensor> res;
  for (auto& v : out) res.push_back(v.t);
  return res;
}

OptimizerStats OptimizeGraph(Graph& g, int level, const std::set<std::string>& disabled, bool gpu,
                             const ConfigOptions& config, int world_size) {
  OptimizerStats stats;
  if (level <= 0) return stats;
  // several rules ask for ranks and element types: resolve what can be resolved statically first
  InferShapes(g, false);
  opt::PassContext ctx{g, gpu, config, world_size};
  int loops = 1;
  const std::string loop_cfg = config.Get("session.graph_optimizations_loop_level", "1");
  if (!loop_cfg.empty()) loops = std::max(1, std::min(10, std::stoi(loop_cfg) + 1));
  for (int iter = 0; iter < loops + 1; ++iter) {
    int changed = 0;
    for (auto& p : opt::AllPasses()) {
      if (p.level > level) continue;
      if (p.gpu_only && !gpu) continue;
      if (disabled.count(p.name)) continue;
      const int n = p.run(ctx);
      g.PurgeRemoved();  // no pass keeps node pointers beyond its own run
      if (n > 0) {
        stats.applied[p.name] += n;
        changed += n;
        g.RemoveDeadNodes();
      }
    }
    if (!changed) break;
  }
  g.RemoveDeadNodes();
  g.PurgeRemoved();
  // recurse into control-flow bodies with the basic passes
  for (Node* n : g.Nodes())
    for (auto& kv : n->subgraphs) {
      OptimizerStats sub = OptimizeGraph(*kv.second, std::min(level, 1), disabled, gpu, config, world_size);
      for (auto& a : sub.applied) stats.applied[a.first] += a.second;
    }
  return stats;
}

}  // namespace ortb
