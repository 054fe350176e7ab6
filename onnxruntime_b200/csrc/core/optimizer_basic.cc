// Level-1 ("basic") graph optimizations: no-op elimination, constant folding,
// common-subexpression elimination, Conv+BatchNorm folding and the Gelu /
// LayerNorm / SimplifiedLayerNorm (RMSNorm) subgraph fusions.
//
// Reference passes: identity_elimination.cc, dropout_elimination.cc,
// noop_elimination.cc, constant_folding.cc (:391 runs CPU kernels),
// common_subexpression_elimination.cc, conv_bn_fusion.cc, gelu_fusion.cc
// (:82-153), layer_norm_fusion.cc (:174-202 LayerNorm, :615-637 RMS form).
#include <cmath>

#include "optimizer.h"

namespace ortb {
namespace opt {

namespace {

bool IsSingleOutputPassthrough(Graph& g, Node* n, const std::string& in, const std::string& out) {
  // Bypassing the node must not turn a graph output into a graph input / initializer alias.
  if (g.IsGraphOutput(out) && (g.IsGraphInput(in) || g.IsInitializer(in) || g.IsGraphOutput(in))) return false;
  return true;
}

void Bypass(Graph& g, Node* n, const std::string& in, const std::string& out) {
  if (g.IsGraphOutput(out)) {
    // rename the producer's output instead, so the graph output name survives
    Node* p = g.Producer(in);
    if (p && g.NumConsumers(in) == 1) {
      for (auto& o : p->outputs)
        if (o == in) o = out;
      g.RemoveNode(n);
      g.Invalidate();
      return;
    }
    return;  // keep the node
  }
  g.ReplaceAllUses(out, in);
  g.RemoveNode(n);
}

int EliminateIdentity(PassContext& c) {
  int count = 0;
  for (Node* n : c.g.Nodes()) {
    if (!n->domain.empty()) continue;
    const bool identity = n->op_type == "Identity";
    const bool dropout = n->op_type == "Dropout" && (!n->has_output(1) || c.g.NumConsumers(n->outputs[1]) == 0) &&
                         n->attr_i("training_mode", 0) == 0 && !n->has_input(2);
    if (!identity && !dropout) continue;
    if (!n->has_input(0) || !n->has_output(0)) continue;
    const std::string in = n->inputs[0], out = n->outputs[0];
    if (!IsSingleOutputPassthrough(c.g, n, in, out)) continue;
    const size_t before = c.g.NumNodes();
    Bypass(c.g, n, in, out);
    if (c.g.NumNodes() < before) ++count;
  }
  return count;
}

int EliminateNoop(PassContext& c) {
  int count = 0;
  for (Node* n : c.g.Nodes()) {
    if (!n->domain.empty() || n->inputs.size() != 2) continue;
    const std::string& op = n->op_type;
    if (op != "Add" && op != "Sub" && op != "Mul" && op != "Div") continue;
    const double neutral = (op == "Add" || op == "Sub") ? 0.0 : 1.0;
    for (int side = 0; side < 2; ++side) {
      if (side == 0 && (op == "Sub" || op == "Div")) continue;  // 0 - x and 1 / x are not no-ops
      const at::Tensor* k = c.g.GetConstant(n->inputs[side]);
      if (!k || k->dim() != 0 || k->numel() != 1) continue;
      if (!c10::isFloatingType(k->scalar_type())) continue;
      if (k->to(at::kCPU, at::kDouble).item<double>() != neutral) continue;
      const std::string in = n->inputs[1 - side], out = n->outputs[0];
      if (!IsSingleOutputPassthrough(c.g, n, in, out)) break;
      const size_t before = c.g.NumNodes();
      Bypass(c.g, n, in, out);
      if (c.g.NumNodes() < before) ++count;
      break;
    }
  }
  return count;
}

bool Foldable(const Node& n) {
  static const std::set<std::string> never = {
      "RandomNormal", "RandomNormalLike", "RandomUniform", "RandomUniformLike", "Multinomial", "Bernoulli",
      "If", "Loop", "Scan", "SequenceMap", "QuantizeLinear", "DequantizeLinear", "DynamicQuantizeLinear", "MemcpyToHost",
      "MemcpyFromHost", "AllReduce", "AllGather", "AllToAll", "ShardedMoE", "SequenceConstruct", "SequenceEmpty",
      "SplitToSequence", "SequenceInsert", "SequenceErase", "SequenceAt", "SequenceLength", "ConcatFromSequence"};
  if (never.count(n.op_type)) return false;
  if (n.op_type.rfind("Distributed", 0) == 0) return false;
  if (!n.subgraphs.empty()) return false;
  if (n.op_type == "Constant" && ConstantHoldsStrings(n)) return false;  // an initializer would lose the string flag
  return true;
}

int ConstantFolding(PassContext& c) {
  int count = 0;
  Graph& g = c.g;
  for (Node* n : g.TopologicalOrder()) {
    if (!Foldable(*n)) continue;
    std::vector<at::Tensor> inputs;
    bool all_const = true;
    int64_t in_bytes = 0;
    for (auto& i : n->inputs) {
      if (i.empty()) {
        inputs.emplace_back();
        continue;
      }
      const at::Tensor* t = g.GetConstant(i);
      if (!t) {
        all_const = false;
        break;
      }
      inputs.push_back(*t);
      in_bytes += static_cast<int64_t>(t->nbytes());
    }
    if (!all_const) continue;
    if (n->inputs.empty() && n->op_type != "Constant") continue;
    bool any_out_used = false;
    for (auto& o : n->outputs)
      if (!o.empty() && g.NumConsumers(o) > 0) any_out_used = true;
    if (!any_out_used) continue;
    std::vector<at::Tensor> outs;
    try {
      outs = EvaluateNodeOnCpu(*n, g, inputs);
    } catch (const std::exception&) {
      continue;  // not foldable with the kernels we have; leave it for run time
    }
    int64_t out_bytes = 0;
    bool ok = true;
    for (size_t i = 0; i < n->outputs.size(); ++i) {
      if (n->outputs[i].empty()) continue;
      if (i >= outs.size() || !outs[i].defined()) {
        if (g.NumConsumers(n->outputs[i]) > 0) ok = false;
        continue;
      }
      out_bytes += static_cast<int64_t>(outs[i].nbytes());
    }
    // do not materialise large broadcast results (Expand / Tile / ConstantOfShape of a small constant)
    if (!ok || (out_bytes > (16 << 20) && out_bytes > 4 * std::max<int64_t>(in_bytes, 1))) continue;
    for (size_t i = 0; i < n->outputs.size(); ++i) {
      if (n->outputs[i].empty() || i >= outs.size() || !outs[i].defined()) continue;
      at::Tensor t = outs[i].contiguous();
      if (g.IsGraphOutput(n->outputs[i])) {
        // keep a producer for graph outputs: turn the node into a Constant
        ok = false;
      }
      if (ok) g.AddInitializer(n->outputs[i], t);
    }
    if (!ok) continue;
    g.RemoveNode(n);
    ++count;
  }
  return count;
}

std::string AttrSignature(const pb::AttributeProto& a) {
  std::ostringstream ss;
  ss << a.name << ":" << a.type << ":";
  switch (a.type) {
    case pb::ATTR_INT: ss << a.i; break;
    case pb::ATTR_FLOAT: ss << a.f; break;
    case pb::ATTR_STRING: ss << a.s; break;
    case pb::ATTR_INTS: for (auto v : a.ints) ss << v << ","; break;
    case pb::ATTR_FLOATS: for (auto v : a.floats) ss << v << ","; break;
    case pb::ATTR_STRINGS: for (auto& v : a.strings) ss << v << ","; break;
    case pb::ATTR_TENSOR: if (a.t) ss << pb::SerializeTensor(*a.t); break;
    default: ss << "?" << reinterpret_cast<uintptr_t>(&a);  // never equal
  }
  return ss.str();
}

int CommonSubexpressionElimination(PassContext& c) {
  int count = 0;
  Graph& g = c.g;
  std::map<std::string, Node*> seen;
  for (Node* n : g.TopologicalOrder()) {
    if (!Foldable(*n) || n->op_type == "Constant") continue;
    bool out_is_graph_output = false;
    for (auto& o : n->outputs)
      if (!o.empty() && g.IsGraphOutput(o)) out_is_graph_output = true;
    if (out_is_graph_output) continue;
    std::ostringstream key;
    key << n->domain << "|" << n->op_type << "|" << n->outputs.size() << "|";
    for (auto& i : n->inputs) key << i << ",";
    key << "|";
    for (auto& kv : n->attrs) key << AttrSignature(kv.second) << ";";
    auto it = seen.find(key.str());
    if (it == seen.end()) {
      seen[key.str()] = n;
      continue;
    }
    Node* keep = it->second;
    for (size_t i = 0; i < n->outputs.size(); ++i)
      if (!n->outputs[i].empty() && i < keep->outputs.size() && !keep->outputs[i].empty())
        g.ReplaceAllUses(n->outputs[i], keep->outputs[i]);
    g.RemoveNode(n);
    ++count;
  }
  return count;
}

int ConvBatchNormFusion(PassContext& c) {
  int count = 0;
  Graph& g = c.g;
  for (Node* bn : g.Nodes()) {
    if (bn->op_type != "BatchNormalization" || !bn->domain.empty() || bn->inputs.size() < 5) continue;
    Node* conv = g.Producer(bn->inputs[0]);
    if (!conv || conv->op_type != "Conv" || !conv->domain.empty()) continue;
    if (g.NumConsumers(conv->outputs[0]) != 1) continue;
    const at::Tensor* w = g.GetConstant(conv->input(1));
    const at::Tensor* scale = g.GetConstant(bn->inputs[1]);
    const at::Tensor* bias = g.GetConstant(bn->inputs[2]);
    const at::Tensor* mean = g.GetConstant(bn->inputs[3]);
    const at::Tensor* var = g.GetConstant(bn->inputs[4]);
    if (!w || !scale || !bias || !mean || !var) continue;
    const at::Tensor* cb = conv->has_input(2) ? g.GetConstant(conv->inputs[2]) : nullptr;
    if (conv->has_input(2) && !cb) continue;
    for (size_t i = 1; i < bn->outputs.size(); ++i)
      if (!bn->outputs[i].empty() && g.NumConsumers(bn->outputs[i]) > 0) goto next;
    {
      const double eps = bn->attr_f("epsilon", 1e-5f);
      at::Tensor f = scale->to(at::kFloat) / at::sqrt(var->to(at::kFloat) + eps);
      std::vector<int64_t> shape(w->dim(), 1);
      shape[0] = -1;
      at::Tensor new_w = (w->to(at::kFloat) * f.reshape(shape)).to(w->scalar_type());
      at::Tensor b0 = cb ? cb->to(at::kFloat) : at::zeros_like(f);
      at::Tensor new_b = ((b0 - mean->to(at::kFloat)) * f + bias->to(at::kFloat)).to(w->scalar_type());
      const std::string wn = g.UniqueName(conv->inputs[1] + "_bn"), bname = g.UniqueName(conv->name + "_bias_bn");
      g.AddInitializer(wn, new_w);
      g.AddInitializer(bname, new_b);
      conv->inputs.resize(3);
      conv->inputs[1] = wn;
      conv->inputs[2] = bname;
      conv->outputs[0] = bn->outputs[0];
      g.RemoveNode(bn);
      g.Invalidate();
      ++count;
    }
  next:;
  }
  return count;
}

// --------------------------------------------------------------- Gelu
int GeluFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  // erf argument: x / sqrt(2) or x * (1 / sqrt(2))
  auto erf_arg = [](int form) {
    return form == 0 ? Op("Div", {V("x"), C(1.4142135623730951)}) : Op("Mul", {V("x"), C(0.7071067811865476)});
  };
  std::vector<Pat> pats;
  for (int form = 0; form < 2; ++form) {
    Pat one_plus_erf = Op("Add", {Op("Erf", {erf_arg(form)}), C(1.0)});
    pats.push_back(Op("Mul", {Op("Mul", {V("x"), one_plus_erf}), C(0.5)}));   // (x * (1 + erf)) * 0.5
    pats.push_back(Op("Mul", {Op("Mul", {V("x"), C(0.5)}), one_plus_erf}));   // (x * 0.5) * (1 + erf)
    pats.push_back(Op("Mul", {V("x"), Op("Mul", {one_plus_erf, C(0.5)})}));   // x * ((1 + erf) * 0.5)
  }
  for (Node* n : g.Nodes()) {
    if (n->op_type != "Mul" || !n->domain.empty()) continue;
    for (auto& p : pats) {
      Match m;
      if (!MatchExpr(g, n->outputs[0], p, &m)) continue;
      if (!IsClosed(g, m, n)) continue;
      Node* f = g.AddNode("Gelu", {m.values["x"]}, {n->outputs[0]}, kMSDomain, g.UniqueName("Gelu"));
      (void)f;
      RemoveMatched(g, m);
      ++count;
      break;
    }
  }
  return count;
}

// ---------------------------------------------------------- LayerNorm
bool LastAxisOnly(const Graph& g, const Node* rm, const std::string& x) {
  std::vector<int64_t> axes = rm->attr_ints("axes");
  if (axes.empty() && rm->has_input(1)) {
    const at::Tensor* a = g.GetConstant(rm->inputs[1]);
    if (!a) return false;
    at::Tensor ac = a->to(at::kCPU, at::kLong).reshape({-1});
    for (int64_t i = 0; i < ac.numel(); ++i) axes.push_back(ac[i].item<int64_t>());
  }
  if (axes.size() != 1) return false;
  if (axes[0] == -1) return true;
  auto it = const_cast<Graph&>(g).ValueInfos().find(x);
  if (it != const_cast<Graph&>(g).ValueInfos().end() && it->second.type.has_shape)
    return axes[0] == static_cast<int64_t>(it->second.type.dims.size()) - 1;
  for (auto& vi : g.Inputs())
    if (vi.name == x && vi.type.has_shape) return axes[0] == static_cast<int64_t>(vi.type.dims.size()) - 1;
  return false;
}

Pat ReduceMeanOf(Pat arg, const std::string& bind) {
  Pat p = Op("ReduceMean", {std::move(arg)}, bind);
  p.allow_extra_inputs = true;  // opset 18 carries axes as an input
  return p;
}

int LayerNormFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  Pat d = Op("Sub", {V("x"), ReduceMeanOf(V("x"), "rm1")}, "d");
  Pat var = ReduceMeanOf(Op("Pow", {d, C(2.0)}), "rm2");
  Pat norm = Op("Div", {d, Op("Sqrt", {Op("Add", {var, K("eps")})})});
  // the same without "+ eps": a half-precision export whose epsilon rounded to zero loses the Add to no-op elimination
  Pat norm0 = Op("Div", {d, Op("Sqrt", {var})});
  Pat with_affine = Op("Add", {Op("Mul", {norm, K("gamma")}), K("beta")});
  Pat scale_only = Op("Mul", {norm, K("gamma")});
  Pat with_affine0 = Op("Add", {Op("Mul", {norm0, K("gamma")}), K("beta")});
  Pat scale_only0 = Op("Mul", {norm0, K("gamma")});
  for (Node* n : g.Nodes()) {
    if (!n->domain.empty() || (n->op_type != "Add" && n->op_type != "Mul")) continue;
    for (int v4 = 0; v4 < 4; ++v4) {
      const int variant = v4 & 1;
      const bool no_eps = v4 >= 2;
      if ((variant == 0) != (n->op_type == "Add")) continue;
      Match m;
      const Pat& pat = variant == 0 ? (no_eps ? with_affine0 : with_affine) : (no_eps ? scale_only0 : scale_only);
      if (!MatchExpr(g, n->outputs[0], pat, &m, /*through_casts=*/true)) continue;
      if (variant == 1 && g.NumConsumers(n->outputs[0]) == 1) {
        // leave "(..) * gamma" alone when an Add(beta) follows: the Add-rooted match will take it
        Node* cons = g.Consumers(n->outputs[0]).empty() ? nullptr : g.Consumers(n->outputs[0])[0];
        if (cons && cons->op_type == "Add" && cons->domain.empty()) {
          const std::string& other = cons->inputs[0] == n->outputs[0] ? cons->inputs[1] : cons->inputs[0];
          if (g.GetConstant(other)) continue;
        }
      }
      if (!IsClosed(g, m, n)) continue;
      if (!LastAxisOnly(g, m.nodes["rm1"], m.values["x"]) || !LastAxisOnly(g, m.nodes["rm2"], m.values["x"])) continue;
      double eps = 0.0;
      if (!no_eps && !ScalarConst(g, m.values["eps"], &eps)) continue;
      if (!IsConst1D(g, m.values["gamma"])) continue;
      std::vector<std::string> ins = {m.values["x"], m.values["gamma"]};
      if (variant == 0) {
        if (!IsConst1D(g, m.values["beta"])) continue;
        ins.push_back(m.values["beta"]);
      }
      Node* f = g.AddNode("LayerNormalization", ins, {n->outputs[0]}, "", g.UniqueName("LayerNorm"));
      f->set_attr_i("axis", -1);
      f->set_attr_f("epsilon", static_cast<float>(eps));
      f->since_version = 17;
      RemoveMatched(g, m);
      ++count;
      break;
    }
  }
  return count;
}

int SimplifiedLayerNormFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  Pat rms = Op("Sqrt", {Op("Add", {ReduceMeanOf(Op("Pow", {V("x"), C(2.0)}), "rm"), K("eps")})});
  Pat inv1 = Op("Div", {C(1.0), rms});
  Pat inv2 = Op("Reciprocal", {rms});
  std::vector<Pat> pats = {
      Op("Mul", {Op("Div", {V("x"), rms}), K("gamma")}),
      Op("Mul", {Op("Mul", {V("x"), inv1}), K("gamma")}),
      Op("Mul", {Op("Mul", {V("x"), inv2}), K("gamma")}),
  };
  for (Node* n : g.Nodes()) {
    if (!n->domain.empty() || n->op_type != "Mul") continue;
    for (auto& p : pats) {
      Match m;
      if (!MatchExpr(g, n->outputs[0], p, &m, /*through_casts=*/true)) continue;
      if (!IsClosed(g, m, n)) continue;
      if (!LastAxisOnly(g, m.nodes["rm"], m.values["x"])) continue;
      double eps;
      if (!ScalarConst(g, m.values["eps"], &eps) || !IsConst1D(g, m.values["gamma"])) continue;
      // x may have been bound behind a Cast-to-float; normalising the original value is equivalent (fp32 statistics)
      std::string x = m.values["x"];
      Node* f = g.AddNode("SimplifiedLayerNormalization", {x, m.values["gamma"]}, {n->outputs[0]}, "",
                          g.UniqueName("SimplifiedLayerNorm"));
      f->set_attr_i("axis", -1);
      f->set_attr_f("epsilon", static_cast<float>(eps));
      RemoveMatched(g, m);
      ++count;
      break;
    }
  }
  return count;
}

}  // namespace

void AddBasicPasses(std::vector<Pass>& v) {
  v.push_back({"EliminateIdentity", 1, false, EliminateIdentity});
  v.push_back({"NoopElimination", 1, false, EliminateNoop});
  v.push_back({"ConstantFolding", 1, false, ConstantFolding});
  v.push_back({"CommonSubexpressionElimination", 1, false, CommonSubexpressionElimination});
  v.push_back({"ConvBNFusion", 1, false, ConvBatchNormFusion});
  v.push_back({"GeluFusion", 1, false, GeluFusion});
  v.push_back({"LayerNormFusion", 1, false, LayerNormFusion});
  v.push_back({"SimplifiedLayerNormFusion", 1, false, SimplifiedLayerNormFusion});
}

}  // namespace opt
}  // namespace ortb
