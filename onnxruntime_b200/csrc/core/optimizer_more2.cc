// Third group of graph rewrites: the remaining rewrite rules and fusions of the reference's level 1 / level 2 lists
// (onnxruntime/core/optimizer/graph_transformer_utils.cc:133-156, 243-499) that have a kernel to land on here:
//   level 1: EliminateSlice, ExpandElimination, ConvAddFusion, ConvMulFusion, GemmSumFusion
//   level 2: MatMulTransposeFusion, MatMulScaleFusion, ConvActivationFusion, MatMulIntegerToFloatFusion,
//            DynamicQuantizeMatMulFusion, BiasSkipLayerNormFusion, GeluApproximation (opt-in through
//            "optimization.enable_gelu_approximation" = "1")
#include <ATen/ATen.h>

#include <cmath>
#include <limits>

#include "optimizer.h"

namespace ortb {
namespace opt {

namespace {

Node* OnlyUser(const Graph& g, const std::string& v) {
  if (g.IsGraphOutput(v)) return nullptr;
  auto cs = g.Consumers(v);
  return cs.size() == 1 ? cs[0] : nullptr;
}

bool IsOnnx(const Node* n, const char* op) { return n && !n->removed && n->op_type == op && n->domain.empty(); }

std::vector<int64_t> StaticShape(Graph& g, const std::string& v, bool* ok) {
  *ok = false;
  std::vector<int64_t> out;
  const pb::TypeProto* t = nullptr;
  pb::TypeProto tmp;
  for (auto& vi : g.Inputs())
    if (vi.name == v) t = &vi.type;
  if (!t) {
    if (const at::Tensor* c = g.GetInitializer(v)) {
      *ok = true;
      return std::vector<int64_t>(c->sizes().begin(), c->sizes().end());
    }
    auto it = g.ValueInfos().find(v);
    if (it != g.ValueInfos().end()) t = &it->second.type;
  }
  if (!t || t->which != 1 || !t->has_shape) return out;
  for (auto& d : t->dims) {
    if (!d.has_value) return {};
    out.push_back(d.value);
  }
  *ok = true;
  return out;
}

std::vector<int64_t> ConstInts(const Graph& g, const std::string& v, bool* ok) {
  *ok = false;
  const at::Tensor* t = g.GetConstant(v);
  if (!t || !(t->scalar_type() == at::kLong || t->scalar_type() == at::kInt)) return {};
  at::Tensor c = t->to(at::kCPU, at::kLong).reshape({-1});
  *ok = true;
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

// Slice that keeps everything (starts 0, ends at or beyond the dimension / INT_MAX, steps 1)
int EliminateSlice(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* n : g.Nodes()) {
    if (!IsOnnx(n, "Slice") || n->inputs.size() < 3 || g.IsGraphOutput(n->outputs[0])) continue;
    bool ok1, ok2, ok3 = true, ok4 = true, oks;
    std::vector<int64_t> starts = ConstInts(g, n->input(1), &ok1), ends = ConstInts(g, n->input(2), &ok2), axes, steps;
    if (n->has_input(3)) axes = ConstInts(g, n->input(3), &ok3);
    if (n->has_input(4)) steps = ConstInts(g, n->input(4), &ok4);
    if (!ok1 || !ok2 || !ok3 || !ok4 || starts.size() != ends.size()) continue;
    std::vector<int64_t> shape = StaticShape(g, n->input(0), &oks);
    bool full = true;
    for (size_t i = 0; i < starts.size() && full; ++i) {
      if (starts[i] != 0 || (!steps.empty() && steps[i] != 1)) full = false;
      if (ends[i] >= std::numeric_limits<int32_t>::max()) continue;  // "to the end", whatever the dimension is
      int64_t ax = axes.empty() ? static_cast<int64_t>(i) : axes[i];
      if (!oks) {
        full = false;
        break;
      }
      if (ax < 0) ax += static_cast<int64_t>(shape.size());
      if (ax < 0 || ax >= static_cast<int64_t>(shape.size()) || ends[i] < shape[static_cast<size_t>(ax)]) full = false;
    }
    if (!full) continue;
    g.ReplaceAllUses(n->outputs[0], n->inputs[0]);
    g.RemoveNode(n);
    ++count;
  }
  return count;
}

// Expand to a shape that broadcasting leaves unchanged
int ExpandElimination(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* n : g.Nodes()) {
    if (!IsOnnx(n, "Expand") || g.IsGraphOutput(n->outputs[0])) continue;
    bool ok1, ok2;
    std::vector<int64_t> target = ConstInts(g, n->input(1), &ok1), shape = StaticShape(g, n->input(0), &ok2);
    if (!ok1 || !ok2 || target.size() > shape.size()) continue;
    bool same = true;
    for (size_t i = 0; i < target.size(); ++i) {
      const int64_t have = shape[shape.size() - target.size() + i];
      if (target[i] != 1 && target[i] != have) same = false;
    }
    if (!same) continue;
    g.ReplaceAllUses(n->outputs[0], n->inputs[0]);
    g.RemoveNode(n);
    ++count;
  }
  return count;
}

// per-output-channel constant of a convolution result: scalar, [M], [M, 1, 1 ...] or [1, M, 1, 1 ...]
bool PerChannel(const at::Tensor& t, int64_t M, int64_t conv_rank, at::Tensor* flat) {
  if (t.numel() == 1) {
    *flat = t.reshape({1}).expand({M});
    return true;
  }
  if (t.numel() != M) return false;
  const int64_t r = t.dim();
  if (r > conv_rank) return false;
  // the channel axis of the result is 1: the constant's M-sized axis must line up with it after right-alignment
  for (int64_t i = 0; i < r; ++i) {
    const int64_t result_axis = conv_rank - r + i;
    if (t.size(i) != 1 && result_axis != 1) return false;
  }
  *flat = t.reshape({M});
  return true;
}

// Conv followed by Add / Mul with a per-channel constant: folded into the bias / the filter
int ConvAddMulFusion(PassContext& c, bool is_mul) {
  Graph& g = c.g;
  int count = 0;
  for (Node* conv : g.Nodes()) {
    if (!IsOnnx(conv, "Conv")) continue;
    Node* op = OnlyUser(g, conv->outputs[0]);
    if (!IsOnnx(op, is_mul ? "Mul" : "Add")) continue;
    const at::Tensor* w = g.GetConstant(conv->input(1));
    if (!w || !w->is_floating_point()) continue;
    const at::Tensor* b = conv->has_input(2) ? g.GetConstant(conv->input(2)) : nullptr;
    if (conv->has_input(2) && !b) continue;
    const std::string other = op->inputs[0] == conv->outputs[0] ? op->input(1) : op->input(0);
    const at::Tensor* k = g.GetConstant(other);
    if (!k || !k->is_floating_point()) continue;
    const int64_t M = w->size(0);
    at::Tensor flat;
    if (!PerChannel(*k, M, w->dim(), &flat)) continue;
    flat = flat.to(w->scalar_type()).contiguous();
    const std::string base = conv->name.empty() ? conv->outputs[0] : conv->name;
    if (is_mul) {
      std::vector<int64_t> shape(static_cast<size_t>(w->dim()), 1);
      shape[0] = M;
      const std::string wn = g.UniqueName(base + "_scaled_weight");
      g.AddInitializer(wn, (*w * flat.reshape(shape)).contiguous());
      conv->inputs[1] = wn;
      if (b) {
        const std::string bn = g.UniqueName(base + "_scaled_bias");
        g.AddInitializer(bn, (*b * flat).contiguous());
        conv->inputs[2] = bn;
      }
    } else {
      const std::string bn = g.UniqueName(base + "_fused_bias");
      g.AddInitializer(bn, b ? (*b + flat).contiguous() : flat.clone());
      while (conv->inputs.size() < 3) conv->inputs.push_back("");
      conv->inputs[2] = bn;
    }
    const std::string out = op->outputs[0];
    g.RemoveNode(op);
    conv->outputs[0] = out;
    g.Invalidate();
    ++count;
  }
  return count;
}

// Sum(Gemm(A, B), C) with a Gemm that has no C: the addend becomes C (beta = 1)
int GemmSumFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* gemm : g.Nodes()) {
    if (!IsOnnx(gemm, "Gemm") || gemm->has_input(2)) continue;
    Node* sum = OnlyUser(g, gemm->outputs[0]);
    if (!IsOnnx(sum, "Sum") || sum->inputs.size() != 2) continue;
    const std::string other = sum->inputs[0] == gemm->outputs[0] ? sum->inputs[1] : sum->inputs[0];
    if (other == gemm->outputs[0]) continue;
    // C must broadcast to the product unidirectionally: require a known shape of rank <= 2 that fits [M, N]
    bool ok_c, ok_y;
    std::vector<int64_t> cs = StaticShape(g, other, &ok_c), ys = StaticShape(g, gemm->outputs[0], &ok_y);
    if (!ok_c || !ok_y || cs.size() > 2 || ys.size() != 2) continue;
    bool fits = true;
    for (size_t i = 0; i < cs.size(); ++i) {
      const int64_t want = ys[2 - cs.size() + i];
      if (cs[i] != 1 && cs[i] != want) fits = false;
    }
    if (!fits) continue;
    while (gemm->inputs.size() < 3) gemm->inputs.push_back("");
    gemm->inputs[2] = other;
    gemm->set_attr_f("beta", 1.0f);
    const std::string out = sum->outputs[0];
    g.RemoveNode(sum);
    gemm->outputs[0] = out;
    g.Invalidate();
    ++count;
  }
  return count;
}

// Transpose of the last two axes in front of MatMul -> com.microsoft FusedMatMul with transA / transB
int MatMulTransposeFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* mm : g.Nodes()) {
    const bool fused = mm->op_type == "FusedMatMul" && mm->domain == kMSDomain && !mm->removed;
    if (!IsOnnx(mm, "MatMul") && !fused) continue;
    for (int side = 0; side < 2; ++side) {
      Node* tr = g.Producer(mm->input(static_cast<size_t>(side)));
      if (!IsOnnx(tr, "Transpose") || g.IsGraphOutput(tr->outputs[0])) continue;
      std::vector<int64_t> perm = tr->attr_ints("perm");
      const int64_t r = static_cast<int64_t>(perm.size());
      if (r < 2) continue;
      bool last_two = perm[static_cast<size_t>(r - 1)] == r - 2 && perm[static_cast<size_t>(r - 2)] == r - 1;
      for (int64_t i = 0; i < r - 2; ++i) last_two = last_two && perm[static_cast<size_t>(i)] == i;
      if (!last_two) continue;
      if (mm->op_type == "MatMul") {
        mm->op_type = "FusedMatMul";
        mm->domain = kMSDomain;
        mm->since_version = 1;
      }
      const char* flag = side == 0 ? "transA" : "transB";
      mm->set_attr_i(flag, mm->attr_i(flag, 0) ? 0 : 1);
      mm->inputs[static_cast<size_t>(side)] = tr->inputs[0];
      g.Invalidate();
      if (g.Consumers(tr->outputs[0]).empty()) g.RemoveNode(tr);
      ++count;
    }
  }
  return count;
}

// scalar Mul / Div on an operand or on the result of a MatMul -> FusedMatMul alpha
int MatMulScaleFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  auto scalar_of = [&](Node* n, std::string* data, double* k) {
    if (!n || n->removed || !n->domain.empty() || (n->op_type != "Mul" && n->op_type != "Div")) return false;
    double v;
    if (ScalarConst(g, n->input(1), &v)) {
      *data = n->input(0);
    } else if (n->op_type == "Mul" && ScalarConst(g, n->input(0), &v)) {
      *data = n->input(1);
    } else {
      return false;
    }
    if (n->op_type == "Div") {
      if (v == 0) return false;
      v = 1.0 / v;
    }
    *k = v;
    return true;
  };
  for (Node* mm : g.Nodes()) {
    const bool fused = mm->op_type == "FusedMatMul" && mm->domain == kMSDomain && !mm->removed;
    if (!IsOnnx(mm, "MatMul") && !fused) continue;
    double alpha = mm->attr_f("alpha", 1.0f);
    bool changed = false;
    for (int side = 0; side < 2; ++side) {
      Node* s = g.Producer(mm->input(static_cast<size_t>(side)));
      std::string data;
      double k;
      if (!s || g.IsGraphOutput(s->outputs[0]) || OnlyUser(g, s->outputs[0]) != mm || !scalar_of(s, &data, &k)) continue;
      mm->inputs[static_cast<size_t>(side)] = data;
      g.Invalidate();
      g.RemoveNode(s);
      alpha *= k;
      changed = true;
    }
    Node* after = OnlyUser(g, mm->outputs[0]);
    std::string data;
    double k;
    if (after && scalar_of(after, &data, &k) && data == mm->outputs[0]) {
      const std::string out = after->outputs[0];
      g.RemoveNode(after);
      mm->outputs[0] = out;
      g.Invalidate();
      alpha *= k;
      changed = true;
    }
    if (!changed) continue;
    if (mm->op_type == "MatMul") {
      mm->op_type = "FusedMatMul";
      mm->domain = kMSDomain;
      mm->since_version = 1;
    }
    mm->set_attr_f("alpha", static_cast<float>(alpha));
    ++count;
  }
  return count;
}

// Conv + Relu / Sigmoid / Tanh / LeakyRelu / HardSigmoid / Clip(constant bounds) -> com.microsoft FusedConv
int ConvActivationFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* conv : g.Nodes()) {
    if (!IsOnnx(conv, "Conv")) continue;
    Node* act = OnlyUser(g, conv->outputs[0]);
    if (!act || act->removed || !act->domain.empty() || act->inputs[0] != conv->outputs[0]) continue;
    std::vector<float> params;
    const std::string& op = act->op_type;
    if (op == "Relu" || op == "Sigmoid" || op == "Tanh") {
    } else if (op == "LeakyRelu") {
      params = {act->attr_f("alpha", 0.01f)};
    } else if (op == "HardSigmoid") {
      params = {act->attr_f("alpha", 0.2f), act->attr_f("beta", 0.5f)};
    } else if (op == "Clip") {
      double lo = -std::numeric_limits<float>::infinity(), hi = std::numeric_limits<float>::infinity();
      if (act->has_attr("min") || act->has_attr("max")) {
        lo = act->attr_f("min", -std::numeric_limits<float>::infinity());
        hi = act->attr_f("max", std::numeric_limits<float>::infinity());
      } else {
        if (act->has_input(1) && !ScalarConst(g, act->input(1), &lo)) continue;
        if (act->has_input(2) && !ScalarConst(g, act->input(2), &hi)) continue;
      }
      params = {static_cast<float>(lo), static_cast<float>(hi)};
    } else {
      continue;
    }
    conv->op_type = "FusedConv";
    conv->domain = kMSDomain;
    conv->since_version = 1;
    conv->set_attr_s("activation", op);
    if (!params.empty()) conv->set_attr_floats("activation_params", params);
    const std::string out = act->outputs[0];
    g.RemoveNode(act);
    conv->outputs[0] = out;
    g.Invalidate();
    ++count;
  }
  return count;
}

// MatMulInteger -> Cast(float) -> Mul(scale) [-> Add(bias)]  ==>  com.microsoft MatMulIntegerToFloat
int MatMulIntegerToFloatFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* mi : g.Nodes()) {
    if (!IsOnnx(mi, "MatMulInteger")) continue;
    Node* cast = OnlyUser(g, mi->outputs[0]);
    if (!IsOnnx(cast, "Cast") || cast->attr_i("to", 0) != 1) continue;
    Node* mul = OnlyUser(g, cast->outputs[0]);
    if (!IsOnnx(mul, "Mul")) continue;
    const std::string scale = mul->inputs[0] == cast->outputs[0] ? mul->input(1) : mul->input(0);
    // the combined scale is usually Mul(a_scale, b_scale): pass its factors when visible, else scale with 1
    std::string a_scale, b_scale;
    Node* sp = g.Producer(scale);
    if (IsOnnx(sp, "Mul") && OnlyUser(g, sp->outputs[0]) == mul) {
      a_scale = sp->input(0);
      b_scale = sp->input(1);
    } else {
      a_scale = scale;
      b_scale = g.UniqueName("unit_scale");
      g.AddInitializer(b_scale, at::ones({1}, at::kFloat));
    }
    std::vector<std::string> in = {mi->input(0), mi->input(1), a_scale, b_scale, mi->input(2), mi->input(3)};
    std::string out = mul->outputs[0];
    Node* add = OnlyUser(g, mul->outputs[0]);
    Node* bias_node = nullptr;
    if (IsOnnx(add, "Add")) {
      const std::string other = add->inputs[0] == mul->outputs[0] ? add->input(1) : add->input(0);
      const at::Tensor* b = g.GetConstant(other);
      if (b && b->dim() == 1) {
        in.push_back(other);
        out = add->outputs[0];
        bias_node = add;
      }
    }
    while (!in.empty() && in.back().empty()) in.pop_back();
    if (bias_node) g.RemoveNode(bias_node);
    g.RemoveNode(mul);
    g.RemoveNode(cast);
    if (sp && IsOnnx(sp, "Mul") && a_scale == sp->input(0) && g.Consumers(sp->outputs[0]).empty()) g.RemoveNode(sp);
    const std::string name = mi->name;
    g.RemoveNode(mi);
    g.AddNode("MatMulIntegerToFloat", in, {out}, kMSDomain, name.empty() ? g.UniqueName("MatMulIntegerToFloat") : name + "_float");
    ++count;
  }
  return count;
}

// DynamicQuantizeLinear(A) feeding MatMulIntegerToFloat  ==>  com.microsoft DynamicQuantizeMatMul(A, B, b_scale, b_zp, bias)
int DynamicQuantizeMatMulFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* m : g.Nodes()) {
    if (m->removed || m->op_type != "MatMulIntegerToFloat" || m->domain != kMSDomain) continue;
    Node* dq = g.Producer(m->input(0));
    if (!IsOnnx(dq, "DynamicQuantizeLinear") || dq->outputs.size() < 3) continue;
    if (m->input(2) != dq->outputs[1] || m->input(4) != dq->outputs[2]) continue;
    bool sole = true;
    for (auto& o : dq->outputs)
      for (Node* u : g.Consumers(o)) sole = sole && u == m;
    if (!sole || !g.GetConstant(m->input(1))) continue;
    std::vector<std::string> in = {dq->input(0), m->input(1), m->input(3), m->input(5), m->input(6)};
    while (!in.empty() && in.back().empty()) in.pop_back();
    const std::string out = m->outputs[0], name = m->name;
    g.RemoveNode(m);
    g.RemoveNode(dq);
    g.AddNode("DynamicQuantizeMatMul", in, {out}, kMSDomain, name.empty() ? g.UniqueName("DynamicQuantizeMatMul") : name + "_dynamic");
    ++count;
  }
  return count;
}

// Add(x, bias[hidden]) feeding the input of SkipLayerNormalization: the bias becomes the operator's fifth input
int BiasSkipLayerNormFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* sln : g.Nodes()) {
    if (sln->removed || sln->domain != kMSDomain || (sln->op_type != "SkipLayerNormalization" && sln->op_type != "SkipSimplifiedLayerNormalization")) continue;
    const size_t bias_index = sln->op_type == "SkipLayerNormalization" ? 4 : 3;
    if (sln->has_input(bias_index)) continue;
    for (int side = 0; side < 2; ++side) {
      Node* add = g.Producer(sln->input(static_cast<size_t>(side)));
      if (!IsOnnx(add, "Add") || OnlyUser(g, add->outputs[0]) != sln) continue;
      int bi = -1;
      for (int i = 0; i < 2; ++i) {
        const at::Tensor* b = g.GetConstant(add->input(static_cast<size_t>(i)));
        if (b && b->dim() == 1) bi = i;
      }
      if (bi < 0) continue;
      while (sln->inputs.size() <= bias_index) sln->inputs.push_back("");
      sln->inputs[bias_index] = add->input(static_cast<size_t>(bi));
      sln->inputs[static_cast<size_t>(side)] = add->input(static_cast<size_t>(1 - bi));
      g.Invalidate();
      g.RemoveNode(add);
      ++count;
      break;
    }
  }
  return count;
}

// Gelu / BiasGelu -> FastGelu (tanh form); changes results slightly, hence opt-in
int GeluApproximation(PassContext& c) {
  if (c.config.Get("optimization.enable_gelu_approximation", "0") != "1") return 0;
  Graph& g = c.g;
  int count = 0;
  for (Node* n : g.Nodes()) {
    if (n->removed) continue;
    const bool ms_gelu = n->domain == kMSDomain && (n->op_type == "Gelu" || n->op_type == "BiasGelu");
    const bool onnx_gelu = n->domain.empty() && n->op_type == "Gelu" && n->attr_s("approximate", "none") == "none";
    if (!ms_gelu && !onnx_gelu) continue;
    n->op_type = "FastGelu";
    n->domain = kMSDomain;
    n->since_version = 1;
    n->attrs.erase("approximate");
    ++count;
  }
  return count;
}

}  // namespace

void AddMorePasses2(std::vector<Pass>& v) {
  v.push_back({"EliminateSlice", 1, false, EliminateSlice});
  v.push_back({"ExpandElimination", 1, false, ExpandElimination});
  v.push_back({"ConvAddFusion", 1, false, [](PassContext& c) { return ConvAddMulFusion(c, false); }});
  v.push_back({"ConvMulFusion", 1, false, [](PassContext& c) { return ConvAddMulFusion(c, true); }});
  v.push_back({"GemmSumFusion", 1, false, GemmSumFusion});
  v.push_back({"MatMulScaleFusion", 2, false, MatMulScaleFusion});
  v.push_back({"MatMulTransposeFusion", 2, false, MatMulTransposeFusion});
  v.push_back({"ConvActivationFusion", 2, false, ConvActivationFusion});
  v.push_back({"MatMulIntegerToFloatFusion", 2, false, MatMulIntegerToFloatFusion});
  v.push_back({"DynamicQuantizeMatMulFusion", 2, false, DynamicQuantizeMatMulFusion});
  v.push_back({"BiasSkipLayerNormFusion", 2, false, BiasSkipLayerNormFusion});
  v.push_back({"GeluApproximation", 2, false, GeluApproximation});
}

}  // namespace opt
}  // namespace ortb
