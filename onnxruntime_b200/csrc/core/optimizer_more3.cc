// Fourth group of graph rewrites, the rest of the reference's level 1 / level 2 lists that have something to land on
// here (onnxruntime/core/optimizer/: cast_chain_elimination.cc, pre_shape_node_elimination.cc, pad_fusion.cc,
// matmul_bn_fusion.cc, label_encoder_fusion.cc, gemm_activation_fusion.cc, ensure_unique_dq_for_node_unit.cc,
// qdq_transformer/qdq_final_cleanup.cc):
//   level 1: CastChainElimination, PreShapeNodeElimination, PadFusion, MatMulBNFusion, LabelEncoderFusion,
//            EnsureUniqueDQForNodeUnit
//   level 2: GemmActivationFusion, QDQFinalCleanup
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

int32_t ElemTypeOf(Graph& g, const std::string& v) {
  for (auto& vi : g.Inputs())
    if (vi.name == v) return vi.type.which == 1 ? vi.type.elem_type : 0;
  if (const at::Tensor* c = g.GetInitializer(v)) return g.IsStringValue(v) ? static_cast<int32_t>(pb::STRING) : ToOnnxType(c->scalar_type());
  auto it = g.ValueInfos().find(v);
  return it != g.ValueInfos().end() && it->second.type.which == 1 ? it->second.type.elem_type : 0;
}

// rank of a type inside its class (floats / signed ints), 0 when it is in neither
int FloatRank(int32_t t) { return t == pb::FLOAT16 || t == pb::BFLOAT16 ? 1 : t == pb::FLOAT ? 2 : t == pb::DOUBLE ? 3 : 0; }
int IntRank(int32_t t) { return t == pb::INT8 ? 1 : t == pb::INT16 ? 2 : t == pb::INT32 ? 3 : t == pb::INT64 ? 4 : 0; }

// Cast(Cast(x, A), B) where A holds every value of x's type: one Cast(x, B)
int CastChainElimination(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* outer : g.Nodes()) {
    if (!IsOnnx(outer, "Cast")) continue;
    Node* inner = g.Producer(outer->inputs[0]);
    if (!IsOnnx(inner, "Cast") || g.NumConsumers(inner->outputs[0]) != 1 || g.IsGraphOutput(inner->outputs[0])) continue;
    const int32_t src = ElemTypeOf(g, inner->inputs[0]), mid = static_cast<int32_t>(inner->attr_i("to", 0));
    if (src == 0) continue;
    const bool widening = (FloatRank(src) && FloatRank(mid) > FloatRank(src) && !(src == pb::FLOAT16 && mid == pb::BFLOAT16)) ||
                          (FloatRank(src) && FloatRank(mid) == FloatRank(src) && src == mid) ||
                          (IntRank(src) && IntRank(mid) >= IntRank(src)) || (src == pb::BOOL && (IntRank(mid) || FloatRank(mid)));
    if (!widening) continue;
    outer->inputs[0] = inner->inputs[0];
    g.RemoveNode(inner);
    g.Invalidate();
    ++count;
  }
  return count;
}

// Shape(Cast(x)) reads the shape of x
int PreShapeNodeElimination(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* shape : g.Nodes()) {
    if (!IsOnnx(shape, "Shape")) continue;
    Node* cast = g.Producer(shape->inputs[0]);
    if (!IsOnnx(cast, "Cast")) continue;
    const bool sole = g.NumConsumers(cast->outputs[0]) == 1 && !g.IsGraphOutput(cast->outputs[0]);
    shape->inputs[0] = cast->inputs[0];
    if (sole) g.RemoveNode(cast);
    g.Invalidate();
    ++count;
  }
  return count;
}

std::vector<int64_t> ConstInts(const Graph& g, const std::string& v, bool* ok) {
  *ok = false;
  const at::Tensor* t = g.GetConstant(v);
  if (!t || !(t->scalar_type() == at::kLong || t->scalar_type() == at::kInt)) return {};
  at::Tensor k = t->to(at::kCPU, at::kLong).reshape({-1});
  *ok = true;
  return std::vector<int64_t>(k.data_ptr<int64_t>(), k.data_ptr<int64_t>() + k.numel());
}

// Pad(constant 0, spatial dims only, no negative pads) -> Conv / AveragePool(count_include_pad): into the `pads` attribute
int PadFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* pad : g.Nodes()) {
    if (!IsOnnx(pad, "Pad") || pad->attr_s("mode", "constant") != "constant") continue;
    Node* user = OnlyUser(g, pad->outputs[0]);
    if (!user || user->inputs[0] != pad->outputs[0]) continue;
    const bool conv = IsOnnx(user, "Conv"), avg = IsOnnx(user, "AveragePool") && user->attr_i("count_include_pad", 0) == 1;
    if (!conv && !avg) continue;
    if (user->attr_s("auto_pad", "NOTSET") != "NOTSET") continue;
    std::vector<int64_t> pads;
    bool ok = true;
    if (pad->has_attr("pads")) pads = pad->attr_ints("pads");
    else if (pad->has_input(1)) pads = ConstInts(g, pad->input(1), &ok);
    else ok = false;
    if (!ok || pads.size() < 6 || pads.size() % 2 != 0 || pad->has_input(3)) continue;  // input 3 = axes: not handled
    double value = pad->has_attr("value") ? pad->attr_f("value", 0.f) : 0.0;
    if (pad->has_input(2) && !ScalarConst(g, pad->input(2), &value)) continue;
    if (value != 0.0) continue;
    const size_t rank = pads.size() / 2, spatial = rank - 2;
    bool fits = pads[0] == 0 && pads[1] == 0 && pads[rank] == 0 && pads[rank + 1] == 0;
    for (int64_t p : pads) fits = fits && p >= 0;
    if (!fits) continue;
    std::vector<int64_t> child = user->attr_ints("pads");
    if (child.empty()) child.assign(2 * spatial, 0);
    if (child.size() != 2 * spatial) continue;
    for (size_t d = 0; d < spatial; ++d) {
      child[d] += pads[2 + d];
      child[spatial + d] += pads[rank + 2 + d];
    }
    user->set_attr_ints("pads", child);
    user->inputs[0] = pad->inputs[0];
    g.RemoveNode(pad);
    g.Invalidate();
    ++count;
  }
  return count;
}

// MatMul(x, W) -> BatchNormalization (inference form, constants, channel = last axis of a rank-2 product) -> Gemm
int MatMulBNFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* mm : g.Nodes()) {
    if (!IsOnnx(mm, "MatMul")) continue;
    const at::Tensor* w = g.GetConstant(mm->inputs[1]);
    if (!w || w->dim() != 2 || !w->is_floating_point()) continue;
    Node* bn = OnlyUser(g, mm->outputs[0]);
    if (!IsOnnx(bn, "BatchNormalization") || bn->inputs.size() < 5 || bn->inputs[0] != mm->outputs[0]) continue;
    if (bn->attr_i("training_mode", 0) != 0 || (bn->outputs.size() > 1 && !bn->outputs[1].empty())) continue;
    // the product must be [N, C] for BatchNormalization's channel axis (1) to be the columns of W
    auto vi = g.ValueInfos().find(mm->inputs[0]);
    int64_t in_rank = -1;
    for (auto& in : g.Inputs())
      if (in.name == mm->inputs[0] && in.type.which == 1 && in.type.has_shape) in_rank = static_cast<int64_t>(in.type.dims.size());
    if (in_rank < 0 && vi != g.ValueInfos().end() && vi->second.type.which == 1 && vi->second.type.has_shape)
      in_rank = static_cast<int64_t>(vi->second.type.dims.size());
    if (in_rank != 2) continue;
    const at::Tensor *scale = g.GetConstant(bn->inputs[1]), *beta = g.GetConstant(bn->inputs[2]), *mean = g.GetConstant(bn->inputs[3]),
                     *var = g.GetConstant(bn->inputs[4]);
    if (!scale || !beta || !mean || !var || scale->numel() != w->size(1)) continue;
    const double eps = bn->attr_f("epsilon", 1e-5f);
    at::Tensor k = scale->to(at::kFloat) / at::sqrt(var->to(at::kFloat) + eps);
    const std::string wn = g.UniqueName(mm->inputs[1] + "_bn"), bname = g.UniqueName(mm->inputs[1] + "_bn_bias");
    g.AddInitializer(wn, (w->to(at::kFloat) * k.reshape({1, -1})).to(w->scalar_type()).contiguous());
    g.AddInitializer(bname, (beta->to(at::kFloat) - mean->to(at::kFloat) * k).to(w->scalar_type()).contiguous());
    g.AddNode("Gemm", {mm->inputs[0], wn, bname}, {bn->outputs[0]}, "", g.UniqueName("Gemm_bn"));
    g.RemoveNode(bn);
    g.RemoveNode(mm);
    ++count;
  }
  return count;
}

// LabelEncoder -> LabelEncoder: one table.  Values of the first must be of the second's key type.
int LabelEncoderFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  auto kind_of = [](const Node& n, const char* prefix) -> int {  // 1 int64, 2 float, 3 string, 0 none / tensor form
    const std::string p(prefix);
    if (n.has_attr(p + "_int64s")) return 1;
    if (n.has_attr(p + "_floats")) return 2;
    if (n.has_attr(p + "_strings")) return 3;
    return 0;
  };
  for (Node* second : g.Nodes()) {
    if (second->removed || second->op_type != "LabelEncoder" || second->domain != "ai.onnx.ml") continue;
    Node* first = g.Producer(second->inputs[0]);
    if (!first || first->removed || first->op_type != "LabelEncoder" || first->domain != "ai.onnx.ml") continue;
    if (g.NumConsumers(first->outputs[0]) != 1 || g.IsGraphOutput(first->outputs[0])) continue;
    const int k1 = kind_of(*first, "keys"), v1 = kind_of(*first, "values"), k2 = kind_of(*second, "keys"), v2 = kind_of(*second, "values");
    if (!k1 || !v1 || !k2 || !v2 || v1 != k2) continue;
    // the second table, keyed by the textual form of its key (exact for int64 and strings; floats compare by value)
    auto keys_as_text = [](const Node& n, const char* prefix, int kind) {
      std::vector<std::string> out;
      const std::string p(prefix);
      if (kind == 1) for (int64_t v : n.attr_ints(p + "_int64s")) out.push_back(std::to_string(v));
      if (kind == 2) for (float v : n.attr_floats(p + "_floats")) out.push_back(std::to_string(static_cast<double>(v)));
      if (kind == 3) out = n.attr_strings(p + "_strings");
      return out;
    };
    const std::vector<std::string> mid_vals = keys_as_text(*first, "values", v1), second_keys = keys_as_text(*second, "keys", k2);
    std::map<std::string, size_t> pos;
    for (size_t i = 0; i < second_keys.size(); ++i) pos.emplace(second_keys[i], i);
    std::string first_default = v1 == 1 ? std::to_string(first->attr_i("default_int64", -1))
                                : v1 == 2 ? std::to_string(static_cast<double>(first->attr_f("default_float", -0.f)))
                                          : first->attr_s("default_string", "_Unused");
    // composed values, as indices into the second's value list (-1 = second's default)
    std::vector<int64_t> pick;
    for (auto& m : mid_vals) pick.push_back(pos.count(m) ? static_cast<int64_t>(pos[m]) : -1);
    const int64_t default_pick = pos.count(first_default) ? static_cast<int64_t>(pos[first_default]) : -1;
    Node* fused = g.AddNode("LabelEncoder", {first->inputs[0]}, {second->outputs[0]}, "ai.onnx.ml", g.UniqueName("LabelEncoder_fused"));
    fused->since_version = second->since_version;
    if (k1 == 1) fused->set_attr_ints("keys_int64s", first->attr_ints("keys_int64s"));
    if (k1 == 2) fused->set_attr_floats("keys_floats", first->attr_floats("keys_floats"));
    if (k1 == 3) fused->set_attr_strings("keys_strings", first->attr_strings("keys_strings"));
    if (v2 == 1) {
      const std::vector<int64_t> vals = second->attr_ints("values_int64s");
      const int64_t d = second->attr_i("default_int64", -1);
      std::vector<int64_t> out;
      for (int64_t p : pick) out.push_back(p < 0 ? d : vals[static_cast<size_t>(p)]);
      fused->set_attr_ints("values_int64s", out);
      fused->set_attr_i("default_int64", default_pick < 0 ? d : vals[static_cast<size_t>(default_pick)]);
    } else if (v2 == 2) {
      const std::vector<float> vals = second->attr_floats("values_floats");
      const float d = second->attr_f("default_float", -0.f);
      std::vector<float> out;
      for (int64_t p : pick) out.push_back(p < 0 ? d : vals[static_cast<size_t>(p)]);
      fused->set_attr_floats("values_floats", out);
      fused->set_attr_f("default_float", default_pick < 0 ? d : vals[static_cast<size_t>(default_pick)]);
    } else {
      const std::vector<std::string> vals = second->attr_strings("values_strings");
      const std::string d = second->attr_s("default_string", "_Unused");
      std::vector<std::string> out;
      for (int64_t p : pick) out.push_back(p < 0 ? d : vals[static_cast<size_t>(p)]);
      fused->set_attr_strings("values_strings", out);
      fused->set_attr_s("default_string", default_pick < 0 ? d : vals[static_cast<size_t>(default_pick)]);
    }
    g.RemoveNode(second);
    g.RemoveNode(first);
    ++count;
  }
  return count;
}

// A DequantizeLinear of a constant that feeds several nodes gets one copy per consumer, so that every quantised
// node unit (DQ -> op -> Q) owns its DQ and the QDQ fusions can take it.
int EnsureUniqueDQForNodeUnit(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* dq : g.Nodes()) {
    if (!IsOnnx(dq, "DequantizeLinear") || !g.GetConstant(dq->inputs[0]) || g.IsGraphOutput(dq->outputs[0])) continue;
    std::vector<Node*> users = g.Consumers(dq->outputs[0]);
    if (users.size() < 2) continue;
    for (size_t u = 1; u < users.size(); ++u) {
      const std::string out = g.UniqueName(dq->outputs[0] + "_dup");
      Node* copy = g.AddNode("DequantizeLinear", dq->inputs, {out}, "", g.UniqueName(dq->name + "_dup"));
      copy->attrs = dq->attrs;
      copy->since_version = dq->since_version;
      for (auto& in : users[u]->inputs)
        if (in == dq->outputs[0]) in = out;
      ++count;
    }
    g.Invalidate();
  }
  return count;
}

// Gemm -> activation  ==>  com.microsoft FusedGemm
int GemmActivationFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  if (c.gpu) return 0;  // the GPU lowering has its own epilogue fusion
  for (Node* gemm : g.Nodes()) {
    if (!IsOnnx(gemm, "Gemm")) continue;
    Node* act = OnlyUser(g, gemm->outputs[0]);
    if (!act || act->removed || !act->domain.empty() || act->inputs.empty() || act->inputs[0] != gemm->outputs[0]) continue;
    const std::string& op = act->op_type;
    if (op == "LeakyRelu") {
      gemm->set_attr_f("activation_alpha", act->attr_f("alpha", 0.01f));
    } else if (op == "HardSigmoid") {
      gemm->set_attr_f("activation_alpha", act->attr_f("alpha", 0.2f));
      gemm->set_attr_f("activation_beta", act->attr_f("beta", 0.5f));
    } else if (op == "Elu") {
      gemm->set_attr_f("activation_alpha", act->attr_f("alpha", 1.0f));
    } else if (op == "ThresholdedRelu") {
      gemm->set_attr_f("activation_alpha", act->attr_f("alpha", 1.0f));
    } else if (op == "Selu") {
      gemm->set_attr_f("activation_alpha", act->attr_f("alpha", 1.67326319f));
      gemm->set_attr_f("activation_gamma", act->attr_f("gamma", 1.05070102f));
    } else if (!(op == "Relu" || op == "Sigmoid" || op == "Tanh" || op == "Softplus" || op == "Softsign")) {
      continue;
    }
    gemm->op_type = "FusedGemm";
    gemm->domain = kMSDomain;
    gemm->since_version = 1;
    gemm->set_attr_s("activation", op);
    const std::string out = act->outputs[0];
    g.RemoveNode(act);
    gemm->outputs[0] = out;
    g.Invalidate();
    ++count;
  }
  return count;
}

// QuantizeLinear -> DequantizeLinear with the same constant scale / zero point that no fusion took, when the pair sits
// at the very end or the very beginning of the graph, is dropped if "session.enable_quant_qdq_cleanup" = "1" (the
// rounding it stands for is lost, so it is opt-in, as in the reference).  DQ -> Q pairs are exact and always go.
int QDQFinalCleanup(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  const bool lossy_ok = c.config.Get("session.enable_quant_qdq_cleanup", "0") == "1";
  auto same_params = [&](const Node* a, const Node* b) {
    for (size_t i = 1; i < 3; ++i) {
      if (a->has_input(i) != b->has_input(i)) return false;
      if (!a->has_input(i)) continue;
      if (a->inputs[i] == b->inputs[i]) continue;
      const at::Tensor *x = g.GetConstant(a->inputs[i]), *y = g.GetConstant(b->inputs[i]);
      if (!x || !y || x->scalar_type() != y->scalar_type() || x->sizes() != y->sizes() || !at::equal(*x, *y)) return false;
    }
    return a->attr_i("axis", 1) == b->attr_i("axis", 1);
  };
  for (Node* second : g.Nodes()) {
    const bool q_dq = IsOnnx(second, "DequantizeLinear"), dq_q = IsOnnx(second, "QuantizeLinear");
    if (!q_dq && !dq_q) continue;
    Node* first = g.Producer(second->inputs[0]);
    if (!IsOnnx(first, q_dq ? "QuantizeLinear" : "DequantizeLinear")) continue;
    if (g.NumConsumers(first->outputs[0]) != 1 || g.IsGraphOutput(first->outputs[0]) || !same_params(first, second)) continue;
    if (q_dq && !lossy_ok) continue;
    if (g.IsGraphOutput(second->outputs[0]) && (g.IsGraphInput(first->inputs[0]) || g.IsInitializer(first->inputs[0]))) continue;
    if (g.IsGraphOutput(second->outputs[0])) {
      Node* producer = g.Producer(first->inputs[0]);
      if (!producer || g.NumConsumers(first->inputs[0]) != 1) continue;
      for (auto& o : producer->outputs)
        if (o == first->inputs[0]) o = second->outputs[0];
    } else {
      g.ReplaceAllUses(second->outputs[0], first->inputs[0]);
    }
    g.RemoveNode(second);
    g.RemoveNode(first);
    g.Invalidate();
    ++count;
  }
  return count;
}

// DequantizeLinear(4-bit constant W [K, N], block-wise along K: axis 0, block_size 16 / 32 / 64 ...) -> MatMul(A, .)
//   ==>  com.microsoft MatMulNBits(A, B [N, K / block, block / 2], scales, zero points)
// (reference: qdq_transformer/selectors_actions/qdq_actions.cc DQMatMulToMatMulNBitsAction).  On with
// "session.enable_dq_matmulnbits_fusion" = "1"; when the key is absent, on for GPU sessions (which have a 4-bit GEMM).
int DQMatMulNBitsFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  const std::string key = c.config.Get("session.enable_dq_matmulnbits_fusion", "");
  if (!(key == "1" || (key.empty() && c.gpu))) return 0;
  const int64_t accuracy = std::stoll(c.config.Get("session.qdq_matmulnbits_accuracy_level", "4"));
  for (Node* mm : g.Nodes()) {
    if (!IsOnnx(mm, "MatMul")) continue;
    Node* dq = g.Producer(mm->inputs[1]);
    if (!IsOnnx(dq, "DequantizeLinear") || g.NumConsumers(dq->outputs[0]) != 1 || g.IsGraphOutput(dq->outputs[0])) continue;
    const int32_t wt = g.FourBitTypeOf(dq->inputs[0]);
    const at::Tensor *w = g.GetConstant(dq->inputs[0]), *scale = g.GetConstant(dq->inputs[1]);
    const at::Tensor* zp = dq->has_input(2) ? g.GetConstant(dq->inputs[2]) : nullptr;
    if (!wt || !w || !scale || w->dim() != 2 || (dq->has_input(2) && (!zp || g.FourBitTypeOf(dq->inputs[2]) != wt))) continue;
    const int64_t K = w->size(0), N = w->size(1), bs = dq->attr_i("block_size", 0);
    int64_t axis = dq->attr_i("axis", 1);
    if (axis < 0) axis += 2;
    if (axis != 0 || bs < 16 || (bs & (bs - 1)) != 0) continue;
    const int64_t nb = (K + bs - 1) / bs;
    if (scale->dim() != 2 || scale->size(0) != nb || scale->size(1) != N || !(scale->scalar_type() == at::kFloat || scale->scalar_type() == at::kHalf)) continue;
    if (zp && (zp->dim() != 2 || zp->size(0) != nb || zp->size(1) != N)) continue;
    const int64_t shift = wt == pb::INT4 ? 8 : 0;  // signed codes become unsigned: q + 8 with zero point + 8
    // B: per output feature, per block, block / 2 bytes, the earlier K index in the low nibble
    at::Tensor wt_nk = (w->to(at::kInt) + shift).t().contiguous();
    if (nb * bs != K) wt_nk = at::constant_pad_nd(wt_nk, {0, nb * bs - K}, 0);
    at::Tensor pairs = wt_nk.reshape({N, nb, bs / 2, 2});
    at::Tensor B = at::bitwise_or(pairs.select(3, 0), at::bitwise_left_shift(pairs.select(3, 1), 4)).to(at::kByte).contiguous();
    at::Tensor scales = scale->t().contiguous().reshape({N * nb});
    const std::string bn = g.UniqueName(dq->inputs[0] + "_nbits"), sn = g.UniqueName(dq->inputs[1] + "_nbits");
    g.AddInitializer(bn, B);
    g.AddInitializer(sn, scales);
    std::vector<std::string> inputs = {mm->inputs[0], bn, sn};
    if (zp || !shift) {  // signed weights without zero points need none: the operator's default zero point is 8
      at::Tensor z = zp ? (zp->to(at::kInt) + shift).t().contiguous() : at::zeros({N, nb}, at::kInt);
      if (nb % 2) z = at::constant_pad_nd(z, {0, 1}, 0);
      at::Tensor zpairs = z.reshape({N, -1, 2});
      at::Tensor Z = at::bitwise_or(zpairs.select(2, 0), at::bitwise_left_shift(zpairs.select(2, 1), 4)).to(at::kByte).contiguous().reshape({-1});
      const std::string zn = g.UniqueName(dq->inputs[0] + "_nbits_zp");
      g.AddInitializer(zn, Z);
      inputs.push_back(zn);
    }
    Node* f = g.AddNode("MatMulNBits", inputs, {mm->outputs[0]}, kMSDomain, g.UniqueName("MatMulNBits_dq"));
    f->set_attr_i("K", K);
    f->set_attr_i("N", N);
    f->set_attr_i("bits", 4);
    f->set_attr_i("block_size", bs);
    f->set_attr_i("accuracy_level", accuracy);
    g.RemoveNode(mm);
    g.RemoveNode(dq);
    ++count;
  }
  return count;
}

}  // namespace

void AddMorePasses3(std::vector<Pass>& v) {
  v.push_back({"CastChainElimination", 1, false, CastChainElimination});
  v.push_back({"PreShapeNodeElimination", 1, false, PreShapeNodeElimination});
  v.push_back({"PadFusion", 1, false, PadFusion});
  v.push_back({"MatMulBNFusion", 1, false, MatMulBNFusion});
  v.push_back({"LabelEncoderFusion", 1, false, LabelEncoderFusion});
  v.push_back({"DQMatMulNBitsFusion", 1, false, DQMatMulNBitsFusion});
  v.push_back({"GemmActivationFusion", 2, false, GemmActivationFusion});
  v.push_back({"QDQFinalCleanup", 2, false, QDQFinalCleanup});
}

// registered ahead of the QDQ fusions (see optimizer.cc)
void AddQdqPrepPasses(std::vector<Pass>& v) { v.push_back({"EnsureUniqueDQForNodeUnit", 1, false, EnsureUniqueDQForNodeUnit}); }

}  // namespace opt
}  // namespace ortb
