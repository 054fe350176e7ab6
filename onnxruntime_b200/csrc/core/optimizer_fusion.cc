// Level-2 ("extended") transformer fusions into com.microsoft operators.
//
// Reference passes and the subgraphs they look for:
//  * fast_gelu_fusion.cc (:173-336) tanh-approximation forms -> FastGelu
//  * bias_gelu_fusion.cc  Add(x, 1-D const) + Gelu/FastGelu -> BiasGelu / FastGelu(bias)
//  * skip_layer_norm_fusion.cc (:130-165) Add + LayerNormalization -> SkipLayerNormalization
//    (and the RMS twin SkipSimplifiedLayerNormalization), with an optional 1-D bias Add
//  * attention_fusion.cc (:1205-1255) the BERT self-attention block -> Attention
//  * embed_layer_norm_fusion.cc  word/position/segment Gather + Add + LayerNorm -> EmbedLayerNormalization
//  * matmul_nbits_fusion.cc  MatMulNBits + Add(1-D const) -> MatMulNBits(bias)
//  * quick_gelu_fusion.cc  x * sigmoid(alpha * x) -> QuickGelu
#include <cmath>

#include "optimizer.h"

namespace ortb {
namespace opt {

namespace {

int FastGeluFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  const double k0 = 0.7978845608028654, k1 = 0.044715, k01 = k0 * k1;
  std::vector<Pat> inners = {
      Op("Mul", {C(k0), Op("Add", {V("x"), Op("Mul", {C(k1), Op("Pow", {V("x"), C(3.0)})})})}),
      Op("Mul", {Op("Mul", {V("x"), C(k0)}), Op("Add", {C(1.0), Op("Mul", {C(k1), Op("Mul", {V("x"), V("x")})})})}),
      Op("Mul", {Op("Mul", {V("x"), C(k0)}), Op("Add", {C(1.0), Op("Mul", {Op("Mul", {C(k1), V("x")}), V("x")})})}),
      Op("Mul", {V("x"), Op("Add", {C(k0), Op("Mul", {C(k01), Op("Mul", {V("x"), V("x")})})})}),
      Op("Mul", {V("x"), Op("Add", {C(k0), Op("Mul", {Op("Mul", {C(k01), V("x")}), V("x")})})}),
      Op("Mul", {C(k0), Op("Add", {V("x"), Op("Mul", {C(k1), Op("Mul", {V("x"), Op("Mul", {V("x"), V("x")})})})})}),
  };
  std::vector<Pat> pats;
  for (auto& inner : inners) {
    Pat t = Op("Add", {C(1.0), Op("Tanh", {inner})});
    pats.push_back(Op("Mul", {Op("Mul", {V("x"), C(0.5)}), t}));
    pats.push_back(Op("Mul", {C(0.5), Op("Mul", {V("x"), t})}));
    pats.push_back(Op("Mul", {V("x"), Op("Mul", {C(0.5), t})}));
  }
  for (Node* n : g.Nodes()) {
    if (n->op_type != "Mul" || !n->domain.empty()) continue;
    for (auto& p : pats) {
      Match m;
      if (!MatchExpr(g, n->outputs[0], p, &m)) continue;
      if (!IsClosed(g, m, n)) continue;
      g.AddNode("FastGelu", {m.values["x"]}, {n->outputs[0]}, kMSDomain, g.UniqueName("FastGelu"));
      RemoveMatched(g, m);
      ++count;
      break;
    }
  }
  return count;
}

int QuickGeluFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  Pat p = Op("Mul", {V("x"), Op("Sigmoid", {Op("Mul", {V("x"), K("alpha")})})});
  for (Node* n : g.Nodes()) {
    if (n->op_type != "Mul" || !n->domain.empty()) continue;
    Match m;
    if (!MatchExpr(g, n->outputs[0], p, &m) || !IsClosed(g, m, n)) continue;
    double alpha;
    if (!ScalarConst(g, m.values["alpha"], &alpha)) continue;
    Node* f = g.AddNode("QuickGelu", {m.values["x"]}, {n->outputs[0]}, kMSDomain, g.UniqueName("QuickGelu"));
    f->set_attr_f("alpha", static_cast<float>(alpha));
    RemoveMatched(g, m);
    ++count;
  }
  return count;
}

int BiasGeluFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* n : g.Nodes()) {
    const bool gelu = n->op_type == "Gelu" && (n->domain == kMSDomain || (n->domain.empty() && n->attr_s("approximate", "none") == "none"));
    const bool fast = (n->op_type == "FastGelu" && n->domain == kMSDomain && !n->has_input(1)) ||
                      (n->op_type == "Gelu" && n->domain.empty() && n->attr_s("approximate", "none") == "tanh");
    if (!gelu && !fast) continue;
    Node* add = g.Producer(n->inputs[0]);
    if (!add || add->op_type != "Add" || !add->domain.empty() || g.NumConsumers(add->outputs[0]) != 1) continue;
    int bias_side = -1;
    for (int s = 0; s < 2; ++s)
      if (IsConst1D(g, add->inputs[s])) bias_side = s;
    if (bias_side < 0) continue;
    const std::string x = add->inputs[1 - bias_side], b = add->inputs[bias_side];
    if (g.GetConstant(x)) continue;
    Node* f = g.AddNode(gelu ? "BiasGelu" : "FastGelu", {x, b}, {n->outputs[0]}, kMSDomain,
                        g.UniqueName(gelu ? "BiasGelu" : "FastGelu"));
    (void)f;
    g.RemoveNode(n);
    g.RemoveNode(add);
    ++count;
  }
  return count;
}

// Add(+bias) + (Simplified)LayerNormalization -> Skip(Simplified)LayerNormalization
int SkipLayerNormFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* ln : g.Nodes()) {
    const bool simplified = ln->op_type == "SimplifiedLayerNormalization" && ln->domain.empty();
    const bool full = ln->op_type == "LayerNormalization" && ln->domain.empty();
    if (!simplified && !full) continue;
    if (ln->attr_i("axis", -1) != -1) continue;
    for (size_t i = 1; i < ln->outputs.size(); ++i)
      if (!ln->outputs[i].empty() && g.NumConsumers(ln->outputs[i]) > 0) goto next;
    {
      Node* add = g.Producer(ln->inputs[0]);
      if (!add || add->op_type != "Add" || !add->domain.empty()) continue;
      if (g.GetConstant(add->inputs[0]) || g.GetConstant(add->inputs[1])) continue;  // that is a bias add, not a residual
      std::string a = add->inputs[0], b = add->inputs[1], bias;
      std::vector<Node*> extra;
      // optional bias: one side is Add(t, 1-D const) consumed only here
      for (int side = 0; side < 2 && bias.empty(); ++side) {
        const std::string& v = side == 0 ? a : b;
        Node* ba = g.Producer(v);
        if (!ba || ba->op_type != "Add" || !ba->domain.empty() || g.NumConsumers(v) != 1) continue;
        for (int s = 0; s < 2; ++s) {
          if (IsConst1D(g, ba->inputs[s]) && !g.GetConstant(ba->inputs[1 - s])) {
            bias = ba->inputs[s];
            (side == 0 ? a : b) = ba->inputs[1 - s];
            extra.push_back(ba);
            break;
          }
        }
      }
      const bool sum_needed = g.NumConsumers(add->outputs[0]) > 1;
      std::vector<std::string> ins = {a, b, ln->inputs[1]};
      if (full) ins.push_back(ln->has_input(2) ? ln->inputs[2] : "");
      if (!bias.empty()) ins.push_back(bias);
      while (!ins.empty() && ins.back().empty()) ins.pop_back();
      std::vector<std::string> outs = {ln->outputs[0]};
      if (sum_needed) outs = {ln->outputs[0], "", "", add->outputs[0]};
      Node* f = g.AddNode(full ? "SkipLayerNormalization" : "SkipSimplifiedLayerNormalization", ins, outs, kMSDomain,
                          g.UniqueName("SkipLayerNorm"));
      f->set_attr_f("epsilon", ln->attr_f("epsilon", 1e-5f));
      g.RemoveNode(ln);
      g.RemoveNode(add);
      for (Node* e : extra) g.RemoveNode(e);
      ++count;
    }
  next:;
  }
  return count;
}

int MatMulNBitsBiasFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* add : g.Nodes()) {
    if (add->op_type != "Add" || !add->domain.empty()) continue;
    for (int s = 0; s < 2; ++s) {
      Node* mm = g.Producer(add->inputs[s]);
      if (!mm || mm->op_type != "MatMulNBits" || mm->domain != kMSDomain || mm->has_input(5)) continue;
      if (g.NumConsumers(mm->outputs[0]) != 1) continue;
      int64_t len = 0;
      if (!IsConst1D(g, add->inputs[1 - s], &len) || len != mm->attr_i("N", -1)) continue;
      mm->inputs.resize(6);
      mm->inputs[5] = add->inputs[1 - s];
      mm->outputs[0] = add->outputs[0];
      g.RemoveNode(add);
      g.Invalidate();
      ++count;
      break;
    }
  }
  return count;
}

// ----------------------------------------------------------- BERT attention
// Looks for: x -> {MatMul(Wq)+Add(bq), MatMul(Wk)+Add(bk), MatMul(Wv)+Add(bv)} -> Reshape -> Transpose ->
// Q.K^T -> (Div | Mul by scale) -> (+ mask) -> Softmax -> .V -> Transpose -> Reshape, and rewrites it to
// Attention(x, W[hidden, 3*hidden], B[3*hidden], mask_index).
struct Proj {
  Node *matmul = nullptr, *add = nullptr, *reshape = nullptr, *transpose = nullptr;
  std::string w, b, x;
  std::vector<Node*> nodes;
};

bool MatchProjection(Graph& g, const std::string& value, bool k_transposed, Proj* p) {
  Node* t = g.Producer(value);
  if (!t || t->op_type != "Transpose" || !t->domain.empty()) return false;
  std::vector<int64_t> perm = t->attr_ints("perm");
  const std::vector<int64_t> want = k_transposed ? std::vector<int64_t>{0, 2, 3, 1} : std::vector<int64_t>{0, 2, 1, 3};
  if (perm != want) return false;
  Node* r = g.Producer(t->inputs[0]);
  if (!r || r->op_type != "Reshape" || !r->domain.empty()) return false;
  Node* add = g.Producer(r->inputs[0]);
  if (!add || add->op_type != "Add" || !add->domain.empty()) return false;
  int bs = -1;
  for (int s = 0; s < 2; ++s)
    if (IsConst1D(g, add->inputs[s])) bs = s;
  if (bs < 0) return false;
  Node* mm = g.Producer(add->inputs[1 - bs]);
  if (!mm || mm->op_type != "MatMul" || !mm->domain.empty()) return false;
  const at::Tensor* w = g.GetConstant(mm->inputs[1]);
  if (!w || w->dim() != 2) return false;
  p->matmul = mm;
  p->add = add;
  p->reshape = r;
  p->transpose = t;
  p->w = mm->inputs[1];
  p->b = add->inputs[bs];
  p->x = mm->inputs[0];
  p->nodes = {t, r, add, mm};
  return true;
}

int AttentionFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* out_reshape : g.Nodes()) {
    if (out_reshape->op_type != "Reshape" || !out_reshape->domain.empty()) continue;
    Node* out_t = g.Producer(out_reshape->inputs[0]);
    if (!out_t || out_t->op_type != "Transpose" || out_t->attr_ints("perm") != std::vector<int64_t>{0, 2, 1, 3}) continue;
    Node* pv = g.Producer(out_t->inputs[0]);
    if (!pv || pv->op_type != "MatMul" || !pv->domain.empty()) continue;
    Node* sm = g.Producer(pv->inputs[0]);
    if (!sm || sm->op_type != "Softmax" || !sm->domain.empty()) continue;
    const int64_t sm_axis = sm->attr_i("axis", sm->since_version >= 13 ? -1 : 1);
    if (sm_axis != -1 && sm_axis != 3) continue;
    Proj v;
    if (!MatchProjection(g, pv->inputs[1], false, &v)) continue;
    // softmax input: optional mask Add, then scaling, then QK
    std::vector<Node*> mid = {out_t, pv, sm};
    std::string cur = sm->inputs[0];
    std::string mask_value;
    Node* n = g.Producer(cur);
    if (n && n->op_type == "Add" && n->domain.empty()) {
      // one side is the attention scores (produced by Div/Mul/MatMul), the other the additive mask
      auto is_score = [&](const std::string& v) {
        Node* p = g.Producer(v);
        if (!p || !p->domain.empty()) return false;
        if (p->op_type == "MatMul") return true;
        if (p->op_type != "Div" && p->op_type != "Mul") return false;
        for (auto& in : p->inputs) {
          Node* pp = g.Producer(in);
          if (pp && pp->domain.empty() && pp->op_type == "MatMul") return true;
        }
        return false;
      };
      int score_side = -1;
      for (int s = 0; s < 2; ++s)
        if (is_score(n->inputs[s])) score_side = s;
      if (score_side < 0) continue;
      mask_value = n->inputs[1 - score_side];
      mid.push_back(n);
      cur = n->inputs[score_side];
      n = g.Producer(cur);
    }
    double scale = 0;
    bool have_scale = false;
    if (n && n->domain.empty() && (n->op_type == "Div" || n->op_type == "Mul")) {
      double k;
      int ks = -1;
      for (int s = 0; s < 2; ++s)
        if (ScalarConst(g, n->inputs[s], &k)) ks = s;
      if (ks < 0 || (n->op_type == "Div" && ks != 1)) continue;
      ScalarConst(g, n->inputs[ks], &k);
      scale = n->op_type == "Div" ? 1.0 / k : k;
      have_scale = true;
      mid.push_back(n);
      cur = n->inputs[1 - ks];
      n = g.Producer(cur);
    }
    if (!n || n->op_type != "MatMul" || !n->domain.empty()) continue;
    Node* qk = n;
    mid.push_back(qk);
    Proj q, k;
    if (!MatchProjection(g, qk->inputs[0], false, &q)) continue;
    bool k_ok = MatchProjection(g, qk->inputs[1], true, &k);
    if (!k_ok) {
      // K as Transpose(perm 0,2,1,3) followed by Transpose(0,1,3,2)
      Node* t2 = g.Producer(qk->inputs[1]);
      if (t2 && t2->op_type == "Transpose" && t2->attr_ints("perm") == std::vector<int64_t>{0, 1, 3, 2} &&
          MatchProjection(g, t2->inputs[0], false, &k)) {
        k.nodes.push_back(t2);
        k_ok = true;
      }
    }
    if (!k_ok) continue;
    if (q.x != k.x || q.x != v.x) continue;
    const at::Tensor* wq = g.GetConstant(q.w);
    const at::Tensor* wk = g.GetConstant(k.w);
    const at::Tensor* wv = g.GetConstant(v.w);
    const at::Tensor* bq = g.GetConstant(q.b);
    const at::Tensor* bk = g.GetConstant(k.b);
    const at::Tensor* bv = g.GetConstant(v.b);
    if (!wq || !wk || !wv || !bq || !bk || !bv) continue;
    if (wq->sizes() != wk->sizes() || wq->sizes() != wv->sizes()) continue;
    // number of heads from the Q reshape target [0 or B, 0 or S, heads, head_size]
    const at::Tensor* shp = g.GetConstant(q.reshape->input(1));
    if (!shp || shp->numel() != 4) continue;
    at::Tensor shc = shp->to(at::kCPU, at::kLong).reshape({-1});
    const int64_t num_heads = shc[2].item<int64_t>(), head = shc[3].item<int64_t>();
    if (num_heads <= 0 || head <= 0 || num_heads * head != wq->size(1)) continue;
    if (have_scale && std::abs(scale - 1.0 / std::sqrt(static_cast<double>(head))) > 1e-4 * scale) {
      // non-default scale is carried as an attribute
    }
    // closedness: every interior value is used only inside the block
    Match m;
    for (Node* x : mid) m.matched.push_back(x);
    for (Proj* p : {&q, &k, &v})
      for (Node* x : p->nodes) m.matched.push_back(x);
    m.matched.insert(m.matched.begin(), out_reshape);
    if (!IsClosed(g, m, out_reshape)) continue;

    // mask: only the exact expansion of a 2-D keep-mask is understood,
    //   Mul(Sub(1, Cast?(Unsqueeze(Unsqueeze(mask)))), negative constant)      (Cast may sit on either side of the
    // Unsqueezes; one Unsqueeze with two axes counts as two).  Anything else added to the scores (an additive float
    // mask, a bias, a differently built expansion) leaves the block unfused: turning it into mask_index would change
    // the result.
    std::string mask_index;
    if (!mask_value.empty()) {
      Node* mul = g.Producer(mask_value);
      if (!mul || !mul->domain.empty() || mul->op_type != "Mul" || mul->inputs.size() != 2) continue;
      double neg = 0;
      int cs = -1;
      for (int s2 = 0; s2 < 2; ++s2)
        if (ScalarConst(g, mul->inputs[s2], &neg)) cs = s2;
      if (cs < 0 || !(neg < -1.0)) continue;
      Node* sub = g.Producer(mul->inputs[1 - cs]);
      double one = 0;
      if (!sub || !sub->domain.empty() || sub->op_type != "Sub" || sub->inputs.size() != 2 ||
          !ScalarConst(g, sub->inputs[0], &one) || std::abs(one - 1.0) > 1e-6)
        continue;
      std::string mv = sub->inputs[1];
      int unsqueezed = 0, guard = 0;
      bool ok = true;
      for (Node* p = g.Producer(mv); p && guard++ < 6; p = g.Producer(mv)) {
        if (!p->domain.empty()) break;
        if (p->op_type == "Cast") {
          mv = p->inputs[0];
        } else if (p->op_type == "Unsqueeze") {
          std::vector<int64_t> axes = p->attr_ints("axes");
          if (axes.empty() && p->has_input(1)) {
            const at::Tensor* ax = g.GetConstant(p->inputs[1]);
            if (!ax) { ok = false; break; }
            at::Tensor axc = ax->to(at::kCPU, at::kLong).reshape({-1});
            for (int64_t i = 0; i < axc.numel(); ++i) axes.push_back(axc[i].item<int64_t>());
          }
          for (int64_t a : axes)
            if (a != 1 && a != 2) ok = false;  // [B, S] -> [B, 1, 1, S]
          unsqueezed += static_cast<int>(axes.size());
          mv = p->inputs[0];
        } else {
          break;
        }
      }
      if (!ok || unsqueezed != 2) continue;
      // a declared rank other than 2 rules the pattern out
      for (auto& vi : g.Inputs())
        if (vi.name == mv && vi.type.which == 1 && vi.type.has_shape && vi.type.dims.size() != 2) ok = false;
      if (!ok) continue;
      mask_index = mv;
    }

    at::Tensor W = at::cat({*wq, *wk, *wv}, 1).contiguous();
    at::Tensor Bv = at::cat({*bq, *bk, *bv}, 0).contiguous();
    const std::string wn = g.UniqueName("attn_qkv_weight"), bn = g.UniqueName("attn_qkv_bias");
    g.AddInitializer(wn, W);
    g.AddInitializer(bn, Bv);
    std::vector<std::string> ins = {q.x, wn, bn};
    if (!mask_index.empty()) {
      // Attention wants an int32 mask
      const std::string cast_out = g.UniqueName(mask_index + "_int32");
      Node* cast = g.AddNode("Cast", {mask_index}, {cast_out}, "", g.UniqueName("MaskCast"));
      cast->set_attr_i("to", pb::INT32);
      ins.push_back(cast_out);
    }
    Node* f = g.AddNode("Attention", ins, {out_reshape->outputs[0]}, kMSDomain, g.UniqueName("Attention"));
    f->set_attr_i("num_heads", num_heads);
    // always explicit: the operator's default is 1 / sqrt(head size), which is wrong for a block that scales elsewhere
    // (folded into the weights) or not at all
    f->set_attr_f("scale", have_scale ? static_cast<float>(scale) : 1.0f);
    RemoveMatched(g, m);
    ++count;
  }
  return count;
}

// ------------------------------------------------------- EmbedLayerNorm
int EmbedLayerNormFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* ln : g.Nodes()) {
    if (ln->op_type != "LayerNormalization" || !ln->domain.empty() || !ln->has_input(2)) continue;
    for (size_t i = 1; i < ln->outputs.size(); ++i)
      if (!ln->outputs[i].empty() && g.NumConsumers(ln->outputs[i]) > 0) goto next;
    {
      // LN(Add(Add(Gather(word, ids), Gather(pos, pos_ids)), Gather(seg, seg_ids))) in any association; segment optional
      std::vector<Node*> gathers, adds;
      std::vector<std::string> work = {ln->inputs[0]};
      bool bad = false;
      while (!work.empty() && !bad) {
        const std::string v = work.back();
        work.pop_back();
        Node* p = g.Producer(v);
        if (!p || !p->domain.empty() || g.NumConsumers(v) != 1) {
          bad = true;
          break;
        }
        if (p->op_type == "Add") {
          adds.push_back(p);
          work.push_back(p->inputs[0]);
          work.push_back(p->inputs[1]);
        } else if (p->op_type == "Gather" && p->attr_i("axis", 0) == 0 && g.GetConstant(p->inputs[0]) &&
                   g.GetConstant(p->inputs[0])->dim() == 2) {
          gathers.push_back(p);
        } else {
          bad = true;
        }
      }
      if (bad || gathers.size() < 2 || gathers.size() > 3) continue;
      // classify: position ids are constant or derived; word ids and segment ids are graph inputs
      Node *word = nullptr, *pos = nullptr, *seg = nullptr;
      for (Node* ga : gathers) {
        const std::string& idx = ga->inputs[1];
        if (g.GetConstant(idx) || !g.IsGraphInput(idx)) {
          if (!pos) pos = ga;
          else bad = true;
        } else if (!word) {
          word = ga;
        } else if (!seg) {
          seg = ga;
        } else {
          bad = true;
        }
      }
      if (bad || !word || !pos) continue;
      // of the two id-driven tables the larger one is the vocabulary
      if (seg && g.GetConstant(seg->inputs[0])->size(0) > g.GetConstant(word->inputs[0])->size(0)) std::swap(word, seg);
      // position ids must be the default 0..S-1 row(s) when constant
      const at::Tensor* pids = g.GetConstant(pos->inputs[1]);
      std::string position_ids_input;
      if (pids) {
        at::Tensor pc = pids->to(at::kCPU, at::kLong);
        at::Tensor first = pc.dim() == 2 ? pc[0] : pc;
        if (!at::equal(first, at::arange(first.numel(), first.options()))) continue;
      } else {
        position_ids_input = pos->inputs[1];
      }
      auto to_int32 = [&](const std::string& ids) {
        const std::string out = g.UniqueName(ids + "_int32");
        Node* cast = g.AddNode("Cast", {ids}, {out}, "", g.UniqueName("IdsCast"));
        cast->set_attr_i("to", pb::INT32);
        return out;
      };
      std::vector<std::string> ins = {to_int32(word->inputs[1]), seg ? to_int32(seg->inputs[1]) : "", word->inputs[0],
                                      pos->inputs[0], seg ? seg->inputs[0] : "", ln->inputs[1], ln->inputs[2]};
      if (!position_ids_input.empty()) {
        ins.push_back("");
        ins.push_back(position_ids_input);
      }
      const std::string mask_out = g.UniqueName("embed_mask_index");
      Node* f = g.AddNode("EmbedLayerNormalization", ins, {ln->outputs[0], mask_out}, kMSDomain, g.UniqueName("EmbedLayerNorm"));
      f->set_attr_f("epsilon", ln->attr_f("epsilon", 1e-12f));
      g.RemoveNode(ln);
      for (Node* a : adds) g.RemoveNode(a);
      for (Node* ga : gathers) g.RemoveNode(ga);
      ++count;
    }
  next:;
  }
  return count;
}

}  // namespace

void AddFusionPasses(std::vector<Pass>& v) {
  v.push_back({"FastGeluFusion", 2, false, FastGeluFusion});
  v.push_back({"QuickGeluFusion", 2, false, QuickGeluFusion});
  v.push_back({"AttentionFusion", 2, false, AttentionFusion});
  v.push_back({"EmbedLayerNormFusion", 2, false, EmbedLayerNormFusion});
  v.push_back({"BiasGeluFusion", 2, false, BiasGeluFusion});
  v.push_back({"SkipLayerNormFusion", 2, false, SkipLayerNormFusion});
  v.push_back({"MatMulNBitsFusion", 2, false, MatMulNBitsBiasFusion});
}

}  // namespace opt
}  // namespace ortb
