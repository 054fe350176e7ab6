// Further level-1 / level-2 graph rewrites: the smaller rules of the reference's optimizer that clean up what
// exporters leave behind.
//
// Reference passes: matmul_add_fusion.cc (MatMul + Add -> Gemm), reshape_fusion.cc (Shape / Gather / Concat target ->
// constant with 0 / -1), constant_sharing.cc, bias_softmax_fusion.cc, cast_elimination.cc, div_mul_fusion.cc,
// not_where_fusion.cc, gemm_transpose_fusion.cc, relu_clip_fusion.cc, slice_elimination.cc, expand_elimination.cc,
// unsqueeze_elimination.cc, and the Transpose-pair handling of
// transpose_optimization/onnx_transpose_optimization.cc; rule list: graph_transformer_utils.cc:133-156, 243-319.
#include <cmath>

#include "optimizer.h"

namespace ortb {
namespace opt {

namespace {

Node* SoleUser(const Graph& g, const std::string& v) {
  if (g.IsGraphOutput(v)) return nullptr;
  auto cs = g.Consumers(v);
  return cs.size() == 1 ? cs[0] : nullptr;
}

// Declared type / rank of a value, from graph inputs, initializers or value_info (filled by shape inference).
const pb::TypeProto* TypeOf(Graph& g, const std::string& v, pb::TypeProto* scratch) {
  for (auto& vi : g.Inputs())
    if (vi.name == v) return &vi.type;
  if (const at::Tensor* t = g.GetInitializer(v)) {
    scratch->which = 1;
    scratch->elem_type = ToOnnxType(t->scalar_type());
    scratch->has_shape = true;
    scratch->dims.clear();
    for (int64_t s : t->sizes()) {
      pb::Dimension d;
      d.has_value = true;
      d.value = s;
      scratch->dims.push_back(d);
    }
    return scratch;
  }
  auto it = g.ValueInfos().find(v);
  return it == g.ValueInfos().end() ? nullptr : &it->second.type;
}

int RankOf(Graph& g, const std::string& v) {
  pb::TypeProto tmp;
  const pb::TypeProto* t = TypeOf(g, v, &tmp);
  return t && t->which == 1 && t->has_shape ? static_cast<int>(t->dims.size()) : -1;
}

std::vector<int64_t> ConstI64(const Graph& g, const std::string& v, bool* ok) {
  *ok = false;
  std::vector<int64_t> out;
  const at::Tensor* t = g.GetConstant(v);
  if (!t || !(t->scalar_type() == at::kLong || t->scalar_type() == at::kInt) || t->dim() > 1) return out;
  at::Tensor c = t->to(at::kCPU, at::kLong).reshape({-1});
  for (int64_t i = 0; i < c.numel(); ++i) out.push_back(c[i].item<int64_t>());
  *ok = true;
  return out;
}

// MatMul(A[M, K], B const [K, N]) + bias const [N]  ->  Gemm(A, B, bias)
int MatMulAddFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* mm : g.Nodes()) {
    if (mm->op_type != "MatMul" || !mm->domain.empty() || mm->inputs.size() != 2) continue;
    const at::Tensor* w = g.GetConstant(mm->inputs[1]);
    if (!w || w->dim() != 2 || RankOf(g, mm->inputs[0]) != 2) continue;
    Node* add = SoleUser(g, mm->outputs[0]);
    if (!add || add->op_type != "Add" || !add->domain.empty() || add->inputs.size() != 2) continue;
    const std::string& other = add->inputs[0] == mm->outputs[0] ? add->inputs[1] : add->inputs[0];
    int64_t len = 0;
    if (!IsConst1D(g, other, &len) || len != w->size(1)) continue;
    if (g.GetConstant(other)->scalar_type() != w->scalar_type()) continue;
    Node* gemm = g.AddNode("Gemm", {mm->inputs[0], mm->inputs[1], other}, {add->outputs[0]}, "", g.UniqueName("Gemm"));
    (void)gemm;
    g.RemoveNode(add);
    g.RemoveNode(mm);
    ++count;
  }
  return count;
}

// Reshape(x, Concat(Unsqueeze(Gather(Shape(x), i)) at position i, constants...))  ->  Reshape(x, const) with 0 at the
// copied positions.  The Shape / Gather / Unsqueeze / Concat chain dies afterwards.
int ReshapeFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* rs : g.Nodes()) {
    if (rs->op_type != "Reshape" || !rs->domain.empty() || rs->inputs.size() != 2 || rs->attr_i("allowzero", 0) != 0) continue;
    Node* cat = g.Producer(rs->inputs[1]);
    if (!cat || cat->op_type != "Concat" || !cat->domain.empty() || cat->attr_i("axis", 0) != 0) continue;
    std::vector<int64_t> target;
    bool ok = true;
    int minus_one = 0;
    for (auto& in : cat->inputs) {
      bool is_const = false;
      std::vector<int64_t> k = ConstI64(g, in, &is_const);
      if (is_const) {
        for (int64_t v : k) {
          if (v == 0) ok = false;  // an explicit 0 would change meaning
          if (v == -1) ++minus_one;
          target.push_back(v);
        }
        continue;
      }
      // Unsqueeze(Gather(Shape(root), idx)) with idx == position and root == the data input
      Node* un = g.Producer(in);
      if (!un || un->op_type != "Unsqueeze" || !un->domain.empty()) { ok = false; break; }
      Node* ga = g.Producer(un->inputs[0]);
      if (!ga || ga->op_type != "Gather" || !ga->domain.empty() || ga->attr_i("axis", 0) != 0) { ok = false; break; }
      Node* sh = g.Producer(ga->inputs[0]);
      if (!sh || sh->op_type != "Shape" || !sh->domain.empty() || sh->inputs[0] != rs->inputs[0] || sh->has_attr("start") || sh->has_attr("end")) { ok = false; break; }
      bool idx_ok = false;
      std::vector<int64_t> idx = ConstI64(g, ga->inputs[1], &idx_ok);
      if (!idx_ok || idx.size() != 1 || idx[0] != static_cast<int64_t>(target.size())) { ok = false; break; }
      target.push_back(0);
    }
    if (!ok || minus_one > 1 || target.empty()) continue;
    const std::string name = g.UniqueName("reshape_target");
    g.AddInitializer(name, at::tensor(target, at::kLong));
    rs->inputs[1] = name;
    g.Invalidate();
    ++count;
  }
  return count;
}

// Identical small constants become one initializer (scalars and short 1-D tensors: axes, shapes, epsilons).
int ConstantSharing(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  std::map<std::string, std::string> canon;  // content key -> first name
  std::vector<std::pair<std::string, std::string>> renames;
  for (auto& kv : g.Initializers()) {
    const at::Tensor& t = kv.second;
    if (!g.IsConstant(kv.first) || g.IsGraphOutput(kv.first) || t.numel() > 8 || t.dim() > 1 || t.numel() == 0) continue;
    if (t.is_cuda() || g.PendingExternal().count(kv.first)) continue;
    at::Tensor b = t.contiguous();
    std::string key = std::to_string(static_cast<int>(t.scalar_type())) + ":" + std::to_string(t.dim()) + ":" +
                      std::string(static_cast<const char*>(b.data_ptr()), b.nbytes());
    auto it = canon.find(key);
    if (it == canon.end()) canon[key] = kv.first;
    else renames.emplace_back(kv.first, it->second);
  }
  for (auto& r : renames) {
    if (g.Consumers(r.first).empty()) continue;
    // subgraph bodies may read the name implicitly: leave those alone
    bool implicit = false;
    for (Node* n : g.Consumers(r.first)) implicit = implicit || !n->subgraphs.empty();
    if (implicit) continue;
    g.ReplaceAllUses(r.first, r.second);
    ++count;
  }
  return count;
}

// Softmax(Add(x, bias), axis = last)  ->  com.microsoft.BiasSoftmax(x, bias)
int BiasSoftmaxFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* sm : g.Nodes()) {
    if (sm->op_type != "Softmax" || !sm->domain.empty()) continue;
    Node* add = g.Producer(sm->inputs[0]);
    if (!add || add->op_type != "Add" || !add->domain.empty() || add->inputs.size() != 2 || SoleUser(g, add->outputs[0]) != sm) continue;
    const int rx = RankOf(g, add->inputs[0]), rb = RankOf(g, add->inputs[1]);
    if (rx < 1 || rb < 1) continue;
    const int64_t axis = sm->attr_i("axis", -1);
    const int rank = std::max(rx, rb);
    if (!(axis == -1 || axis == rank - 1)) continue;
    // the larger operand is the data, the other one the bias that broadcasts onto it
    const bool swap = rb > rx;
    const std::string x = add->inputs[swap ? 1 : 0], b = add->inputs[swap ? 0 : 1];
    Node* f = g.AddNode("BiasSoftmax", {x, b}, {sm->outputs[0]}, kMSDomain, g.UniqueName("BiasSoftmax"));
    f->set_attr_i("axis", -1);
    f->set_attr_i("is_inner_broadcast", 0);
    g.RemoveNode(sm);
    g.RemoveNode(add);
    ++count;
  }
  return count;
}

// Cast to the type the value already has; Cast(Cast(x, wider), T) of a value whose type is T is left to the first rule
// after the inner cast goes away.
int CastElimination(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* n : g.Nodes()) {
    if (n->op_type != "Cast" || !n->domain.empty() || n->inputs.size() != 1) continue;
    pb::TypeProto tmp;
    const pb::TypeProto* t = TypeOf(g, n->inputs[0], &tmp);
    if (!t || t->which != 1 || t->elem_type == 0 || t->elem_type != n->attr_i("to", 0)) continue;
    const std::string in = n->inputs[0], out = n->outputs[0];
    if (g.IsGraphOutput(out)) continue;
    g.ReplaceAllUses(out, in);
    g.RemoveNode(n);
    ++count;
  }
  return count;
}

// (1 / x) * y  ->  y / x     (Div with a constant 1 numerator feeding a Mul)
int DivMulFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* div : g.Nodes()) {
    if (div->op_type != "Div" || !div->domain.empty() || div->inputs.size() != 2) continue;
    double one = 0;
    if (!ScalarConst(g, div->inputs[0], &one) || one != 1.0) continue;
    Node* mul = SoleUser(g, div->outputs[0]);
    if (!mul || mul->op_type != "Mul" || !mul->domain.empty() || mul->inputs.size() != 2) continue;
    const std::string y = mul->inputs[0] == div->outputs[0] ? mul->inputs[1] : mul->inputs[0];
    if (y == div->outputs[0]) continue;
    g.AddNode("Div", {y, div->inputs[1]}, {mul->outputs[0]}, "", g.UniqueName("Div"));
    g.RemoveNode(mul);
    g.RemoveNode(div);
    ++count;
  }
  return count;
}

// Where(Not(c), a, b)  ->  Where(c, b, a)
int NotWhereFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* w : g.Nodes()) {
    if (w->op_type != "Where" || !w->domain.empty() || w->inputs.size() != 3) continue;
    Node* nt = g.Producer(w->inputs[0]);
    if (!nt || nt->op_type != "Not" || !nt->domain.empty()) continue;
    w->inputs[0] = nt->inputs[0];
    std::swap(w->inputs[1], w->inputs[2]);
    g.Invalidate();
    ++count;
  }
  return count;
}

// Transpose(perm swapping the last two of a 2-D value) feeding Gemm  ->  the Gemm's transA / transB flag
int GemmTransposeFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* gemm : g.Nodes()) {
    if (gemm->op_type != "Gemm" || !gemm->domain.empty()) continue;
    for (int side = 0; side < 2; ++side) {
      Node* tr = g.Producer(gemm->inputs[static_cast<size_t>(side)]);
      if (!tr || tr->op_type != "Transpose" || !tr->domain.empty() || g.IsGraphOutput(tr->outputs[0])) continue;
      std::vector<int64_t> perm = tr->attr_ints("perm");
      if (!(perm.empty() ? RankOf(g, tr->inputs[0]) == 2 : perm == std::vector<int64_t>{1, 0})) continue;
      const char* flag = side == 0 ? "transA" : "transB";
      gemm->set_attr_i(flag, gemm->attr_i(flag, 0) ? 0 : 1);
      gemm->inputs[static_cast<size_t>(side)] = tr->inputs[0];
      g.Invalidate();
      ++count;
    }
  }
  return count;
}

// Relu followed by Clip: the lower bound absorbs the Relu
int ReluClipFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* relu : g.Nodes()) {
    if (relu->op_type != "Relu" || !relu->domain.empty()) continue;
    Node* clip = SoleUser(g, relu->outputs[0]);
    if (!clip || clip->op_type != "Clip" || !clip->domain.empty() || clip->inputs[0] != relu->outputs[0]) continue;
    double lo = 0;
    const bool attr_form = clip->has_attr("min") || clip->has_attr("max");
    if (attr_form) {
      lo = clip->attr_f("min", -3.4e38f);
      if (lo < 0) clip->set_attr_f("min", 0.f);
    } else if (clip->has_input(1)) {
      if (!ScalarConst(g, clip->inputs[1], &lo)) continue;
      if (lo < 0) {
        const at::Tensor* t = g.GetConstant(clip->inputs[1]);
        const std::string name = g.UniqueName("clip_min");
        g.AddInitializer(name, at::zeros_like(*t));
        clip->inputs[1] = name;
      }
    } else {
      pb::TypeProto tmp;
      const pb::TypeProto* t = TypeOf(g, relu->inputs[0], &tmp);
      if (!t || t->which != 1) continue;
      const std::string name = g.UniqueName("clip_min");
      g.AddInitializer(name, at::zeros({}, at::TensorOptions().dtype(ToTorchType(t->elem_type))));
      if (clip->inputs.size() < 2) clip->inputs.resize(2);
      clip->inputs[1] = name;
    }
    clip->inputs[0] = relu->inputs[0];
    g.RemoveNode(relu);
    ++count;
  }
  return count;
}

// Transpose(Transpose(x, p1), p2): one Transpose with the composed permutation, or nothing when it is the identity
int TransposePairFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* t2 : g.Nodes()) {
    if (t2->op_type != "Transpose" || !t2->domain.empty()) continue;
    Node* t1 = g.Producer(t2->inputs[0]);
    if (!t1 || t1->op_type != "Transpose" || !t1->domain.empty()) continue;
    std::vector<int64_t> p1 = t1->attr_ints("perm"), p2 = t2->attr_ints("perm");
    const int rank = !p1.empty() ? static_cast<int>(p1.size()) : (!p2.empty() ? static_cast<int>(p2.size()) : RankOf(g, t1->inputs[0]));
    if (rank <= 0) continue;
    auto fill = [rank](std::vector<int64_t>& p) {
      if (p.empty())
        for (int i = rank - 1; i >= 0; --i) p.push_back(i);
    };
    fill(p1);
    fill(p2);
    if (static_cast<int>(p1.size()) != rank || static_cast<int>(p2.size()) != rank) continue;
    std::vector<int64_t> comp(static_cast<size_t>(rank));
    bool identity = true;
    for (int i = 0; i < rank; ++i) {
      comp[static_cast<size_t>(i)] = p1[static_cast<size_t>(p2[static_cast<size_t>(i)])];
      identity = identity && comp[static_cast<size_t>(i)] == i;
    }
    if (identity) {
      if (g.IsGraphOutput(t2->outputs[0])) continue;
      g.ReplaceAllUses(t2->outputs[0], t1->inputs[0]);
      g.RemoveNode(t2);
    } else {
      t2->inputs[0] = t1->inputs[0];
      t2->set_attr_ints("perm", comp);
      g.Invalidate();
    }
    ++count;  // t1 dies with its last user
  }
  return count;
}

// Slice that keeps everything, Expand to the shape the value already has (all ones target), Unsqueeze of a constant
int TrivialNodeElimination(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* n : g.Nodes()) {
    if (!n->domain.empty() || n->inputs.empty() || g.IsGraphOutput(n->outputs[0])) continue;
    bool drop = false;
    if (n->op_type == "Slice" && n->inputs.size() >= 3 && !n->has_attr("starts")) {
      bool a = false, b = false, s_ok = true;
      std::vector<int64_t> st = ConstI64(g, n->inputs[1], &a), en = ConstI64(g, n->inputs[2], &b), steps;
      if (n->has_input(4)) steps = ConstI64(g, n->inputs[4], &s_ok);
      if (a && b && s_ok && !st.empty()) {
        drop = true;
        for (size_t i = 0; i < st.size(); ++i) drop = drop && st[i] == 0 && en[i] >= (int64_t{1} << 31) - 1 && (steps.empty() || steps[i] == 1);
      }
    } else if (n->op_type == "Expand" && n->inputs.size() == 2) {
      bool ok = false;
      std::vector<int64_t> tgt = ConstI64(g, n->inputs[1], &ok);
      const int rank = RankOf(g, n->inputs[0]);
      if (ok && rank >= 0 && static_cast<int>(tgt.size()) <= rank) {
        drop = true;
        for (int64_t v : tgt) drop = drop && v == 1;
      }
    }
    if (!drop) continue;
    g.ReplaceAllUses(n->outputs[0], n->inputs[0]);
    g.RemoveNode(n);
    ++count;
  }
  return count;
}

// DequantizeLinear(QuantizeLinear(x, s, z), s, z) immediately re-quantised with the same parameters:
//   Q -> DQ -> Q(s, z) -> DQ   ->   Q -> DQ        (the reference's DoubleQDQPairsRemover for identical parameters)
int DoubleQDQPairsRemover(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  auto same_const = [&](const std::string& a, const std::string& b) {
    if (a == b) return true;
    const at::Tensor* x = g.GetConstant(a);
    const at::Tensor* y = g.GetConstant(b);
    return x && y && x->scalar_type() == y->scalar_type() && x->sizes() == y->sizes() && at::equal(x->cpu(), y->cpu());
  };
  for (Node* q2 : g.Nodes()) {
    if (q2->op_type != "QuantizeLinear" || !q2->domain.empty() || q2->inputs.size() < 2) continue;
    Node* dq1 = g.Producer(q2->inputs[0]);
    if (!dq1 || dq1->op_type != "DequantizeLinear" || !dq1->domain.empty() || SoleUser(g, dq1->outputs[0]) != q2) continue;
    if (!same_const(dq1->input(1), q2->input(1))) continue;
    if (dq1->has_input(2) != q2->has_input(2) || (q2->has_input(2) && !same_const(dq1->input(2), q2->input(2)))) continue;
    if (dq1->attr_i("axis", 1) != q2->attr_i("axis", 1) || g.IsGraphOutput(q2->outputs[0])) continue;
    g.ReplaceAllUses(q2->outputs[0], dq1->inputs[0]);
    g.RemoveNode(q2);
    g.RemoveNode(dq1);
    ++count;
  }
  return count;
}

// GroupQueryAttentionFusion (onnxruntime/core/optimizer/group_query_attention_fusion.cc): a GroupQueryAttention whose
// query and key come from two RotaryEmbedding nodes over the same caches and positions does the rotation itself
// (do_rotary = 1, position_ids passed through as input 9), and three MatMul projections of one activation with
// constant weights become one MatMul feeding the operator's packed-QKV form.
int GroupQueryAttentionFusion(PassContext& c) {
  Graph& g = c.g;
  int count = 0;
  for (Node* a : g.Nodes()) {
    if (a->removed || a->op_type != "GroupQueryAttention" || a->domain != kMSDomain) continue;
    bool changed = false;
    // ---- rotary embedding into the attention
    if (a->attr_i("do_rotary", 0) == 0 && !a->has_input(7) && !a->has_input(8) && a->has_input(1) && a->has_input(2)) {
      Node* rq = g.Producer(a->input(0));
      Node* rk = g.Producer(a->input(1));
      auto is_rotary = [&](Node* r) {
        return r && r->op_type == "RotaryEmbedding" && r->domain == kMSDomain && r->inputs.size() >= 4 && SoleUser(g, r->outputs[0]) == a &&
               r->attr_i("rotary_embedding_dim", 0) == 0 && r->attr_f("scale", 1.0f) == 1.0f && !r->attr_i("is_packed_batching", 0);
      };
      if (is_rotary(rq) && is_rotary(rk) && rq != rk && rq->input(1) == rk->input(1) && rq->input(2) == rk->input(2) &&
          rq->input(3) == rk->input(3) && rq->attr_i("interleaved", 0) == rk->attr_i("interleaved", 0) &&
          RankOf(g, rq->input(0)) != 4) {  // the operator takes [batch, sequence, hidden] projections
        const std::string pos = rq->input(1), cosv = rq->input(2), sinv = rq->input(3);
        const int64_t inter = rq->attr_i("interleaved", 0);
        a->inputs[0] = rq->input(0);
        a->inputs[1] = rk->input(0);
        while (a->inputs.size() < 10) a->inputs.push_back("");
        a->inputs[7] = cosv;
        a->inputs[8] = sinv;
        a->inputs[9] = pos;
        a->set_attr_i("do_rotary", 1);
        a->set_attr_i("rotary_interleaved", inter);
        g.Invalidate();
        g.RemoveNode(rq);
        g.RemoveNode(rk);
        changed = true;
      }
    }
    // ---- three projections of one activation into one packed projection
    if (a->has_input(1) && a->has_input(2)) {
      Node* mq = g.Producer(a->input(0));
      Node* mk = g.Producer(a->input(1));
      Node* mv = g.Producer(a->input(2));
      auto is_proj = [&](Node* m) {
        if (!m || m->op_type != "MatMul" || !m->domain.empty() || SoleUser(g, m->outputs[0]) != a) return false;
        const at::Tensor* w = g.GetConstant(m->input(1));
        return w != nullptr && w->dim() == 2;
      };
      if (is_proj(mq) && is_proj(mk) && is_proj(mv) && mq != mk && mk != mv && mq != mv && mq->input(0) == mk->input(0) &&
          mq->input(0) == mv->input(0)) {
        const at::Tensor* wq = g.GetConstant(mq->input(1));
        const at::Tensor* wk = g.GetConstant(mk->input(1));
        const at::Tensor* wv = g.GetConstant(mv->input(1));
        if (wq->size(0) == wk->size(0) && wq->size(0) == wv->size(0) && wq->scalar_type() == wk->scalar_type() &&
            wq->scalar_type() == wv->scalar_type() && wk->size(1) == wv->size(1)) {
          const std::string wname = g.UniqueName(mq->input(1) + "_qkv");
          g.AddInitializer(wname, at::cat({*wq, *wk, *wv}, 1).contiguous());
          const std::string packed = g.UniqueName(a->name + "_packed_qkv");
          Node* m = g.AddNode("MatMul", {mq->input(0), wname}, {packed}, "", g.UniqueName(mq->name + "_qkv"));
          (void)m;
          a->inputs[0] = packed;
          a->inputs[1] = "";
          a->inputs[2] = "";
          g.Invalidate();
          g.RemoveNode(mq);
          g.RemoveNode(mk);
          g.RemoveNode(mv);
          changed = true;
        }
      }
    }
    if (changed) ++count;
  }
  return count;
}

}  // namespace

void AddMorePasses(std::vector<Pass>& v) {
  v.push_back({"ConstantSharing", 1, false, ConstantSharing});
  v.push_back({"CastElimination", 1, false, CastElimination});
  v.push_back({"TrivialNodeElimination", 1, false, TrivialNodeElimination});
  v.push_back({"DivMulFusion", 1, false, DivMulFusion});
  v.push_back({"NotWhereFusion", 1, false, NotWhereFusion});
  v.push_back({"ReluClipFusion", 1, false, ReluClipFusion});
  v.push_back({"TransposePairFusion", 1, false, TransposePairFusion});
  v.push_back({"ReshapeFusion", 1, false, ReshapeFusion});
  v.push_back({"DoubleQDQPairsRemover", 1, false, DoubleQDQPairsRemover});
  v.push_back({"MatMulAddFusion", 1, false, MatMulAddFusion});
  v.push_back({"GemmTransposeFusion", 1, false, GemmTransposeFusion});
  v.push_back({"BiasSoftmaxFusion", 2, false, BiasSoftmaxFusion});
  v.push_back({"GroupQueryAttentionFusion", 2, false, GroupQueryAttentionFusion});
}

}  // namespace opt
}  // namespace ortb
