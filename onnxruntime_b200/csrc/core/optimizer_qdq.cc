// QDQ fusion: DequantizeLinear -> float operator -> QuantizeLinear groups become the matching quantised operator.
//
// Organised like the reference's selector / action framework (onnxruntime/core/optimizer/qdq_transformer/
// selectors_actions/qdq_selectors.cc, qdq_selector_action_transformer.cc): a *selector* recognises a node group
// (target node, the DequantizeLinear nodes on its data inputs, the QuantizeLinear node on its output) and checks that
// nothing else reads the float values; an *action* rewires the group into one node.  The table below lists one entry
// per target operator.  The quantised kernels compute "dequantise, float operator, requantise", so the rewrite
// does not change results; it removes the float intermediates and two thirds of the nodes.
// Config key "session.disable_quant_qdq" = "1" switches the pass off (same key as the reference).
#include <ATen/ATen.h>

#include "optimizer.h"

namespace ortb {
namespace opt {

namespace {

bool IsDQ(const Node* n) { return n && n->op_type == "DequantizeLinear" && (n->domain.empty() || n->domain == kMSDomain); }
bool IsQ(const Node* n) { return n && n->op_type == "QuantizeLinear" && (n->domain.empty() || n->domain == kMSDomain); }

struct Group {
  Node* target = nullptr;
  std::vector<Node*> dq;  // one per data input of the target, in input order (nullptr where the selector allows none)
  Node* q = nullptr;
};

// element type of a quantised value: initializer, graph input or value_info
int ElemTypeOf(Graph& g, const std::string& v) {
  if (const at::Tensor* t = g.GetInitializer(v)) return ToOnnxType(t->scalar_type());
  for (auto& vi : g.Inputs())
    if (vi.name == v) return vi.type.elem_type;
  auto it = g.ValueInfos().find(v);
  return it == g.ValueInfos().end() ? 0 : it->second.type.elem_type;
}

// zero point input of a Q / DQ node; creates a zero constant of the right type when the node has none
bool ZeroPointOf(Graph& g, Node* qdq, const std::string& quantised_value, std::string* out) {
  if (qdq->has_input(2)) {
    *out = qdq->input(2);
    return true;
  }
  const int et = ElemTypeOf(g, quantised_value);
  if (et != 2 && et != 3) return false;  // unknown quantised type: leave the group alone
  const std::string name = g.UniqueName(qdq->name + "_zero_point");
  g.AddInitializer(name, at::zeros({}, at::TensorOptions().dtype(et == 2 ? at::kByte : at::kChar)));
  *out = name;
  return true;
}

// A QuantizeLinear without zero point produces uint8.
bool OutputZeroPoint(Graph& g, Node* q, std::string* out) {
  if (q->has_input(2)) {
    *out = q->input(2);
    return true;
  }
  const std::string name = g.UniqueName(q->name + "_zero_point");
  g.AddInitializer(name, at::zeros({}, at::TensorOptions().dtype(at::kByte)));
  *out = name;
  return true;
}

bool ScalarQParams(const Graph& g, const Node* n) {
  const at::Tensor* s = g.GetConstant(n->input(1));
  if (!s || s->numel() != 1) return false;
  if (n->has_input(2)) {
    const at::Tensor* z = g.GetConstant(n->input(2));
    if (!z || z->numel() != 1) return false;
  }
  return true;
}

bool ConstQParams(const Graph& g, const Node* n) {
  if (!g.GetConstant(n->input(1))) return false;
  return !n->has_input(2) || g.GetConstant(n->input(2)) != nullptr;
}

bool SameQParams(const Graph& g, const Node* a, const Node* b) {
  auto same = [&](const std::string& x, const std::string& y) {
    if (x == y) return true;
    const at::Tensor* tx = g.GetConstant(x);
    const at::Tensor* ty = g.GetConstant(y);
    return tx && ty && tx->scalar_type() == ty->scalar_type() && tx->numel() == ty->numel() &&
           at::equal(tx->cpu().reshape({-1}), ty->cpu().reshape({-1}));
  };
  if (!same(a->input(1), b->input(1))) return false;
  if (a->has_input(2) != b->has_input(2)) return false;
  return !a->has_input(2) || same(a->input(2), b->input(2));
}

// Selector shared by every entry: data inputs `data_inputs` come from DequantizeLinear nodes that only feed the
// target, the single output goes to exactly one QuantizeLinear.  `per_axis_ok[i]` allows a per-axis scale on input i.
bool Select(Graph& g, Node* t, const std::vector<int>& data_inputs, const std::vector<bool>& per_axis_ok, Group* out) {
  if (t->outputs.size() != 1 || g.IsGraphOutput(t->outputs[0])) return false;
  auto users = g.Consumers(t->outputs[0]);
  if (users.size() != 1 || !IsQ(users[0]) || users[0]->inputs[0] != t->outputs[0]) return false;
  Node* q = users[0];
  if (!ScalarQParams(g, q)) return false;
  out->target = t;
  out->q = q;
  out->dq.clear();
  for (size_t k = 0; k < data_inputs.size(); ++k) {
    const int i = data_inputs[k];
    if (!t->has_input(i)) return false;
    Node* d = g.Producer(t->input(i));
    if (!IsDQ(d) || g.IsGraphOutput(d->outputs[0]) || g.Consumers(d->outputs[0]).size() != 1) return false;
    if (per_axis_ok[k] ? !ConstQParams(g, d) : !ScalarQParams(g, d)) return false;
    out->dq.push_back(d);
  }
  return true;
}

void Finish(Graph& g, const Group& grp, Node* fused, bool same_operator = false) {
  fused->name = grp.target->name.empty() ? g.UniqueName(fused->op_type) : grp.target->name + (same_operator ? "" : "_quant");
  for (auto& kv : grp.target->attrs) fused->attrs[kv.first] = kv.second;
  g.RemoveNode(grp.q);
  g.RemoveNode(grp.target);
  for (Node* d : grp.dq)
    if (d && !d->removed) g.RemoveNode(d);
}

// (x, x_scale, x_zp) triple of a DQ node
bool Triple(Graph& g, Node* d, std::vector<std::string>* in) {
  std::string zp;
  if (!ZeroPointOf(g, d, d->input(0), &zp)) return false;
  in->push_back(d->input(0));
  in->push_back(d->input(1));
  in->push_back(zp);
  return true;
}

int QdqFusion(PassContext& c) {
  Graph& g = c.g;
  if (c.config.Get("session.disable_quant_qdq", "0") == "1") return 0;
  int count = 0;
  for (Node* t : g.Nodes()) {
    if (t->removed || !t->domain.empty()) continue;
    const std::string& op = t->op_type;
    Group grp;
    std::vector<std::string> in;
    std::string yzp;
    if (op == "Conv" || op == "ConvTranspose") {
      if (!Select(g, t, {0, 1}, {false, op == "Conv"}, &grp)) continue;
      // a per-channel filter scale must run along the output channels (axis 0 of a Conv filter)
      if (g.GetConstant(grp.dq[1]->input(1))->numel() > 1 && grp.dq[1]->attr_i("axis", 1) != 0) continue;
      std::string bias;
      Node* bias_dq = nullptr;
      if (t->has_input(2)) {
        // the bias of a QDQ model is DequantizeLinear(int32, x_scale * w_scale, 0): the quantised operator takes the int32
        bias_dq = g.Producer(t->input(2));
        if (!IsDQ(bias_dq) || g.Consumers(bias_dq->outputs[0]).size() != 1) continue;
        const at::Tensor* b = g.GetConstant(bias_dq->input(0));
        if (!b || b->scalar_type() != at::kInt) continue;
        bias = bias_dq->input(0);
      }
      if (!Triple(g, grp.dq[0], &in) || !Triple(g, grp.dq[1], &in) || !OutputZeroPoint(g, grp.q, &yzp)) continue;
      in.push_back(grp.q->input(1));
      in.push_back(yzp);
      if (!bias.empty()) in.push_back(bias);
      Node* f = op == "Conv" ? g.AddNode("QLinearConv", in, {grp.q->outputs[0]})
                             : g.AddNode("QLinearConvTranspose", in, {grp.q->outputs[0]}, kMSDomain);
      if (bias_dq) grp.dq.push_back(bias_dq);
      Finish(g, grp, f);
    } else if (op == "MatMul") {
      if (!Select(g, t, {0, 1}, {false, false}, &grp)) continue;
      if (!Triple(g, grp.dq[0], &in) || !Triple(g, grp.dq[1], &in) || !OutputZeroPoint(g, grp.q, &yzp)) continue;
      in.push_back(grp.q->input(1));
      in.push_back(yzp);
      Finish(g, grp, g.AddNode("QLinearMatMul", in, {grp.q->outputs[0]}));
    } else if (op == "Add" || op == "Mul") {
      if (!Select(g, t, {0, 1}, {false, false}, &grp)) continue;
      if (!Triple(g, grp.dq[0], &in) || !Triple(g, grp.dq[1], &in) || !OutputZeroPoint(g, grp.q, &yzp)) continue;
      in.push_back(grp.q->input(1));
      in.push_back(yzp);
      Finish(g, grp, g.AddNode(op == "Add" ? "QLinearAdd" : "QLinearMul", in, {grp.q->outputs[0]}, kMSDomain));
    } else if (op == "AveragePool" || op == "GlobalAveragePool" || op == "Sigmoid" || op == "LeakyRelu" || op == "Softmax" ||
               op == "ReduceMean") {
      if (op == "ReduceMean" && t->has_input(1)) continue;  // axes as an input (opset 18): the quantised form takes an attribute
      if (!Select(g, t, {0}, {false}, &grp)) continue;
      if (!Triple(g, grp.dq[0], &in) || !OutputZeroPoint(g, grp.q, &yzp)) continue;
      in.push_back(grp.q->input(1));
      in.push_back(yzp);
      Node* f = g.AddNode("QLinear" + op, in, {grp.q->outputs[0]}, kMSDomain);
      const int since = t->since_version;
      Finish(g, grp, f);
      if (op == "Softmax") f->set_attr_i("opset", since > 0 ? since : 13);
    } else if (op == "Concat") {
      std::vector<int> idx;
      for (size_t i = 0; i < t->inputs.size(); ++i) idx.push_back(static_cast<int>(i));
      if (idx.empty() || !Select(g, t, idx, std::vector<bool>(idx.size(), false), &grp)) continue;
      if (!OutputZeroPoint(g, grp.q, &yzp)) continue;
      in.push_back(grp.q->input(1));
      in.push_back(yzp);
      bool ok = true;
      for (Node* d : grp.dq) ok = ok && Triple(g, d, &in);
      if (!ok) continue;
      Finish(g, grp, g.AddNode("QLinearConcat", in, {grp.q->outputs[0]}, kMSDomain));
    } else if (op == "Where") {
      if (!Select(g, t, {1, 2}, {false, false}, &grp)) continue;
      in.push_back(t->input(0));
      if (!Triple(g, grp.dq[0], &in) || !Triple(g, grp.dq[1], &in) || !OutputZeroPoint(g, grp.q, &yzp)) continue;
      in.push_back(grp.q->input(1));
      in.push_back(yzp);
      Finish(g, grp, g.AddNode("QLinearWhere", in, {grp.q->outputs[0]}, kMSDomain));
    } else if (op == "MaxPool" || op == "Reshape" || op == "Transpose" || op == "Flatten" || op == "Squeeze" || op == "Unsqueeze" ||
               op == "Relu") {
      // operators that commute with the affine code: run them on the quantised values when both sides use the same
      // parameters (Relu additionally needs the zero point to sit at the type's lowest value or be clamped there, so
      // it is only dropped when the quantised type cannot represent negative numbers: zero point == lowest)
      if (!Select(g, t, {0}, {false}, &grp) || !SameQParams(g, grp.dq[0], grp.q)) continue;
      if (op == "MaxPool" && t->outputs.size() > 1) continue;
      if (op == "Relu") {
        std::string zp;
        if (!ZeroPointOf(g, grp.dq[0], grp.dq[0]->input(0), &zp)) continue;
        const at::Tensor* z = g.GetConstant(zp);
        if (!z) continue;
        const int64_t zv = z->to(at::kLong).reshape({-1})[0].item<int64_t>();
        const int64_t lowest = z->scalar_type() == at::kChar ? -128 : 0;
        if (zv != lowest) continue;
        g.ReplaceAllUses(grp.q->outputs[0], grp.dq[0]->input(0));
        g.RemoveNode(grp.q);
        g.RemoveNode(grp.target);
        g.RemoveNode(grp.dq[0]);
      } else {
        std::vector<std::string> ins = t->inputs;
        ins[0] = grp.dq[0]->input(0);
        Finish(g, grp, g.AddNode(op, ins, {grp.q->outputs[0]}), /*same_operator=*/true);
      }
    } else {
      continue;
    }
    ++count;
  }
  return count;
}

}  // namespace

void AddQdqPasses(std::vector<Pass>& v) { v.push_back({"QDQFusion", 2, false, QdqFusion}); }

}  // namespace opt
}  // namespace ortb
