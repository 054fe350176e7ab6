#include "shape_inference.h"

#include <algorithm>
#include <set>

namespace ortb {

namespace {

using Dim = pb::Dimension;
using Dims = std::vector<Dim>;
using Ctx = InferenceContext;

Dim Known(int64_t v) {
  Dim d;
  d.has_value = true;
  d.value = v;
  return d;
}
bool Same(const Dim& a, const Dim& b) {
  if (a.has_value != b.has_value) return false;
  return a.has_value ? a.value == b.value : (!a.param.empty() && a.param == b.param);
}
bool IsOne(const Dim& d) { return d.has_value && d.value == 1; }

// numpy-style broadcasting of two shapes; an unknown pair gives a fresh symbol
Dims Broadcast(Ctx& c, const Dims& a, const Dims& b) {
  const size_t r = std::max(a.size(), b.size());
  Dims out(r);
  for (size_t i = 0; i < r; ++i) {
    const Dim* da = i + a.size() >= r ? &a[i + a.size() - r] : nullptr;
    const Dim* db = i + b.size() >= r ? &b[i + b.size() - r] : nullptr;
    if (!da) out[i] = *db;
    else if (!db) out[i] = *da;
    else if (IsOne(*da)) out[i] = *db;
    else if (IsOne(*db)) out[i] = *da;
    else if (Same(*da, *db)) out[i] = *da;
    else if (da->has_value) out[i] = *da;   // a symbol against a value other than 1: the value wins (or it is an error)
    else if (db->has_value) out[i] = *db;
    else if (da->param.rfind("unk__", 0) == 0 && !db->param.empty()) out[i] = *db;  // a named size against an unknown one
    else if (db->param.rfind("unk__", 0) == 0 && !da->param.empty()) out[i] = *da;
    else out[i] = c.FreshDim();
  }
  return out;
}

int64_t NormAxis(int64_t axis, int rank) { return axis < 0 ? axis + rank : axis; }

std::vector<int64_t> ConstInts(const Ctx& c, size_t i, bool* ok) {
  std::vector<int64_t> out;
  *ok = false;
  const Dims* v = c.IntValue(i);
  if (!v) return out;
  for (auto& d : *v) {
    if (!d.has_value) return out;
    out.push_back(d.value);
  }
  *ok = true;
  return out;
}

// axes from an attribute (older opsets) or from a constant input (newer ones)
bool AxesOf(const Ctx& c, size_t input_idx, std::vector<int64_t>* axes) {
  if (c.node.has_attr("axes")) {
    *axes = c.node.attr_ints("axes");
    return true;
  }
  if (c.node.has_input(input_idx)) {
    bool ok = false;
    *axes = ConstInts(c, input_idx, &ok);
    return ok;
  }
  axes->clear();
  return true;
}

// ---------------------------------------------------------------------------------------------- generic functions
void SameAsFirst(Ctx& c) { c.PassThrough(0, 0); }

void BinaryBroadcast(Ctx& c, int32_t out_type /* 0 = type of input 0 */) {
  if (!c.Type(0) || !c.Type(1)) return;
  const int32_t t = out_type ? out_type : c.ElemType(0);
  if (c.HasShape(0) && c.HasShape(1)) c.SetOutput(0, t, Broadcast(c, c.Dims(0), c.Dims(1)));
  else c.SetOutputType(0, t);
  // integer arithmetic on tracked values (shape computations)
  const Dims* a = c.IntValue(0);
  const Dims* b = c.IntValue(1);
  if (a && b && !out_type && (a->size() == b->size() || a->size() == 1 || b->size() == 1)) {
    const std::string& op = c.node.op_type;
    if (op != "Add" && op != "Sub" && op != "Mul" && op != "Div") return;
    const size_t n = std::max(a->size(), b->size());
    Dims out(n);
    for (size_t i = 0; i < n; ++i) {
      const Dim& x = (*a)[a->size() == 1 ? 0 : i];
      const Dim& y = (*b)[b->size() == 1 ? 0 : i];
      if (x.has_value && y.has_value) {
        int64_t v = 0;
        if (op == "Add") v = x.value + y.value;
        else if (op == "Sub") v = x.value - y.value;
        else if (op == "Mul") v = x.value * y.value;
        else v = y.value != 0 ? x.value / y.value : 0;
        out[i] = Known(v);
      } else if (op == "Mul" && IsOne(x)) {
        out[i] = y;
      } else if ((op == "Mul" || op == "Div") && IsOne(y)) {
        out[i] = x;
      } else {
        out[i] = c.FreshDim();
      }
    }
    c.SetOutputIntValue(0, out);
  }
}

void InferMatMul(Ctx& c) {
  if (!c.Type(0)) return;
  if (!c.HasShape(0) || !c.HasShape(1)) {
    c.SetOutputType(0, c.ElemType(0));
    return;
  }
  Dims a = c.Dims(0), b = c.Dims(1);
  if (a.empty() || b.empty()) return;
  const bool a1 = a.size() == 1, b1 = b.size() == 1;
  if (a1) a.insert(a.begin(), Known(1));
  if (b1) b.push_back(Known(1));
  Dims batch = Broadcast(c, Dims(a.begin(), a.end() - 2), Dims(b.begin(), b.end() - 2));
  if (!a1) batch.push_back(a[a.size() - 2]);
  if (!b1) batch.push_back(b.back());
  c.SetOutput(0, c.ElemType(0), batch);
}

void InferGemm(Ctx& c) {
  if (!c.HasShape(0) || !c.HasShape(1) || c.Rank(0) != 2 || c.Rank(1) != 2) {
    if (c.Type(0)) c.SetOutputType(0, c.ElemType(0));
    return;
  }
  const bool ta = c.node.attr_i("transA", 0) != 0, tb = c.node.attr_i("transB", 0) != 0;
  c.SetOutput(0, c.ElemType(0), {c.Dims(0)[ta ? 1 : 0], c.Dims(1)[tb ? 0 : 1]});
}

void InferTranspose(Ctx& c) {
  if (!c.HasShape(0)) {
    if (c.Type(0)) c.SetOutputType(0, c.ElemType(0));
    return;
  }
  const Dims& in = c.Dims(0);
  std::vector<int64_t> perm = c.node.attr_ints("perm");
  if (perm.empty())
    for (int i = static_cast<int>(in.size()) - 1; i >= 0; --i) perm.push_back(i);
  if (perm.size() != in.size()) return;
  Dims out;
  for (int64_t p : perm) out.push_back(in[static_cast<size_t>(NormAxis(p, static_cast<int>(in.size())))]);
  c.SetOutput(0, c.ElemType(0), out);
}

void InferReshape(Ctx& c) {
  if (!c.Type(0)) return;
  const Dims* target = c.IntValue(1);
  if (!target) {
    // rank from the shape tensor's own length, when known
    if (c.HasShape(1) && c.Rank(1) == 1 && c.Dims(1)[0].has_value) {
      Dims out;
      for (int64_t i = 0; i < c.Dims(1)[0].value; ++i) out.push_back(c.FreshDim());
      c.SetOutput(0, c.ElemType(0), out);
    } else {
      c.SetOutputType(0, c.ElemType(0));
    }
    return;
  }
  const bool allowzero = c.node.attr_i("allowzero", 0) != 0;
  Dims out = *target;
  int infer_at = -1;
  for (size_t i = 0; i < out.size(); ++i) {
    if (out[i].has_value && out[i].value == 0 && !allowzero) {
      if (c.HasShape(0) && i < c.Dims(0).size()) out[i] = c.Dims(0)[i];
      else out[i] = c.FreshDim();
    } else if (out[i].has_value && out[i].value == -1) {
      infer_at = static_cast<int>(i);
    }
  }
  if (infer_at >= 0) {
    // -1: total elements of the input over the product of the other output dimensions; symbols that appear on both
    // sides cancel
    Dim res = c.FreshDim();
    if (c.HasShape(0)) {
      int64_t num = 1, den = 1;
      std::vector<std::string> sym_in, sym_out;
      for (auto& d : c.Dims(0)) {
        if (d.has_value) num *= d.value;
        else sym_in.push_back(d.param);
      }
      for (size_t i = 0; i < out.size(); ++i) {
        if (static_cast<int>(i) == infer_at) continue;
        if (out[i].has_value) den *= out[i].value;
        else sym_out.push_back(out[i].param);
      }
      bool cancels = true;
      for (auto& s : sym_out) {
        auto it = std::find(sym_in.begin(), sym_in.end(), s);
        if (s.empty() || it == sym_in.end()) {
          cancels = false;
          break;
        }
        sym_in.erase(it);
      }
      if (cancels && den != 0 && num % den == 0) {
        if (sym_in.empty()) res = Known(num / den);
        else if (sym_in.size() == 1 && num / den == 1 && !sym_in[0].empty()) {
          res = Dim();
          res.param = sym_in[0];
        }
      }
    }
    out[static_cast<size_t>(infer_at)] = res;
  }
  c.SetOutput(0, c.ElemType(0), out);
}

void InferShapeOp(Ctx& c) {
  if (c.HasShape(0)) {
    const Dims& in = c.Dims(0);
    int64_t start = NormAxis(c.node.attr_i("start", 0), static_cast<int>(in.size()));
    int64_t end = c.node.has_attr("end") ? NormAxis(c.node.attr_i("end", 0), static_cast<int>(in.size())) : static_cast<int64_t>(in.size());
    start = std::max<int64_t>(0, std::min<int64_t>(start, in.size()));
    end = std::max<int64_t>(start, std::min<int64_t>(end, in.size()));
    Dims v(in.begin() + start, in.begin() + end);
    c.SetOutput(0, pb::INT64, {Known(static_cast<int64_t>(v.size()))});
    c.SetOutputIntValue(0, v);
  } else {
    c.SetOutput(0, pb::INT64, {c.FreshDim()});
  }
}

void InferGather(Ctx& c) {
  if (!c.Type(0)) return;
  const int64_t axis_attr = c.node.attr_i("axis", 0);
  if (c.HasShape(0) && c.HasShape(1)) {
    const Dims& d = c.Dims(0);
    const int64_t axis = NormAxis(axis_attr, static_cast<int>(d.size()));
    if (axis < 0 || axis >= static_cast<int64_t>(d.size())) return;
    Dims out(d.begin(), d.begin() + axis);
    out.insert(out.end(), c.Dims(1).begin(), c.Dims(1).end());
    out.insert(out.end(), d.begin() + axis + 1, d.end());
    c.SetOutput(0, c.ElemType(0), out);
  } else {
    c.SetOutputType(0, c.ElemType(0));
  }
  // picking entries of a tracked shape value
  const Dims* v = c.IntValue(0);
  bool ok = false;
  std::vector<int64_t> idx = ConstInts(c, 1, &ok);
  if (v && ok && axis_attr == 0) {
    Dims out;
    for (int64_t i : idx) {
      if (i < 0) i += static_cast<int64_t>(v->size());
      if (i < 0 || i >= static_cast<int64_t>(v->size())) return;
      out.push_back((*v)[static_cast<size_t>(i)]);
    }
    c.SetOutputIntValue(0, out);
  }
}

void InferUnsqueeze(Ctx& c) {
  if (!c.Type(0)) return;
  std::vector<int64_t> axes;
  if (!AxesOf(c, 1, &axes) || !c.HasShape(0)) {
    c.SetOutputType(0, c.ElemType(0));
    return;
  }
  const int out_rank = c.Rank(0) + static_cast<int>(axes.size());
  std::set<int64_t> at;
  for (int64_t a : axes) at.insert(NormAxis(a, out_rank));
  Dims out;
  size_t src = 0;
  for (int i = 0; i < out_rank; ++i) {
    if (at.count(i)) out.push_back(Known(1));
    else if (src < c.Dims(0).size()) out.push_back(c.Dims(0)[src++]);
  }
  c.SetOutput(0, c.ElemType(0), out);
  if (const Dims* v = c.IntValue(0)) c.SetOutputIntValue(0, *v);  // the values do not change
}

void InferSqueeze(Ctx& c) {
  if (!c.Type(0)) return;
  std::vector<int64_t> axes;
  if (!AxesOf(c, 1, &axes) || !c.HasShape(0)) {
    c.SetOutputType(0, c.ElemType(0));
    return;
  }
  const int rank = c.Rank(0);
  std::set<int64_t> at;
  for (int64_t a : axes) at.insert(NormAxis(a, rank));
  Dims out;
  for (int i = 0; i < rank; ++i) {
    const Dim& d = c.Dims(0)[static_cast<size_t>(i)];
    if (axes.empty() ? IsOne(d) : at.count(i) != 0) continue;
    out.push_back(d);
  }
  c.SetOutput(0, c.ElemType(0), out);
  if (const Dims* v = c.IntValue(0)) c.SetOutputIntValue(0, *v);
}

void InferConcat(Ctx& c) {
  if (!c.Type(0)) return;
  const size_t n = c.NumInputs();
  bool all = true;
  for (size_t i = 0; i < n; ++i) all = all && c.HasShape(i);
  if (all && c.Rank(0) > 0) {
    const int rank = c.Rank(0);
    const int64_t axis = NormAxis(c.node.attr_i("axis", 0), rank);
    Dims out = c.Dims(0);
    bool known = out[static_cast<size_t>(axis)].has_value;
    int64_t sum = known ? out[static_cast<size_t>(axis)].value : 0;
    for (size_t i = 1; i < n; ++i) {
      if (c.Rank(i) != rank) return;
      const Dim& d = c.Dims(i)[static_cast<size_t>(axis)];
      known = known && d.has_value;
      if (d.has_value) sum += d.value;
      for (int k = 0; k < rank; ++k)
        if (k != axis && !out[static_cast<size_t>(k)].has_value && c.Dims(i)[static_cast<size_t>(k)].has_value) out[static_cast<size_t>(k)] = c.Dims(i)[static_cast<size_t>(k)];
    }
    out[static_cast<size_t>(axis)] = known ? Known(sum) : c.FreshDim();
    c.SetOutput(0, c.ElemType(0), out);
  } else {
    c.SetOutputType(0, c.ElemType(0));
  }
  // concatenation of tracked integer values (building a Reshape target)
  Dims v;
  for (size_t i = 0; i < n; ++i) {
    const Dims* p = c.IntValue(i);
    if (!p) return;
    v.insert(v.end(), p->begin(), p->end());
  }
  c.SetOutputIntValue(0, v);
}

}  // namespace

// declared here, defined in shape_inference_ops.cc: the operator table
void RegisterBuiltinSchemas(std::map<std::string, OpSchema>& table);

namespace shape_fn {
void Same(InferenceContext& c) { SameAsFirst(c); }
void Binary(InferenceContext& c) { BinaryBroadcast(c, 0); }
void Compare(InferenceContext& c) { BinaryBroadcast(c, pb::BOOL); }
void MatMul(InferenceContext& c) { InferMatMul(c); }
void Gemm(InferenceContext& c) { InferGemm(c); }
void Transpose(InferenceContext& c) { InferTranspose(c); }
void Reshape(InferenceContext& c) { InferReshape(c); }
void ShapeOp(InferenceContext& c) { InferShapeOp(c); }
void Gather(InferenceContext& c) { InferGather(c); }
void Unsqueeze(InferenceContext& c) { InferUnsqueeze(c); }
void Squeeze(InferenceContext& c) { InferSqueeze(c); }
void Concat(InferenceContext& c) { InferConcat(c); }
std::vector<pb::Dimension> BroadcastDims(InferenceContext& c, const std::vector<pb::Dimension>& a, const std::vector<pb::Dimension>& b) {
  return Broadcast(c, a, b);
}
}  // namespace shape_fn

// ------------------------------------------------------------------------------------------------ context
const pb::TypeProto* InferenceContext::Type(size_t i) const {
  if (i >= node.inputs.size() || node.inputs[i].empty()) return nullptr;
  auto it = types_.find(node.inputs[i]);
  return it == types_.end() || it->second.which != 1 ? nullptr : &it->second;
}

const std::vector<pb::Dimension>& InferenceContext::Dims(size_t i) const { return Type(i)->dims; }

const std::vector<pb::Dimension>* InferenceContext::IntValue(size_t i) const {
  if (i >= node.inputs.size() || node.inputs[i].empty()) return nullptr;
  auto it = values_.find(node.inputs[i]);
  return it == values_.end() ? nullptr : &it->second;
}

const at::Tensor* InferenceContext::Constant(size_t i) const {
  if (i >= node.inputs.size() || node.inputs[i].empty()) return nullptr;
  return graph_.GetConstant(node.inputs[i]);
}

void InferenceContext::SetOutput(size_t i, int32_t elem_type, const std::vector<pb::Dimension>& dims) {
  if (i >= node.outputs.size() || node.outputs[i].empty()) return;
  pb::TypeProto t;
  t.which = 1;
  t.elem_type = elem_type;
  t.has_shape = true;
  t.dims = dims;
  types_[node.outputs[i]] = std::move(t);
}

void InferenceContext::SetOutputType(size_t i, int32_t elem_type) {
  if (i >= node.outputs.size() || node.outputs[i].empty()) return;
  pb::TypeProto t;
  t.which = 1;
  t.elem_type = elem_type;
  types_[node.outputs[i]] = std::move(t);
}

void InferenceContext::SetOutputIntValue(size_t i, const std::vector<pb::Dimension>& value) {
  if (i >= node.outputs.size() || node.outputs[i].empty() || value.size() > 32) return;
  values_[node.outputs[i]] = value;
}

void InferenceContext::PassThrough(size_t in, size_t out) {
  const pb::TypeProto* t = Type(in);
  if (!t) return;
  if (t->has_shape) SetOutput(out, t->elem_type, t->dims);
  else SetOutputType(out, t->elem_type);
}

pb::Dimension InferenceContext::FreshDim() {
  pb::Dimension d;
  d.param = "unk__" + std::to_string(counter_++);
  return d;
}

// ------------------------------------------------------------------------------------------------ registry + driver
namespace {
std::map<std::string, OpSchema>& Table() {
  static std::map<std::string, OpSchema> table = [] {
    std::map<std::string, OpSchema> t;
    RegisterBuiltinSchemas(t);
    return t;
  }();
  return table;
}
}  // namespace

const OpSchema* FindSchema(const std::string& domain, const std::string& op_type) {
  auto& t = Table();
  auto it = t.find(domain + "::" + op_type);
  return it == t.end() ? nullptr : &it->second;
}

std::vector<const OpSchema*> AllSchemas() {
  std::vector<const OpSchema*> out;
  for (auto& kv : Table()) out.push_back(&kv.second);
  return out;
}

InferenceReport InferShapes(Graph& g, bool strict) {
  InferenceReport rep;
  std::map<std::string, pb::TypeProto> types;
  std::map<std::string, std::vector<pb::Dimension>> values;
  int counter = 0;
  for (auto& vi : g.Inputs()) types[vi.name] = vi.type;
  for (auto& kv : g.Initializers()) {
    pb::TypeProto t;
    t.which = 1;
    t.elem_type = ToOnnxType(kv.second.scalar_type());
    t.has_shape = true;
    for (int64_t s : kv.second.sizes()) t.dims.push_back(Known(s));
    types[kv.first] = std::move(t);
    // small integer constants are shape material
    if ((kv.second.scalar_type() == at::kLong || kv.second.scalar_type() == at::kInt) && kv.second.dim() <= 1 && kv.second.numel() <= 32 &&
        g.IsConstant(kv.first)) {
      at::Tensor c = kv.second.to(at::kCPU, at::kLong).reshape({-1});
      std::vector<pb::Dimension> v;
      for (int64_t i = 0; i < c.numel(); ++i) v.push_back(Known(c[i].item<int64_t>()));
      values[kv.first] = std::move(v);
    }
  }
  for (Node* n : g.TopologicalOrder()) {
    ++rep.nodes;
    const OpSchema* schema = FindSchema(n->domain, n->op_type);
    if (!schema) continue;
    size_t given = n->inputs.size();
    while (given > 0 && n->inputs[given - 1].empty()) --given;
    if (static_cast<int>(given) < schema->min_inputs || static_cast<int>(n->inputs.size()) > schema->max_inputs) {
      const std::string msg = MakeString(n->op_type, " node '", n->name, "' has ", given, " inputs, expected ", schema->min_inputs, "..",
                                         schema->max_inputs);
      if (strict) ORTB_THROW(INVALID_GRAPH, msg);
      rep.problems.push_back(msg);
      continue;
    }
    if (!schema->infer) continue;
    InferenceContext ctx(*n, g, types, values, counter);
    try {
      schema->infer(ctx);
    } catch (const std::exception& e) {
      rep.problems.push_back(MakeString(n->op_type, " node '", n->name, "': ", e.what()));
      continue;
    }
    bool all = true;
    for (auto& o : n->outputs)
      if (!o.empty()) {
        auto it = types.find(o);
        all = all && it != types.end() && it->second.has_shape;
      }
    if (all) ++rep.inferred;
  }
  // publish: value_info for intermediates, and shapes for outputs that were declared without one
  std::set<std::string> io;
  for (auto& vi : g.Inputs()) io.insert(vi.name);
  for (auto& vi : g.Outputs()) {
    io.insert(vi.name);
    auto it = types.find(vi.name);
    if (it == types.end()) continue;
    if (vi.type.which == 0 || vi.type.elem_type == 0) vi.type = it->second;
    else if (!vi.type.has_shape && it->second.has_shape) {
      vi.type.has_shape = true;
      vi.type.dims = it->second.dims;
    }
  }
  for (auto& kv : types) {
    if (io.count(kv.first) || g.IsInitializer(kv.first)) continue;
    ValueInfo vi;
    vi.name = kv.first;
    vi.type = kv.second;
    g.ValueInfos()[kv.first] = std::move(vi);
  }
  return rep;
}

}  // namespace ortb
