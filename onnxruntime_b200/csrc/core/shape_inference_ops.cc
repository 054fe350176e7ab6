// The operator schema table: input counts and the shape function of every operator the runtime resolves statically.
// ONNX-domain entries follow the operator specifications; com.microsoft entries follow the reference's schema
// definitions (onnxruntime/core/graph/contrib_ops/bert_defs.cc, contrib_defs.cc, quantization_defs.cc,
// collective_defs.cc) as documented in docs/ContribOperators.md.
#include <algorithm>
#include <set>

#include "shape_inference.h"

namespace ortb {

namespace shape_fn {
void Same(InferenceContext& c);
void Binary(InferenceContext& c);
void Compare(InferenceContext& c);
void MatMul(InferenceContext& c);
void Gemm(InferenceContext& c);
void Transpose(InferenceContext& c);
void Reshape(InferenceContext& c);
void ShapeOp(InferenceContext& c);
void Gather(InferenceContext& c);
void Unsqueeze(InferenceContext& c);
void Squeeze(InferenceContext& c);
void Concat(InferenceContext& c);
std::vector<pb::Dimension> BroadcastDims(InferenceContext& c, const std::vector<pb::Dimension>& a, const std::vector<pb::Dimension>& b);
}  // namespace shape_fn

namespace {

using Dim = pb::Dimension;
using Dims = std::vector<Dim>;
using Ctx = InferenceContext;
constexpr const char* MS = "com.microsoft";
constexpr const char* FUSED = "com.ortb200";
constexpr int kAny = 1 << 20;

Dim Known(int64_t v) {
  Dim d;
  d.has_value = true;
  d.value = v;
  return d;
}
int64_t NormAxis(int64_t a, int rank) { return a < 0 ? a + rank : a; }

bool Ints(const Ctx& c, size_t i, std::vector<int64_t>* out) {
  out->clear();
  const Dims* v = c.IntValue(i);
  if (!v) return false;
  for (auto& d : *v) {
    if (!d.has_value) return false;
    out->push_back(d.value);
  }
  return true;
}

void Cast(Ctx& c) {
  if (!c.Type(0)) return;
  const int32_t to = static_cast<int32_t>(c.node.attr_i("to", c.ElemType(0)));
  if (c.HasShape(0)) c.SetOutput(0, to, c.Dims(0));
  else c.SetOutputType(0, to);
  if (const Dims* v = c.IntValue(0)) c.SetOutputIntValue(0, *v);
}

void Where(Ctx& c) {
  if (!c.Type(1)) return;
  if (c.HasShape(0) && c.HasShape(1) && c.HasShape(2))
    c.SetOutput(0, c.ElemType(1), shape_fn::BroadcastDims(c, shape_fn::BroadcastDims(c, c.Dims(0), c.Dims(1)), c.Dims(2)));
  else c.SetOutputType(0, c.ElemType(1));
}

void Expand(Ctx& c) {
  if (!c.Type(0)) return;
  const Dims* target = c.IntValue(1);
  if (c.HasShape(0) && target) c.SetOutput(0, c.ElemType(0), shape_fn::BroadcastDims(c, c.Dims(0), *target));
  else c.SetOutputType(0, c.ElemType(0));
}

void Flatten(Ctx& c) {
  if (!c.HasShape(0)) {
    if (c.Type(0)) c.SetOutputType(0, c.ElemType(0));
    return;
  }
  const Dims& d = c.Dims(0);
  const int64_t axis = NormAxis(c.node.attr_i("axis", 1), static_cast<int>(d.size()));
  auto prod = [&](size_t lo, size_t hi) {
    int64_t p = 1;
    for (size_t i = lo; i < hi; ++i) {
      if (!d[i].has_value) return hi - lo == 1 ? d[i] : c.FreshDim();
      p *= d[i].value;
    }
    return Known(p);
  };
  c.SetOutput(0, c.ElemType(0), {prod(0, static_cast<size_t>(axis)), prod(static_cast<size_t>(axis), d.size())});
}

void Reduce(Ctx& c) {
  if (!c.Type(0)) return;
  int32_t t = c.ElemType(0);
  if (c.node.op_type == "ArgMax" || c.node.op_type == "ArgMin") t = pb::INT64;
  if (!c.HasShape(0)) {
    c.SetOutputType(0, t);
    return;
  }
  const int rank = c.Rank(0);
  const bool keep = c.node.attr_i("keepdims", 1) != 0;
  std::vector<int64_t> axes;
  if (c.node.op_type == "ArgMax" || c.node.op_type == "ArgMin") {
    axes = {c.node.attr_i("axis", 0)};
  } else if (c.node.has_attr("axes")) {
    axes = c.node.attr_ints("axes");
  } else if (c.node.has_input(1)) {
    if (!Ints(c, 1, &axes)) {
      c.SetOutputType(0, t);
      return;
    }
  }
  if (axes.empty() && c.node.attr_i("noop_with_empty_axes", 0) != 0) {
    c.SetOutput(0, t, c.Dims(0));
    return;
  }
  std::set<int64_t> at;
  for (int64_t a : axes) at.insert(NormAxis(a, rank));
  Dims out;
  for (int i = 0; i < rank; ++i) {
    const bool red = axes.empty() || at.count(i) != 0;
    if (!red) out.push_back(c.Dims(0)[static_cast<size_t>(i)]);
    else if (keep) out.push_back(Known(1));
  }
  c.SetOutput(0, t, out);
}

void Slice(Ctx& c) {
  if (!c.Type(0)) return;
  std::vector<int64_t> starts, ends, axes, steps;
  bool ok = c.HasShape(0);
  if (c.node.has_attr("starts")) {
    starts = c.node.attr_ints("starts");
    ends = c.node.attr_ints("ends");
    axes = c.node.attr_ints("axes");
  } else {
    ok = ok && Ints(c, 1, &starts) && Ints(c, 2, &ends);
    if (c.node.has_input(3)) ok = ok && Ints(c, 3, &axes);
    if (c.node.has_input(4)) ok = ok && Ints(c, 4, &steps);
  }
  if (!ok && c.HasShape(0) && !c.node.has_attr("starts")) {
    // a prefix slice whose end is a tracked symbolic size (x[:, :seq]): the sliced axis takes that size
    const Dims* sv = c.IntValue(1);
    const Dims* ev = c.IntValue(2);
    std::vector<int64_t> ax, stp;
    const bool ax_ok = c.node.has_input(3) ? Ints(c, 3, &ax) : false;
    const bool st_ok = c.node.has_input(4) ? Ints(c, 4, &stp) : true;
    if (sv && ev && ax_ok && st_ok && sv->size() == ev->size() && ax.size() == ev->size()) {
      Dims out = c.Dims(0);
      bool fine = true;
      for (size_t i = 0; i < ev->size() && fine; ++i) {
        const size_t a = static_cast<size_t>(NormAxis(ax[i], c.Rank(0)));
        fine = a < out.size() && (*sv)[i].has_value && (*sv)[i].value == 0 && (stp.empty() || stp[i] == 1);
        if (!fine) break;
        if ((*ev)[i].has_value) out[a] = out[a].has_value ? Known(std::min(out[a].value, (*ev)[i].value)) : c.FreshDim();
        else out[a] = (*ev)[i];
      }
      if (fine) {
        c.SetOutput(0, c.ElemType(0), out);
        return;
      }
    }
  }
  if (!ok) {
    if (c.HasShape(0)) {
      // the rank survives; sliced axes are unknown
      Dims out = c.Dims(0);
      std::vector<int64_t> ax;
      if (c.node.has_input(3) && Ints(c, 3, &ax)) {
        for (int64_t a : ax) out[static_cast<size_t>(NormAxis(a, c.Rank(0)))] = c.FreshDim();
      } else {
        for (auto& d : out) d = c.FreshDim();
      }
      c.SetOutput(0, c.ElemType(0), out);
    } else {
      c.SetOutputType(0, c.ElemType(0));
    }
    return;
  }
  Dims out = c.Dims(0);
  const int rank = c.Rank(0);
  if (axes.empty())
    for (size_t i = 0; i < starts.size(); ++i) axes.push_back(static_cast<int64_t>(i));
  if (steps.empty()) steps.assign(starts.size(), 1);
  for (size_t i = 0; i < starts.size() && i < axes.size(); ++i) {
    const size_t ax = static_cast<size_t>(NormAxis(axes[i], rank));
    if (ax >= out.size()) return;
    if (!out[ax].has_value) {
      // a whole-axis slice keeps the symbol
      if (!(starts[i] == 0 && ends[i] >= (int64_t{1} << 30) && steps[i] == 1)) out[ax] = c.FreshDim();
      continue;
    }
    const int64_t dim = out[ax].value, step = steps[i] == 0 ? 1 : steps[i];
    int64_t s = starts[i] < 0 ? starts[i] + dim : starts[i], e = ends[i] < 0 ? ends[i] + dim : ends[i];
    if (step > 0) {
      s = std::max<int64_t>(0, std::min(s, dim));
      e = std::max<int64_t>(0, std::min(e, dim));
      out[ax] = Known(std::max<int64_t>(0, (e - s + step - 1) / step));
    } else {
      s = std::max<int64_t>(-1, std::min(s, dim - 1));
      e = std::max<int64_t>(-1, std::min(e, dim - 1));
      out[ax] = Known(std::max<int64_t>(0, (s - e - step - 1) / (-step)));
    }
  }
  c.SetOutput(0, c.ElemType(0), out);
  // slicing a tracked shape value
  const Dims* v = c.IntValue(0);
  if (v && starts.size() == 1 && NormAxis(axes[0], 1) == 0 && steps[0] == 1) {
    const int64_t n = static_cast<int64_t>(v->size());
    int64_t s = starts[0] < 0 ? starts[0] + n : starts[0], e = ends[0] < 0 ? ends[0] + n : ends[0];
    s = std::max<int64_t>(0, std::min(s, n));
    e = std::max<int64_t>(s, std::min(e, n));
    c.SetOutputIntValue(0, Dims(v->begin() + s, v->begin() + e));
  }
}

void Split(Ctx& c) {
  if (!c.Type(0)) return;
  const size_t n_out = c.node.outputs.size();
  if (!c.HasShape(0)) {
    for (size_t i = 0; i < n_out; ++i) c.SetOutputType(i, c.ElemType(0));
    return;
  }
  const int rank = c.Rank(0);
  const size_t axis = static_cast<size_t>(NormAxis(c.node.attr_i("axis", 0), rank));
  std::vector<int64_t> split = c.node.attr_ints("split");
  if (split.empty() && c.node.has_input(1)) Ints(c, 1, &split);
  for (size_t i = 0; i < n_out; ++i) {
    Dims out = c.Dims(0);
    if (split.size() == n_out) out[axis] = Known(split[i]);
    else if (out[axis].has_value && n_out > 0) {
      const int64_t per = (out[axis].value + static_cast<int64_t>(n_out) - 1) / static_cast<int64_t>(n_out);
      out[axis] = Known(i + 1 < n_out ? per : out[axis].value - per * static_cast<int64_t>(n_out - 1));
    } else out[axis] = c.FreshDim();
    c.SetOutput(i, c.ElemType(0), out);
  }
}

void ConstantOfShape(Ctx& c) {
  int32_t t = pb::FLOAT;
  at::Tensor v = c.node.attr_tensor("value");
  if (v.defined()) t = ToOnnxType(v.scalar_type());
  if (const Dims* target = c.IntValue(0)) c.SetOutput(0, t, *target);
  else c.SetOutputType(0, t);
}

void ConstantOp(Ctx& c) {
  at::Tensor v = c.node.attr_tensor("value");
  if (v.defined()) {
    Dims d;
    for (int64_t s : v.sizes()) d.push_back(Known(s));
    c.SetOutput(0, ToOnnxType(v.scalar_type()), d);
    if ((v.scalar_type() == at::kLong || v.scalar_type() == at::kInt) && v.dim() <= 1 && v.numel() <= 32) {
      at::Tensor f = v.to(at::kCPU, at::kLong).reshape({-1});
      Dims val;
      for (int64_t i = 0; i < f.numel(); ++i) val.push_back(Known(f[i].item<int64_t>()));
      c.SetOutputIntValue(0, val);
    }
  } else if (c.node.has_attr("value_int")) {
    c.SetOutput(0, pb::INT64, {});
    c.SetOutputIntValue(0, {Known(c.node.attr_i("value_int", 0))});
  } else if (c.node.has_attr("value_ints")) {
    std::vector<int64_t> v2 = c.node.attr_ints("value_ints");
    c.SetOutput(0, pb::INT64, {Known(static_cast<int64_t>(v2.size()))});
    Dims val;
    for (int64_t x : v2) val.push_back(Known(x));
    c.SetOutputIntValue(0, val);
  } else if (c.node.has_attr("value_float")) {
    c.SetOutput(0, pb::FLOAT, {});
  }
}

// Conv / pooling: N, C_out, spatial...
void ConvLike(Ctx& c, bool is_conv) {
  if (!c.HasShape(0)) {
    if (c.Type(0)) c.SetOutputType(0, c.ElemType(0));
    return;
  }
  const Dims& x = c.Dims(0);
  if (x.size() < 3) return;
  const size_t sp = x.size() - 2;
  std::vector<int64_t> k = c.node.attr_ints("kernel_shape"), st = c.node.attr_ints("strides"), pads = c.node.attr_ints("pads"),
                       dil = c.node.attr_ints("dilations");
  Dims out = {x[0], x[1]};
  if (is_conv) {
    if (!c.HasShape(1)) {
      c.SetOutputType(0, c.ElemType(0));
      return;
    }
    out[1] = c.Dims(1)[0];
    if (k.empty())
      for (size_t i = 0; i < sp; ++i) k.push_back(c.Dims(1)[2 + i].has_value ? c.Dims(1)[2 + i].value : -1);
  }
  if (k.size() != sp) return;
  if (st.empty()) st.assign(sp, 1);
  if (dil.empty()) dil.assign(sp, 1);
  if (pads.empty()) pads.assign(2 * sp, 0);
  const std::string auto_pad = c.node.attr_s("auto_pad", "NOTSET");
  const bool ceil_mode = c.node.attr_i("ceil_mode", 0) != 0;
  for (size_t i = 0; i < sp; ++i) {
    if (!x[2 + i].has_value || k[i] < 0) {
      out.push_back(c.FreshDim());
      continue;
    }
    const int64_t in = x[2 + i].value, eff = (k[i] - 1) * dil[i] + 1;
    int64_t o;
    if (auto_pad == "SAME_UPPER" || auto_pad == "SAME_LOWER") o = (in + st[i] - 1) / st[i];
    else {
      const int64_t total = auto_pad == "VALID" ? 0 : pads[i] + pads[i + sp];
      const int64_t num = in + total - eff;
      o = (ceil_mode ? (num + st[i] - 1) / st[i] : num / st[i]) + 1;
    }
    out.push_back(Known(std::max<int64_t>(o, 0)));
  }
  c.SetOutput(0, c.ElemType(0), out);
}

void GlobalPool(Ctx& c) {
  if (!c.HasShape(0) || c.Rank(0) < 3) return;
  Dims out = {c.Dims(0)[0], c.Dims(0)[1]};
  for (int i = 2; i < c.Rank(0); ++i) out.push_back(Known(1));
  c.SetOutput(0, c.ElemType(0), out);
}

void TopK(Ctx& c) {
  if (!c.HasShape(0)) return;
  Dims out = c.Dims(0);
  const size_t axis = static_cast<size_t>(NormAxis(c.node.attr_i("axis", -1), c.Rank(0)));
  std::vector<int64_t> k;
  if (c.node.has_attr("k")) out[axis] = Known(c.node.attr_i("k", 1));
  else if (Ints(c, 1, &k) && k.size() == 1) out[axis] = Known(k[0]);
  else out[axis] = c.FreshDim();
  c.SetOutput(0, c.ElemType(0), out);
  c.SetOutput(1, pb::INT64, out);
}

void LayerNorm(Ctx& c) {
  c.PassThrough(0, 0);
  // optional mean / inverse standard deviation outputs: reduced over the normalised axes
  if (c.HasShape(0) && c.node.outputs.size() > 1) {
    const int rank = c.Rank(0);
    const int64_t axis = NormAxis(c.node.attr_i("axis", -1), rank);
    Dims red = c.Dims(0);
    for (int i = static_cast<int>(axis); i < rank; ++i) red[static_cast<size_t>(i)] = Known(1);
    for (size_t o = 1; o < c.node.outputs.size() && o < 3; ++o) c.SetOutput(o, pb::FLOAT, red);
  }
}

// ---- com.microsoft
void SkipLayerNorm(Ctx& c) {
  c.PassThrough(0, 0);
  if (c.node.outputs.size() > 3) c.PassThrough(0, 3);  // input + skip (+ bias)
}

void EmbedLayerNorm(Ctx& c) {
  // (input_ids [B, S], ..., word_embedding [V, H]) -> [B, S, H], mask_index [B]
  if (!c.HasShape(0) || !c.HasShape(2) || c.Rank(0) != 2 || c.Rank(2) != 2) return;
  c.SetOutput(0, c.ElemType(2), {c.Dims(0)[0], c.Dims(0)[1], c.Dims(2)[1]});
  c.SetOutput(1, pb::INT32, {c.Dims(0)[0]});
  if (c.node.outputs.size() > 2) c.SetOutput(2, c.ElemType(2), {c.Dims(0)[0], c.Dims(0)[1], c.Dims(2)[1]});
}

void BertAttention(Ctx& c) {
  // input [B, S, Hin], weights [Hin, 3 * Hout] -> [B, S, Hout]
  if (!c.HasShape(0) || c.Rank(0) != 3) return;
  Dims out = c.Dims(0);
  std::vector<int64_t> sizes = c.node.attr_ints("qkv_hidden_sizes");
  if (sizes.size() == 3) out[2] = Known(sizes[2]);
  else if (c.HasShape(1) && c.Rank(1) == 2 && c.Dims(1)[1].has_value) out[2] = Known(c.Dims(1)[1].value / 3);
  c.SetOutput(0, c.ElemType(0), out);
}

void MultiHeadAttention(Ctx& c) {
  // query [B, S, H] (or packed [B, S, N, 3, h]) -> [B, S, H_v]
  if (!c.HasShape(0)) return;
  if (c.Rank(0) == 3) {
    Dims out = c.Dims(0);
    if (c.HasShape(2) && c.Rank(2) == 3) out[2] = c.Dims(2)[2];
    c.SetOutput(0, c.ElemType(0), out);
  } else if (c.Rank(0) == 5) {
    const Dims& q = c.Dims(0);
    Dim h = c.FreshDim();
    if (q[2].has_value && q[4].has_value) h = Known(q[2].value * q[4].value);
    c.SetOutput(0, c.ElemType(0), {q[0], q[1], h});
  }
}

void GroupQueryAttention(Ctx& c) {
  // query [B, S, N * h] or packed [B, S, (N + 2 Nk) h]; present caches [B, Nk, max(past, total), h]
  if (!c.HasShape(0) || c.Rank(0) != 3) return;
  const int64_t N = c.node.attr_i("num_heads", 0), Nk = c.node.attr_i("kv_num_heads", 0);
  Dims out = c.Dims(0);
  const bool packed = !c.node.has_input(1);
  int64_t head = 0;
  if (out[2].has_value && N > 0) {
    head = packed ? out[2].value / (N + 2 * Nk) : out[2].value / N;
    out[2] = Known(head * N);
  }
  c.SetOutput(0, c.ElemType(0), out);
  for (size_t o = 1; o <= 2 && o < c.node.outputs.size(); ++o) {
    const size_t past = 2 + o;  // past_key = input 3, past_value = input 4
    if (c.HasShape(past)) c.SetOutput(o, c.ElemType(past), {c.Dims(past)[0], c.Dims(past)[1], c.FreshDim(), c.Dims(past)[3]});
    else if (head > 0) c.SetOutput(o, c.ElemType(0), {c.Dims(0)[0], Known(Nk), c.FreshDim(), Known(head)});
  }
}

void MatMulNBits(Ctx& c) {
  if (!c.HasShape(0) || c.Rank(0) < 1) return;
  Dims out = c.Dims(0);
  out.back() = Known(c.node.attr_i("N", 0));
  c.SetOutput(0, c.ElemType(0), out);
}

void FusedGemm(Ctx& c) {
  // x [..., K] @ W [K, N]
  if (!c.HasShape(0) || !c.HasShape(1) || c.Rank(1) != 2) return;
  Dims out = c.Dims(0);
  out.back() = c.Dims(1)[1];
  c.SetOutput(0, c.ElemType(0), out);
}

void FusedMatMul(Ctx& c) {
  if (!c.HasShape(0) || !c.HasShape(1) || c.Rank(0) < 2 || c.Rank(1) < 2) return;
  Dims a = c.Dims(0), b = c.Dims(1);
  if (c.node.attr_i("transA", 0)) std::swap(a[a.size() - 1], a[a.size() - 2]);
  if (c.node.attr_i("transB", 0)) std::swap(b[b.size() - 1], b[b.size() - 2]);
  Dims out = shape_fn::BroadcastDims(c, Dims(a.begin(), a.end() - 2), Dims(b.begin(), b.end() - 2));
  out.push_back(a[a.size() - 2]);
  out.push_back(b.back());
  c.SetOutput(0, c.ElemType(0), out);
}

void AllGatherOp(Ctx& c) {
  if (!c.HasShape(0)) return;
  Dims out = c.Dims(0);
  const int64_t axis = NormAxis(c.node.attr_i("axis", 0), c.Rank(0)), group = c.node.attr_i("group_size", 0);
  if (axis >= 0 && axis < c.Rank(0)) {
    Dim& d = out[static_cast<size_t>(axis)];
    d = (d.has_value && group > 0) ? Known(d.value * group) : c.FreshDim();
  }
  c.SetOutput(0, c.ElemType(0), out);
}

void GemmFloat8(Ctx& c) {
  if (!c.HasShape(0) || !c.HasShape(1) || c.Rank(0) != 2 || c.Rank(1) != 2) return;
  const bool ta = c.node.attr_i("transA", 0) != 0, tb = c.node.attr_i("transB", 0) != 0;
  const int32_t dt = static_cast<int32_t>(c.node.attr_i("dtype", pb::FLOAT));
  c.SetOutput(0, dt, {c.Dims(0)[ta ? 1 : 0], c.Dims(1)[tb ? 0 : 1]});
}

void QuantizeLinear(Ctx& c) {
  if (!c.Type(0)) return;
  const int32_t t = c.HasInput(2) ? c.ElemType(2) : pb::UINT8;
  if (c.HasShape(0)) c.SetOutput(0, t, c.Dims(0));
  else c.SetOutputType(0, t);
}
void DequantizeLinear(Ctx& c) {
  if (!c.Type(0)) return;
  const int32_t t = c.Type(1) ? c.ElemType(1) : pb::FLOAT;
  if (c.HasShape(0)) c.SetOutput(0, t, c.Dims(0));
  else c.SetOutputType(0, t);
}

void Reg(std::map<std::string, OpSchema>& t, const char* domain, const char* op, int min_in, int max_in,
         std::function<void(Ctx&)> fn = nullptr) {
  OpSchema s;
  s.domain = domain;
  s.op_type = op;
  s.min_inputs = min_in;
  s.max_inputs = max_in;
  s.infer = std::move(fn);
  t[std::string(domain) + "::" + op] = std::move(s);
}

}  // namespace

void RegisterBuiltinSchemas(std::map<std::string, OpSchema>& t) {
  using namespace shape_fn;
  for (const char* op : {"Abs", "Neg", "Exp", "Log", "Sqrt", "Reciprocal", "Relu", "Sigmoid", "Tanh", "Erf", "Sin", "Cos", "Tan", "Asin",
                         "Acos", "Atan", "Sinh", "Cosh", "Asinh", "Acosh", "Atanh", "Ceil", "Floor", "Round", "Sign", "Softplus",
                         "Softsign", "Elu", "Selu", "LeakyRelu", "HardSigmoid", "HardSwish", "ThresholdedRelu", "Celu", "Mish", "Gelu",
                         "Identity", "Softmax", "LogSoftmax", "Hardmax", "CumSum", "Not", "IsNaN", "IsInf", "Shrink", "LRN",
                         "InstanceNormalization", "LpNormalization", "MeanVarianceNormalization", "Trilu", "ReverseSequence",
                         "ScatterElements", "ScatterND", "Scatter", "BitwiseNot"})
    Reg(t, "", op, 1, 5, Same);
  Reg(t, "", "Clip", 1, 3, Same);
  Reg(t, "", "Dropout", 1, 3, Same);
  Reg(t, "", "PRelu", 2, 2, Binary);
  Reg(t, "", "BatchNormalization", 5, 5, Same);
  Reg(t, "", "RMSNormalization", 2, 2, Same);
  Reg(t, "", "SimplifiedLayerNormalization", 2, 2, LayerNorm);
  Reg(t, "", "LayerNormalization", 2, 3, LayerNorm);
  Reg(t, "", "RotaryEmbedding", 3, 4, Same);
  for (const char* op : {"Add", "Sub", "Mul", "Div", "Pow", "Mod", "Min", "Max", "Sum", "Mean", "BitShift", "BitwiseAnd", "BitwiseOr", "BitwiseXor"})
    Reg(t, "", op, 1, kAny, Binary);
  for (const char* op : {"Equal", "Less", "Greater", "LessOrEqual", "GreaterOrEqual", "And", "Or", "Xor"}) Reg(t, "", op, 2, 2, Compare);
  Reg(t, "", "MatMul", 2, 2, MatMul);
  Reg(t, "", "MatMulInteger", 2, 4, [](Ctx& c) {
    // the MatMul shape rule with an int32 result
    if (c.HasShape(0) && c.HasShape(1) && c.Rank(0) >= 2 && c.Rank(1) >= 2) {
      Dims out = shape_fn::BroadcastDims(c, Dims(c.Dims(0).begin(), c.Dims(0).end() - 2), Dims(c.Dims(1).begin(), c.Dims(1).end() - 2));
      out.push_back(c.Dims(0)[c.Dims(0).size() - 2]);
      out.push_back(c.Dims(1).back());
      c.SetOutput(0, pb::INT32, out);
    } else {
      c.SetOutputType(0, pb::INT32);
    }
  });
  Reg(t, "", "Gemm", 2, 3, Gemm);
  Reg(t, "", "Transpose", 1, 1, Transpose);
  Reg(t, "", "Reshape", 2, 2, Reshape);
  Reg(t, "", "Flatten", 1, 1, Flatten);
  Reg(t, "", "Shape", 1, 1, ShapeOp);
  Reg(t, "", "Size", 1, 1, [](Ctx& c) { c.SetOutput(0, pb::INT64, {}); });
  Reg(t, "", "Gather", 2, 2, Gather);
  Reg(t, "", "GatherElements", 2, 2, [](Ctx& c) {
    if (c.Type(0) && c.HasShape(1)) c.SetOutput(0, c.ElemType(0), c.Dims(1));
  });
  Reg(t, "", "Unsqueeze", 1, 2, Unsqueeze);
  Reg(t, "", "Squeeze", 1, 2, Squeeze);
  Reg(t, "", "Concat", 1, kAny, Concat);
  Reg(t, "", "Split", 1, 2, Split);
  Reg(t, "", "Slice", 1, 5, Slice);
  Reg(t, "", "Cast", 1, 1, Cast);
  Reg(t, "", "CastLike", 2, 2, [](Ctx& c) {
    if (c.Type(0) && c.Type(1)) {
      if (c.HasShape(0)) c.SetOutput(0, c.ElemType(1), c.Dims(0));
      else c.SetOutputType(0, c.ElemType(1));
    }
  });
  Reg(t, "", "Where", 3, 3, Where);
  Reg(t, "", "Expand", 2, 2, Expand);
  Reg(t, "", "Tile", 2, 2, [](Ctx& c) {
    std::vector<int64_t> reps;
    if (c.HasShape(0) && Ints(c, 1, &reps) && reps.size() == c.Dims(0).size()) {
      Dims out = c.Dims(0);
      for (size_t i = 0; i < out.size(); ++i) out[i] = out[i].has_value ? Known(out[i].value * reps[i]) : (reps[i] == 1 ? out[i] : c.FreshDim());
      c.SetOutput(0, c.ElemType(0), out);
    } else if (c.Type(0)) {
      c.SetOutputType(0, c.ElemType(0));
    }
  });
  for (const char* op : {"ReduceSum", "ReduceMean", "ReduceMax", "ReduceMin", "ReduceProd", "ReduceL1", "ReduceL2", "ReduceLogSum",
                         "ReduceLogSumExp", "ReduceSumSquare", "ArgMax", "ArgMin"})
    Reg(t, "", op, 1, 2, Reduce);
  Reg(t, "", "Constant", 0, 0, ConstantOp);
  Reg(t, "", "ConstantOfShape", 1, 1, ConstantOfShape);
  Reg(t, "", "Range", 3, 3, [](Ctx& c) {
    std::vector<int64_t> s, l, d;
    if (c.Type(0)) {
      if (Ints(c, 0, &s) && Ints(c, 1, &l) && Ints(c, 2, &d) && s.size() == 1 && l.size() == 1 && d.size() == 1 && d[0] != 0)
        c.SetOutput(0, c.ElemType(0), {Known(std::max<int64_t>(0, (l[0] - s[0] + d[0] - (d[0] > 0 ? 1 : -1)) / d[0]))});
      else c.SetOutput(0, c.ElemType(0), {c.FreshDim()});
    }
  });
  Reg(t, "", "Conv", 2, 3, [](Ctx& c) { ConvLike(c, true); });
  Reg(t, "", "MaxPool", 1, 1, [](Ctx& c) { ConvLike(c, false); });
  Reg(t, "", "AveragePool", 1, 1, [](Ctx& c) { ConvLike(c, false); });
  Reg(t, "", "GlobalAveragePool", 1, 1, GlobalPool);
  Reg(t, "", "GlobalMaxPool", 1, 1, GlobalPool);
  Reg(t, "", "TopK", 1, 2, TopK);
  Reg(t, "", "NonZero", 1, 1, [](Ctx& c) {
    if (c.HasShape(0)) c.SetOutput(0, pb::INT64, {Known(c.Rank(0)), c.FreshDim()});
  });
  Reg(t, "", "OneHot", 3, 3, [](Ctx& c) {
    if (c.HasShape(0) && c.Type(2)) {
      Dims out = c.Dims(0);
      std::vector<int64_t> depth;
      const int64_t axis = NormAxis(c.node.attr_i("axis", -1), c.Rank(0) + 1);
      out.insert(out.begin() + axis, Ints(c, 1, &depth) && depth.size() == 1 ? Known(depth[0]) : c.FreshDim());
      c.SetOutput(0, c.ElemType(2), out);
    }
  });
  Reg(t, "", "QuantizeLinear", 2, 3, QuantizeLinear);
  Reg(t, "", "DequantizeLinear", 2, 3, DequantizeLinear);
  Reg(t, "", "Einsum", 1, kAny);
  Reg(t, "", "Pad", 1, 4);
  Reg(t, "", "Resize", 1, 4);
  Reg(t, "", "If", 1, 1);
  Reg(t, "", "Loop", 2, kAny);
  Reg(t, "", "Scan", 1, kAny);
  Reg(t, "", "Attention", 3, 6, [](Ctx& c) {  // opset-23 attention: Q [B, Nq, S, h] or [B, S, Nq h]
    c.PassThrough(0, 0);
  });

  // ---- com.microsoft
  for (const char* op : {"FastGelu", "BiasGelu", "Gelu", "QuickGelu", "BiasSoftmax", "BiasDropout", "GemmaRotaryEmbedding", "RotaryEmbedding",
                         "MRotaryEmbedding", "GatedAdd", "GatedRMSNorm", "Inverse", "Trilu", "SimplifiedLayerNormalization"})
    Reg(t, MS, op, 1, 6, Same);
  Reg(t, MS, "LayerNormalization", 2, 3, LayerNorm);
  Reg(t, MS, "SkipLayerNormalization", 3, 5, SkipLayerNorm);
  Reg(t, MS, "SkipSimplifiedLayerNormalization", 3, 4, SkipLayerNorm);
  Reg(t, MS, "EmbedLayerNormalization", 7, 9, EmbedLayerNorm);
  Reg(t, MS, "Attention", 2, 7, BertAttention);
  Reg(t, MS, "MultiHeadAttention", 1, 10, MultiHeadAttention);
  Reg(t, MS, "GroupQueryAttention", 7, 16, GroupQueryAttention);
  Reg(t, MS, "PagedAttention", 5, 12, [](Ctx& c) {
    if (!c.HasShape(0) || c.Rank(0) != 2) return;
    Dims out = c.Dims(0);
    const int64_t N = c.node.attr_i("num_heads", 0), Nk = c.node.attr_i("kv_num_heads", 0);
    if (!c.node.has_input(1) && out[1].has_value && N > 0) out[1] = Known(out[1].value / (N + 2 * Nk) * N);
    c.SetOutput(0, c.ElemType(0), out);
  });
  Reg(t, MS, "MatMulNBits", 3, 7, MatMulNBits);  // input 6: residual added by this runtime's GPU lowering
  Reg(t, MS, "FusedMatMul", 2, 2, FusedMatMul);
  Reg(t, MS, "TransposeMatMul", 2, 2, FusedMatMul);
  Reg(t, MS, "GemmFloat8", 2, 6, GemmFloat8);
  Reg(t, MS, "MoE", 5, 8, Same);
  Reg(t, MS, "QMoE", 7, 14, Same);
  Reg(t, MS, "ShardedMoE", 5, 8, Same);
  Reg(t, MS, "AllReduce", 1, 1, Same);
  Reg(t, MS, "AllToAll", 1, 1, Same);
  Reg(t, MS, "AllGather", 1, 1, AllGatherOp);
  Reg(t, MS, "QuantizeLinear", 2, 3, QuantizeLinear);
  Reg(t, MS, "DequantizeLinear", 2, 3, DequantizeLinear);
  Reg(t, MS, "DistributedMatMul", 2, 2);
  Reg(t, MS, "RemovePadding", 2, 2);
  Reg(t, MS, "RestorePadding", 2, 2);
  Reg(t, MS, "PackedAttention", 5, 6);
  Reg(t, MS, "PackedMultiHeadAttention", 6, 8);
  Reg(t, MS, "BeamSearch", 5, 12);
  Reg(t, MS, "GreedySearch", 2, 7);
  Reg(t, MS, "Sampling", 2, 9);
  Reg(t, MS, "WhisperBeamSearch", 5, 15);
  Reg(t, MS, "DecoderMaskedMultiHeadAttention", 1, 14, [](Ctx& c) { c.PassThrough(0, 0); });
  // third / fourth batch of contrib operators: arity checks for all, shape functions where the output follows an input
  Reg(t, MS, "DecoderMaskedSelfAttention", 3, 10, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "LongformerAttention", 7, 7, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "SparseAttention", 9, 11, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "MRotaryEmbedding", 4, 4, Same);
  Reg(t, MS, "LinearAttentionGate", 3, 4, Same);
  Reg(t, MS, "CausalConvWithState", 2, 4, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "LinearAttention", 3, 6);
  Reg(t, MS, "GatedRelativePositionBias", 6, 7);
  Reg(t, MS, "FusedConv", 2, 4, [](Ctx& c) { ConvLike(c, true); });
  Reg(t, MS, "NhwcConv", 2, 3);
  Reg(t, MS, "NhwcFusedConv", 2, 4);
  Reg(t, MS, "NhwcMaxPool", 1, 1);
  Reg(t, MS, "ConvTransposeWithDynamicPads", 2, 4);
  Reg(t, MS, "FusedMatMulActivation", 2, 2, FusedMatMul);
  Reg(t, MS, "GemmFastGelu", 2, 3, MatMul);
  Reg(t, MS, "MaxpoolWithMask", 2, 2);
  Reg(t, MS, "ExpandDims", 2, 2);
  Reg(t, MS, "IsAllFinite", 1, 1 << 20);
  Reg(t, MS, "CDist", 2, 2);
  Reg(t, MS, "MurmurHash3", 1, 1);
  Reg(t, MS, "CropAndResize", 4, 4);
  Reg(t, MS, "SampleOp", 1, 1, Same);
  Reg(t, MS, "ShrunkenGather", 2, 2, Gather);
  Reg(t, MS, "TorchEmbedding", 2, 4);
  Reg(t, MS, "BitmaskBiasDropout", 2, 5, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "QLinearAveragePool", 4, 5);
  Reg(t, MS, "QLinearGlobalAveragePool", 4, 5);
  Reg(t, MS, "QLinearConcat", 5, 1 << 20);
  Reg(t, MS, "QLinearSoftmax", 4, 5, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "QLinearConvTranspose", 8, 9);
  Reg(t, MS, "QLinearReduceMean", 4, 5);
  Reg(t, MS, "QLinearWhere", 9, 9);
  Reg(t, MS, "MulInteger", 3, 4);
  Reg(t, MS, "ReduceSumInteger", 1, 1);
  Reg(t, MS, "MatMulInteger16", 2, 2);
  Reg(t, MS, "QAttention", 5, 9);
  Reg(t, MS, "QEmbedLayerNormalization", 13, 18);
  Reg(t, MS, "MatMulBlockQuantizedFp4Weight", 4, 6);
  Reg(t, MS, "DynamicQuantizeLSTM", 12, 12);
  Reg(t, MS, "MatMulNBitsMlp", 8, 9);
  Reg(t, MS, "MatMulNBitsQkv", 11, 12);
  Reg(t, MS, "DecoderAttention", 12, 12, [](Ctx& c) { c.PassThrough(0, 0); });
  Reg(t, MS, "BifurcationDetector", 3, 4);

  // ---- this runtime's fused operators
  Reg(t, FUSED, "FusedGemm", 2, 5, FusedGemm);
  Reg(t, FUSED, "GemmSwiGLU", 3, 4, FusedGemm);
  Reg(t, FUSED, "SwiGLU", 1, 1, [](Ctx& c) {
    if (!c.HasShape(0) || c.Rank(0) < 1) return;
    Dims out = c.Dims(0);
    out.back() = out.back().has_value ? Known(out.back().value / 2) : c.FreshDim();
    c.SetOutput(0, c.ElemType(0), out);
  });
}

}  // namespace ortb
