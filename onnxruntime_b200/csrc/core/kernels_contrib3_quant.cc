// com.microsoft quantised operators: the QLinear* family beyond Add / Mul / Conv / MatMul, integer arithmetic
// helpers, QAttention, QEmbedLayerNormalization and the NVFP4 weight-only MatMul.  Each QLinear operator is
// "dequantise, apply the float operator, requantise with round-half-to-even and saturation", which is what the
// reference's CPU kernels compute (onnxruntime/contrib_ops/cpu/quantization/*.cc).
#include <ATen/ATen.h>

#include <cmath>
#include <limits>

#include "contrib_math.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

at::Tensor Dq(const at::Tensor& x, const at::Tensor& scale, const at::Tensor* zp) {
  at::Tensor f = x.to(at::kFloat);
  if (zp != nullptr && zp->defined()) f = f - zp->to(at::kFloat);
  return f * scale.to(at::kFloat);
}

at::Tensor Dq(Ctx& ctx, int xi, int si, int zi) {
  at::Tensor zp = ctx.HasInput(zi) ? ctx.Input(zi) : at::Tensor();
  return Dq(ctx.RequiredInput(xi), ctx.RequiredInput(si), &zp);
}

at::Tensor Qz(const at::Tensor& y, const at::Tensor& scale, const at::Tensor& zp, at::ScalarType dtype) {
  double lo = 0, hi = 255;
  if (dtype == at::kChar) { lo = -128; hi = 127; }
  at::Tensor q = at::round(y / scale.to(at::kFloat));
  if (zp.defined()) q = q + zp.to(at::kFloat);
  return at::clamp(q, lo, hi).to(dtype);
}

// output type = type of the output zero point when present, else of the (first) quantised input
at::ScalarType OutType(Ctx& ctx, int zp_index, int x_index) {
  return ctx.HasInput(zp_index) ? ctx.Input(zp_index).scalar_type() : ctx.RequiredInput(x_index).scalar_type();
}

at::Tensor OptT(Ctx& ctx, int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); }

// QLinearAveragePool / QLinearGlobalAveragePool: X, x_scale, x_zp, y_scale, y_zp; channels_last = 1 means N...C.
void QLinearPoolImpl(Ctx& ctx, bool global) {
  const bool nhwc = ctx.node().attr_i("channels_last", 0) != 0;
  at::Tensor x = Dq(ctx, 0, 1, 2);
  if (nhwc) x = x.movedim(-1, 1);
  at::Tensor y;
  if (global) {
    std::vector<int64_t> dims;
    for (int64_t d = 2; d < x.dim(); ++d) dims.push_back(d);
    y = x.mean(dims, true);
  } else {
    y = PoolWithNodeAttrs(ctx.node(), x.contiguous(), false);
  }
  if (nhwc) y = y.movedim(1, -1);
  ctx.SetOutput(0, Qz(y, ctx.RequiredInput(3), OptT(ctx, 4), OutType(ctx, 4, 0)).contiguous());
}

void QLinearConcatImpl(Ctx& ctx) {
  std::vector<at::Tensor> parts;
  for (int i = 2; i + 2 < ctx.InputCount() + 1 && i < ctx.InputCount(); i += 3) {
    at::Tensor zp = OptT(ctx, i + 2);
    parts.push_back(Dq(ctx.RequiredInput(i), ctx.RequiredInput(i + 1), &zp));
  }
  ORTB_ENFORCE_ARG(!parts.empty(), "QLinearConcat needs at least one (tensor, scale, zero point) triple");
  int64_t axis = ctx.node().attr_i("axis", 0);
  if (axis < 0) axis += parts[0].dim();
  ctx.SetOutput(0, Qz(at::cat(parts, axis), ctx.RequiredInput(0), OptT(ctx, 1), OutType(ctx, 1, 2)));
}

void QLinearSoftmaxImpl(Ctx& ctx) {
  at::Tensor x = Dq(ctx, 0, 1, 2);
  const int64_t opset = ctx.node().attr_i("opset", 13);
  int64_t axis = ctx.node().attr_i("axis", opset < 13 ? 1 : -1);
  if (axis < 0) axis += x.dim();
  at::Tensor y;
  if (opset < 13) {  // the tensor is coerced to 2-D at `axis`
    int64_t rows = 1;
    for (int64_t d = 0; d < axis; ++d) rows *= x.size(d);
    y = at::softmax(x.reshape({rows, -1}), 1).reshape(x.sizes());
  } else {
    y = at::softmax(x, axis);
  }
  ctx.SetOutput(0, Qz(y, ctx.RequiredInput(3), OptT(ctx, 4), OutType(ctx, 4, 0)));
}

// QLinearConvTranspose: x, x_scale, x_zp, w, w_scale, w_zp, y_scale, y_zp, bias (int32, scale x_scale * w_scale)
void QLinearConvTransposeImpl(Ctx& ctx) {
  at::Tensor x = Dq(ctx, 0, 1, 2);
  at::Tensor w_scale = ctx.RequiredInput(4).to(at::kFloat), w_zp = OptT(ctx, 5);
  at::Tensor wq = ctx.RequiredInput(3).to(at::kFloat);
  // a per-channel filter scale runs along the output channels, which is dim 1 (per group) of a ConvTranspose filter
  auto along_out = [&](const at::Tensor& t) {
    if (t.numel() == 1) return t.reshape({1});
    std::vector<int64_t> shape(wq.dim(), 1);
    shape[1] = t.numel();
    return t.reshape(shape);
  };
  at::Tensor w = wq;
  if (w_zp.defined()) w = w - along_out(w_zp.to(at::kFloat));
  w = w * along_out(w_scale);
  c10::optional<at::Tensor> bias;
  if (ctx.HasInput(8)) bias = ctx.Input(8).to(at::kFloat) * ctx.RequiredInput(1).to(at::kFloat) * w_scale.reshape({-1});
  at::Tensor y = ConvTransposeWithNodeAttrs(ctx.node(), x, w, bias);
  ctx.SetOutput(0, Qz(y, ctx.RequiredInput(6), OptT(ctx, 7), OutType(ctx, 7, 0)));
}

// QAttention (contrib_ops/cpu/quantization/attention_quant.cc): input and weight are 8-bit, the projection result is
// scaled by input_scale * weight_scale (a scalar or one per column), everything after it is the float Attention.
void QAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& xq = ctx.RequiredInput(0);
  const at::Tensor& wq = ctx.RequiredInput(1);
  const int64_t B = xq.size(0), S = xq.size(1), N = n.attr_i("num_heads", 1);
  at::Tensor x = xq.to(at::kFloat), w = wq.to(at::kFloat);
  if (ctx.HasInput(6)) x = x - ctx.Input(6).to(at::kFloat);
  if (ctx.HasInput(7)) w = w - ctx.Input(7).to(at::kFloat).reshape({1, -1});
  at::Tensor qkv = at::matmul(x, w) * (ctx.RequiredInput(3).to(at::kFloat) * ctx.RequiredInput(4).to(at::kFloat).reshape({1, -1}));
  qkv = qkv + ctx.RequiredInput(2).to(at::kFloat);
  const int64_t hidden = qkv.size(-1) / 3, H = hidden / N;
  at::Tensor q = qkv.narrow(-1, 0, hidden).reshape({B, S, N, H}).transpose(1, 2);
  at::Tensor k = qkv.narrow(-1, hidden, hidden).reshape({B, S, N, H}).transpose(1, 2);
  at::Tensor v = qkv.narrow(-1, 2 * hidden, hidden).reshape({B, S, N, H}).transpose(1, 2);
  if (ctx.HasInput(8)) {
    const at::Tensor past = ctx.Input(8).to(at::kFloat);  // [2, B, N, P, H]
    k = at::cat({past[0], k}, 2);
    v = at::cat({past[1], v}, 2);
  }
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, at::stack({k, v}, 0).contiguous());
  const int64_t T = k.size(2);
  const double scale = n.attr_f("scale", 0.f) != 0.f ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor s = at::matmul(q, k.transpose(-1, -2)) * scale;
  const float filter = n.attr_f("mask_filter_value", -10000.f);
  if (ctx.HasInput(5)) s = s + contrib::AttentionMaskBias(ctx.Input(5), B, S, T, filter, s.device());
  if (n.attr_i("unidirectional", 0)) {
    at::Tensor causal = at::ones({S, T}, s.options().dtype(at::kBool)).tril(T - S);
    s = s.masked_fill(causal.logical_not(), filter);
  }
  at::Tensor y = at::matmul(at::softmax(s, -1), v);
  ctx.SetOutput(0, y.transpose(1, 2).reshape({B, S, hidden}).contiguous());
}

// QEmbedLayerNormalization (contrib_ops/cpu/quantization/qembed_layer_norm.cc): the three embedding tables, gamma and
// beta are 8-bit with one scale / zero point each (inputs 8 - 17); the output is float.
void QEmbedLayerNormImpl(Ctx& ctx) {
  at::Tensor ids = ctx.RequiredInput(0).to(at::kLong);
  const int64_t B = ids.size(0), S = ids.size(1);
  auto table = [&](int qi, int si, int zi) {
    at::Tensor zp = OptT(ctx, zi);
    return Dq(ctx.RequiredInput(qi), ctx.RequiredInput(si), &zp);
  };
  at::Tensor word = table(2, 8, 13), pos = table(3, 9, 14);
  at::Tensor e = at::embedding(word, ids) + pos.narrow(0, 0, S).unsqueeze(0);
  if (ctx.HasInput(1) && ctx.HasInput(4)) e = e + at::embedding(table(4, 10, 15), ctx.Input(1).to(at::kLong));
  at::Tensor gamma = table(5, 11, 16), beta = table(6, 12, 17);
  const double eps = ctx.node().attr_f("epsilon", 1e-12f);
  ctx.SetOutput(0, at::layer_norm(e, {e.size(-1)}, gamma, beta, eps));
  if (ctx.OutputCount() > 1) {
    at::Tensor mask_index = ctx.HasInput(7) ? ctx.Input(7).to(at::kLong).ne(0).sum(1).to(at::kInt)
                                            : at::zeros({B}, at::TensorOptions().dtype(at::kInt).device(ids.device()));
    ctx.SetOutput(1, mask_index);
  }
}

// E2M1 (sign, 2 exponent bits, 1 mantissa bit): 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives
at::Tensor E2m1ToFloat(const at::Tensor& nibbles) {
  at::Tensor lut = at::tensor({0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f},
                              at::TensorOptions().dtype(at::kFloat)).to(nibbles.device());
  return lut.index_select(0, nibbles.reshape({-1}).to(at::kLong)).reshape(nibbles.sizes());
}

// MatMulBlockQuantizedFp4Weight: B [N, K/2] packed E2M1 (low nibble first), weight_scale [N, ceil(K / block)] raw E4M3
// bytes, weight_scale_2 global fp32 scale; Y = A @ dequant(B)^T + bias.
void MatMulFp4Impl(Ctx& ctx) {
  const at::Tensor& a = ctx.RequiredInput(0);
  at::Tensor packed = ctx.RequiredInput(1).to(at::kInt);
  const int64_t N = packed.size(0), K = 2 * packed.size(1), block = ctx.node().attr_i("block_size", 16);
  at::Tensor nib = at::stack({packed.bitwise_and(0xF), packed.bitwise_right_shift(4).bitwise_and(0xF)}, -1).reshape({N, K});
  at::Tensor w = E2m1ToFloat(nib);
  at::Tensor sc = ctx.RequiredInput(2).contiguous().view(at::kFloat8_e4m3fn).to(at::kFloat);  // [N, blocks]
  sc = sc.repeat_interleave(block, 1).narrow(1, 0, K);
  w = w * sc * ctx.RequiredInput(3).to(at::kFloat).reshape({});
  at::Tensor y = at::matmul(a.to(at::kFloat), w.t());
  if (ctx.HasInput(5)) y = y + ctx.Input(5).to(at::kFloat);
  ctx.SetOutput(0, y.to(a.scalar_type()));
}

}  // namespace

void RegisterContribKernels3Quant(KernelRegistry& r) {
  r.RegisterFn(MS, "QLinearAveragePool", 1, kMax, [](Ctx& ctx) { QLinearPoolImpl(ctx, false); });
  r.RegisterFn(MS, "QLinearGlobalAveragePool", 1, kMax, [](Ctx& ctx) { QLinearPoolImpl(ctx, true); });
  r.RegisterFn(MS, "QLinearConcat", 1, kMax, QLinearConcatImpl);
  r.RegisterFn(MS, "QLinearSoftmax", 1, kMax, QLinearSoftmaxImpl);
  r.RegisterFn(MS, "QLinearConvTranspose", 1, kMax, QLinearConvTransposeImpl);
  r.RegisterFn(MS, "QLinearReduceMean", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = Dq(ctx, 0, 1, 2);
    std::vector<int64_t> axes = ctx.node().attr_ints("axes");
    if (axes.empty()) for (int64_t d = 0; d < x.dim(); ++d) axes.push_back(d);
    at::Tensor y = x.mean(axes, ctx.node().attr_i("keepdims", 1) != 0);
    ctx.SetOutput(0, Qz(y, ctx.RequiredInput(3), OptT(ctx, 4), OutType(ctx, 4, 0)));
  });
  r.RegisterFn(MS, "QLinearWhere", 1, kMax, [](Ctx& ctx) {
    at::Tensor y = at::where(ctx.RequiredInput(0).to(at::kBool), Dq(ctx, 1, 2, 3), Dq(ctx, 4, 5, 6));
    ctx.SetOutput(0, Qz(y, ctx.RequiredInput(7), OptT(ctx, 8), OutType(ctx, 8, 1)));
  });
  r.RegisterFn(MS, "MulInteger", 1, kMax, [](Ctx& ctx) {
    at::Tensor a = ctx.RequiredInput(0).to(at::kInt), b = ctx.RequiredInput(2).to(at::kInt);
    if (ctx.HasInput(1)) a = a - ctx.Input(1).to(at::kInt);
    if (ctx.HasInput(3)) b = b - ctx.Input(3).to(at::kInt);
    ctx.SetOutput(0, a * b);
  });
  r.RegisterFn(MS, "ReduceSumInteger", 1, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0).to(at::kInt);
    std::vector<int64_t> axes = ctx.node().attr_ints("axes");
    if (axes.empty()) for (int64_t d = 0; d < x.dim(); ++d) axes.push_back(d);
    ctx.SetOutput(0, x.sum(axes, ctx.node().attr_i("keepdims", 1) != 0).to(at::kInt));
  });
  r.RegisterFn(MS, "MatMulInteger16", 1, kMax, [](Ctx& ctx) {
    // int16 x int16 -> int32; 64-bit accumulation on the host path keeps the products exact
    at::Tensor y = at::matmul(ctx.RequiredInput(0).to(at::kCPU, at::kLong), ctx.RequiredInput(1).to(at::kCPU, at::kLong));
    ctx.SetOutput(0, y.to(at::kInt).to(ctx.RequiredInput(0).device()));
  });
  r.RegisterFn(MS, "QAttention", 1, kMax, QAttentionImpl);
  r.RegisterFn(MS, "QEmbedLayerNormalization", 1, kMax, QEmbedLayerNormImpl);
  r.RegisterFn(MS, "MatMulBlockQuantizedFp4Weight", 1, kMax, MatMulFp4Impl);
}

}  // namespace ortb
