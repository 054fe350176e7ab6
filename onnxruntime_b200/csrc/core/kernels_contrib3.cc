// com.microsoft contrib operators, third group: fused / channels-last convolutions and pools, integer and
// QLinear* arithmetic, and small utility operators.  Written against ATen, so the same code serves the CPU provider
// and CUDA tensors.  Semantics follow docs/ContribOperators.md of the reference and the kernels named beside each
// operator.
#include <ATen/ATen.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>

#include "contrib_math.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

std::vector<int64_t> HostInts(const at::Tensor& t) {
  at::Tensor c = t.to(at::kCPU, at::kLong).contiguous().reshape({-1});
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

double HostScalar(const at::Tensor& t) { return t.to(at::kCPU, at::kDouble).reshape({-1})[0].item<double>(); }

c10::optional<at::Tensor> OptInput(Ctx& ctx, int i) {
  if (ctx.HasInput(i)) return ctx.Input(i);
  return c10::nullopt;
}

// Activation names of the fused operators (onnxruntime/core/providers/cpu/activation/activations.h and
// contrib_ops/cpu/fused_activation.cc): parameters come in `params` in the order alpha, beta.
at::Tensor FusedActivation(const at::Tensor& x, const std::string& name, const std::vector<float>& params) {
  auto p = [&](size_t i, float dflt) { return i < params.size() ? params[i] : dflt; };
  if (name.empty()) return x;
  if (name == "Relu") return at::relu(x);
  if (name == "Sigmoid") return at::sigmoid(x);
  if (name == "Tanh") return at::tanh(x);
  if (name == "LeakyRelu") return at::leaky_relu(x, p(0, 0.01f));
  if (name == "Clip") return at::clamp(x, p(0, -std::numeric_limits<float>::infinity()), p(1, std::numeric_limits<float>::infinity()));
  if (name == "HardSigmoid") return at::clamp(x * p(0, 0.2f) + p(1, 0.5f), 0.0, 1.0);
  if (name == "Softplus") return at::softplus(x);
  if (name == "Elu") return at::elu(x, p(0, 1.0f));
  if (name == "Gelu") return at::gelu(x);
  if (name == "Softsign") return x / (1 + x.abs());
  if (name == "ThresholdedRelu") return at::where(x > p(0, 1.0f), x, at::zeros_like(x));
  if (name == "Selu") return p(2, 1.05070102f) * at::where(x > 0, x, p(0, 1.67326319f) * (at::exp(x) - 1));
  ORTB_THROW(INVALID_ARGUMENT, "unsupported fused activation '", name, "'");
}

at::Tensor ToNchw(const at::Tensor& x) {  // N, spatial..., C -> N, C, spatial...
  return x.movedim(-1, 1).contiguous();
}
at::Tensor ToNhwc(const at::Tensor& x) { return x.movedim(1, -1).contiguous(); }

// FusedConv (contrib_ops/cpu/fused_conv.cc, contrib_ops/cuda/fused_conv.cc): Y = act(Conv(X, W, B) + Z)
void FusedConvImpl(Ctx& ctx, bool nhwc_x, bool ohwi_w) {
  at::Tensor x = ctx.RequiredInput(0), w = ctx.RequiredInput(1);
  if (nhwc_x) x = ToNchw(x);
  if (ohwi_w) w = ToNchw(w);  // (M, k..., C/g) -> (M, C/g, k...)
  at::Tensor y = ConvWithNodeAttrs(ctx.node(), x, w, OptInput(ctx, 2));
  if (ctx.HasInput(3)) y = y + (nhwc_x ? ToNchw(ctx.Input(3)) : ctx.Input(3));
  y = FusedActivation(y, ctx.node().attr_s("activation", ""), ctx.node().attr_floats("activation_params"));
  ctx.SetOutput(0, nhwc_x ? ToNhwc(y) : y);
}

at::Tensor FusedMatMulCore(Ctx& ctx) {
  const Node& n = ctx.node();
  at::Tensor a = ctx.RequiredInput(0), b = ctx.RequiredInput(1);
  if (n.attr_i("transBatchA", 0)) a = a.movedim(0, -2);
  if (n.attr_i("transBatchB", 0)) b = b.movedim(0, -2);
  if (n.attr_i("transA", 0) && a.dim() >= 2) a = a.transpose(-1, -2);
  if (n.attr_i("transB", 0) && b.dim() >= 2) b = b.transpose(-1, -2);
  at::Tensor y = at::matmul(a, b);
  const float alpha = n.attr_f("alpha", 1.f);
  return alpha == 1.f ? y : y * alpha;
}

// MaxpoolWithMask (contrib_ops/cpu/maxpool_with_mask.h): the scan of a window row stops at the first position whose
// mask is zero (flat position 0 is never tested).  Host loop: the operator is marked "for internal use".
void MaxpoolWithMaskImpl(Ctx& ctx) {
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = x_in.to(at::kCPU, at::kFloat).contiguous();
  at::Tensor m = ctx.RequiredInput(1).to(at::kCPU, at::kInt).contiguous();
  const Node& n = ctx.node();
  const int64_t nd = x.dim() - 2;
  ORTB_ENFORCE_ARG(nd == 1 || nd == 2, "MaxpoolWithMask supports 1-D and 2-D pooling");
  std::vector<int64_t> k = n.attr_ints("kernel_shape"), st = n.attr_ints("strides"), pads = n.attr_ints("pads");
  if (st.empty()) st.assign(nd, 1);
  if (pads.empty()) pads.assign(2 * nd, 0);
  // 1-D pooling runs as a single row, so that the scan that stops at a masked element is the innermost loop
  const int64_t N = x.size(0), C = x.size(1), H = nd == 2 ? x.size(2) : 1, W = nd == 2 ? x.size(3) : x.size(2);
  const int64_t kh = nd == 2 ? k[0] : 1, kw = nd == 2 ? k[1] : k[0], sh = nd == 2 ? st[0] : 1, sw = nd == 2 ? st[1] : st[0];
  const int64_t ph = nd == 2 ? pads[0] : 0, pw = nd == 2 ? pads[1] : pads[0];
  const int64_t pe_h = nd == 2 ? pads[2] : 0, pe_w = nd == 2 ? pads[3] : pads[1];
  const int64_t OH = (H + ph + pe_h - kh) / sh + 1, OW = (W + pw + pe_w - kw) / sw + 1;
  const int64_t first_tested = nd == 2 ? 1 : 0;  // the 2-D kernel of the reference never tests flat position 0
  at::Tensor y = at::empty(nd == 2 ? std::vector<int64_t>{N, C, OH, OW} : std::vector<int64_t>{N, C, OW}, x.options());
  const float* xd = x.data_ptr<float>();
  const int32_t* md = m.data_ptr<int32_t>();
  float* yd = y.data_ptr<float>();
  const int64_t plane = H * W, mask_planes = m.numel() / plane;
  for (int64_t c = 0; c < N * C; ++c) {
    const float* xp = xd + c * plane;
    const int32_t* mp = md + (c % mask_planes) * plane;
    for (int64_t oh = 0; oh < OH; ++oh) {
      for (int64_t ow = 0; ow < OW; ++ow) {
        const int64_t h0 = std::max<int64_t>(oh * sh - ph, 0), h1 = std::min(oh * sh - ph + kh, H);
        const int64_t w0 = std::max<int64_t>(ow * sw - pw, 0), w1 = std::min(ow * sw - pw + kw, W);
        float best = std::numeric_limits<float>::lowest();
        for (int64_t h = h0; h < h1; ++h) {
          for (int64_t w = w0; w < w1; ++w) {
            const int64_t idx = h * W + w;
            if (idx >= first_tested && mp[idx] == 0) break;
            best = std::max(best, xp[idx]);
          }
        }
        yd[(c * OH + oh) * OW + ow] = best;
      }
    }
  }
  ctx.SetOutput(0, y.to(x_in.device(), x_in.scalar_type()));
}

// MurmurHash3 x86 32-bit (public-domain algorithm by Austin Appleby) over the bytes of one element.
uint32_t Murmur3(const uint8_t* data, int len, uint32_t seed) {
  auto rotl = [](uint32_t v, int r) { return (v << r) | (v >> (32 - r)); };
  uint32_t h = seed;
  const int nblocks = len / 4;
  for (int i = 0; i < nblocks; ++i) {
    uint32_t k;
    std::memcpy(&k, data + 4 * i, 4);
    k *= 0xcc9e2d51u;
    k = rotl(k, 15);
    k *= 0x1b873593u;
    h ^= k;
    h = rotl(h, 13);
    h = h * 5 + 0xe6546b64u;
  }
  const uint8_t* tail = data + 4 * nblocks;
  uint32_t k = 0;
  switch (len & 3) {
    case 3: k ^= static_cast<uint32_t>(tail[2]) << 16; [[fallthrough]];
    case 2: k ^= static_cast<uint32_t>(tail[1]) << 8; [[fallthrough]];
    case 1:
      k ^= tail[0];
      k *= 0xcc9e2d51u;
      k = rotl(k, 15);
      k *= 0x1b873593u;
      h ^= k;
  }
  h ^= static_cast<uint32_t>(len);
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}

void MurmurHash3Impl(Ctx& ctx) {
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = x_in.to(at::kCPU).contiguous();
  const uint32_t seed = static_cast<uint32_t>(ctx.node().attr_i("seed", 0));
  const bool positive = ctx.node().attr_i("positive", 1) != 0;
  const int es = static_cast<int>(x.element_size());
  const uint8_t* bytes = static_cast<const uint8_t*>(x.data_ptr());
  at::Tensor out = at::empty(x.sizes(), at::TensorOptions().dtype(at::kInt));
  int32_t* o = out.data_ptr<int32_t>();
  for (int64_t i = 0; i < x.numel(); ++i) {
    const uint32_t h = Murmur3(bytes + i * es, es, seed);
    std::memcpy(o + i, &h, 4);
  }
  // positive = 1: the result is an unsigned 32-bit number (held in 64 bits here, ATen's uint32 support is partial)
  if (positive) out = out.to(at::kLong).bitwise_and(0xffffffffLL);
  ctx.SetOutput(0, out.to(x_in.device()));
}

// CropAndResize (contrib_ops/cpu/crop_and_resize.cc): TensorFlow-style crop of normalised boxes [y1, x1, y2, x2] from
// image batch_indices[i], resized to crop_size with bilinear or nearest sampling; samples outside the image take
// extrapolation_value.
void CropAndResizeImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  at::Tensor rois = ctx.RequiredInput(1).to(at::kFloat);
  at::Tensor bidx = ctx.RequiredInput(2).to(at::kLong);
  const std::vector<int64_t> cs = HostInts(ctx.RequiredInput(3));
  ORTB_ENFORCE_ARG(cs.size() == 2, "CropAndResize: crop_size must hold two values");
  const int64_t ch = cs[0], cw = cs[1], H = x.size(2), W = x.size(3), R = rois.size(0);
  const std::string mode = ctx.node().attr_s("mode", "bilinear");
  const float extra = ctx.node().attr_f("extrapolation_value", 0.f);
  auto fopt = at::TensorOptions().dtype(at::kFloat).device(x.device());
  at::Tensor y1 = rois.select(1, 0), x1 = rois.select(1, 1), y2 = rois.select(1, 2), x2 = rois.select(1, 3);
  auto coords = [&](const at::Tensor& lo, const at::Tensor& hi, int64_t crop, int64_t size) {
    at::Tensor t = at::arange(crop, fopt).unsqueeze(0);  // [1, crop]
    if (crop > 1) {
      at::Tensor scale = (hi - lo) * static_cast<double>(size - 1) / static_cast<double>(crop - 1);
      return lo.unsqueeze(1) * static_cast<double>(size - 1) + t * scale.unsqueeze(1);
    }
    return (0.5 * (lo + hi) * static_cast<double>(size - 1)).unsqueeze(1).expand({R, 1});
  };
  at::Tensor ys = coords(y1, y2, ch, H), xs = coords(x1, x2, cw, W);       // [R, ch], [R, cw]
  at::Tensor valid = ((ys >= 0) & (ys <= static_cast<double>(H - 1))).unsqueeze(2) &
                     ((xs >= 0) & (xs <= static_cast<double>(W - 1))).unsqueeze(1);  // [R, ch, cw]
  at::Tensor img = x.index_select(0, bidx.to(x.device())).to(at::kFloat);  // [R, C, H, W]
  auto gather2 = [&](const at::Tensor& yi, const at::Tensor& xi) {           // integer [R, ch], [R, cw] -> [R, C, ch, cw]
    at::Tensor yy = yi.clamp(0, H - 1), xx = xi.clamp(0, W - 1);
    at::Tensor rows = img.gather(2, yy.reshape({R, 1, ch, 1}).expand({R, img.size(1), ch, W}));
    return rows.gather(3, xx.reshape({R, 1, 1, cw}).expand({R, img.size(1), ch, cw}));
  };
  at::Tensor out;
  if (mode == "nearest") {
    out = gather2(at::round(ys).to(at::kLong), at::round(xs).to(at::kLong));
  } else {
    at::Tensor y0 = at::floor(ys), x0 = at::floor(xs);
    at::Tensor ly = (ys - y0).reshape({R, 1, ch, 1}), lx = (xs - x0).reshape({R, 1, 1, cw});
    at::Tensor y0i = y0.to(at::kLong), x0i = x0.to(at::kLong);
    at::Tensor y1i = at::ceil(ys).to(at::kLong), x1i = at::ceil(xs).to(at::kLong);
    at::Tensor top = gather2(y0i, x0i) * (1 - lx) + gather2(y0i, x1i) * lx;
    at::Tensor bot = gather2(y1i, x0i) * (1 - lx) + gather2(y1i, x1i) * lx;
    out = top * (1 - ly) + bot * ly;
  }
  out = at::where(valid.unsqueeze(1), out, at::full({}, extra, fopt));
  ctx.SetOutput(0, out.to(x.scalar_type()));
}

}  // namespace

void RegisterContribKernels3Quant(KernelRegistry& r);

void RegisterContribKernels3(KernelRegistry& r) {
  r.RegisterFn(MS, "FusedConv", 1, kMax, [](Ctx& ctx) { FusedConvImpl(ctx, false, false); });
  r.RegisterFn(MS, "NhwcFusedConv", 1, kMax, [](Ctx& ctx) { FusedConvImpl(ctx, true, false); });
  // NhwcConv (contrib_ops/cuda/diffusion/nhwc_conv.cc): activations and filters both channels-last (M, kH, kW, C/g)
  r.RegisterFn(MS, "NhwcConv", 1, kMax, [](Ctx& ctx) { FusedConvImpl(ctx, true, true); });
  r.RegisterFn(MS, "NhwcMaxPool", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor y = PoolWithNodeAttrs(ctx.node(), ToNchw(x).to(at::kFloat), true);
    ctx.SetOutput(0, ToNhwc(y).to(x.scalar_type()));
  });
  r.RegisterFn(MS, "ConvTransposeWithDynamicPads", 1, kMax, [](Ctx& ctx) {
    std::vector<int64_t> pads;
    if (ctx.HasInput(2)) pads = HostInts(ctx.Input(2));
    ctx.SetOutput(0, ConvTransposeWithNodeAttrs(ctx.node(), ctx.RequiredInput(0), ctx.RequiredInput(1), OptInput(ctx, 3),
                                                pads.empty() ? nullptr : &pads));
  }, {2});
  r.RegisterFn(MS, "FusedMatMulActivation", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    std::vector<float> params;
    if (n.has_attr("activation_alpha")) params.push_back(n.attr_f("activation_alpha", 0.f));
    if (n.has_attr("activation_beta")) {
      if (params.empty()) params.push_back(0.f);
      params.push_back(n.attr_f("activation_beta", 0.f));
    }
    ctx.SetOutput(0, FusedActivation(FusedMatMulCore(ctx), n.attr_s("activation", ""), params));
  });
  // FusedGemm (contrib_ops/cpu/fused_gemm.cc): Gemm followed by an activation
  r.RegisterFn(MS, "FusedGemm", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    at::Tensor a = ctx.RequiredInput(0), b = ctx.RequiredInput(1);
    if (n.attr_i("transA", 0)) a = a.t();
    if (n.attr_i("transB", 0)) b = b.t();
    at::Tensor y = at::matmul(a, b) * n.attr_f("alpha", 1.f);
    if (ctx.HasInput(2)) y = y + ctx.Input(2) * n.attr_f("beta", 1.f);
    const std::vector<float> params = {n.attr_f("activation_alpha", n.attr_s("activation", "") == "LeakyRelu" ? 0.01f : (n.attr_s("activation", "") == "HardSigmoid" ? 0.2f : (n.attr_s("activation", "") == "Selu" ? 1.67326319f : 1.0f))),
                                       n.attr_f("activation_beta", 0.5f), n.attr_f("activation_gamma", 1.05070102f)};
    ctx.SetOutput(0, FusedActivation(y, n.attr_s("activation", ""), params));
  });
  r.RegisterFn(MS, "GemmFastGelu", 1, kMax, [](Ctx& ctx) {
    at::Tensor y = at::matmul(ctx.RequiredInput(0), ctx.RequiredInput(1));
    if (ctx.HasInput(2)) y = y + ctx.Input(2);
    ctx.SetOutput(0, at::gelu(y, "tanh"));
  });
  r.RegisterFn(MS, "MaxpoolWithMask", 1, kMax, MaxpoolWithMaskImpl);
  r.RegisterFn(MS, "ExpandDims", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    int64_t axis = HostInts(ctx.RequiredInput(1)).at(0);
    if (axis < 0) axis += x.dim() + 1;
    ORTB_ENFORCE_ARG(axis >= 0 && axis <= x.dim(), "ExpandDims: axis out of range");
    ctx.SetOutput(0, x.unsqueeze(axis));
  }, {1});
  r.RegisterFn(MS, "IsAllFinite", 1, kMax, [](Ctx& ctx) {
    const bool inf_only = ctx.node().attr_i("isinf_only", 0) != 0, nan_only = ctx.node().attr_i("isnan_only", 0) != 0;
    ORTB_ENFORCE_ARG(!(inf_only && nan_only), "IsAllFinite: isinf_only and isnan_only exclude each other");
    bool ok = true;
    for (int i = 0; i < ctx.InputCount() && ok; ++i) {
      if (!ctx.HasInput(i)) continue;
      const at::Tensor& t = ctx.Input(i);
      at::Tensor bad = inf_only ? at::isinf(t) : (nan_only ? at::isnan(t) : at::logical_not(at::isfinite(t)));
      ok = !bad.any().item<bool>();
    }
    ctx.SetOutput(0, at::full({}, ok ? 1 : 0, at::TensorOptions().dtype(at::kBool).device(ctx.RequiredInput(0).device())));
  });
  r.RegisterFn(MS, "CDist", 1, kMax, [](Ctx& ctx) {
    const std::string metric = ctx.node().attr_s("metric", "sqeuclidean");
    ORTB_ENFORCE_ARG(metric == "euclidean" || metric == "sqeuclidean", "CDist: metric '", metric, "' is not supported");
    at::Tensor d = at::cdist(ctx.RequiredInput(0), ctx.RequiredInput(1), 2.0, 2 /* exact pairwise differences */);
    ctx.SetOutput(0, metric == "euclidean" ? d : d * d);
  });
  r.RegisterFn(MS, "MurmurHash3", 1, kMax, MurmurHash3Impl);
  r.RegisterFn(MS, "CropAndResize", 1, kMax, CropAndResizeImpl, {3});
  r.RegisterFn(MS, "SampleOp", 1, kMax, [](Ctx& ctx) { ctx.SetOutput(0, ctx.RequiredInput(0).clone()); });
  r.RegisterFn(MS, "ShrunkenGather", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    int64_t axis = ctx.node().attr_i("axis", 0);
    if (axis < 0) axis += x.dim();
    at::Tensor idx = ctx.RequiredInput(1).to(at::kLong);
    idx = at::where(idx < 0, idx + x.size(axis), idx);
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().begin() + axis);
    shape.insert(shape.end(), idx.sizes().begin(), idx.sizes().end());
    shape.insert(shape.end(), x.sizes().begin() + axis + 1, x.sizes().end());
    ctx.SetOutput(0, x.index_select(axis, idx.reshape({-1})).reshape(shape));
  });
  r.RegisterFn(MS, "TorchEmbedding", 1, kMax, [](Ctx& ctx) {
    // contrib_ops: weight [V, D], indices; padding_idx and scale_grad_by_freq only matter for the gradient
    ctx.SetOutput(0, at::embedding(ctx.RequiredInput(0), ctx.RequiredInput(1).to(at::kLong)));
  }, {2, 3});
  r.RegisterFn(MS, "BitmaskBiasDropout", 1, kMax, [](Ctx& ctx) {
    // inference (training_mode false or ratio 0): data + bias (+ residual), every mask bit set
    at::Tensor y = ctx.RequiredInput(0) + ctx.RequiredInput(1);
    if (ctx.HasInput(2)) y = y + ctx.Input(2);
    const bool training = ctx.HasInput(4) && ctx.Input(4).to(at::kCPU).reshape({-1})[0].item<bool>();
    const double ratio = ctx.HasInput(3) ? HostScalar(ctx.Input(3)) : 0.5;
    ORTB_ENFORCE(!training || ratio == 0.0, "BitmaskBiasDropout: training mode is not supported by this inference engine");
    ctx.SetOutput(0, y);
    if (ctx.OutputCount() > 1) {
      const int64_t words = (y.numel() + 31) / 32;
      ctx.SetOutput(1, at::full({words}, static_cast<int64_t>(0xffffffffLL), at::TensorOptions().dtype(at::kLong).device(y.device())).to(at::kUInt32));
    }
  }, {3, 4});
  RegisterContribKernels3Quant(r);
}

}  // namespace ortb
