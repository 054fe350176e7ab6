// Neural-network ONNX operators over ATen (normalisation, convolution, pooling,
// resize, quantisation, random, opset-23 Attention / RotaryEmbedding).
// Device-agnostic; the hot transformer ops have sm_100a overrides in kernels_cuda.cc.
#include <ATen/ATen.h>

#include <cmath>
#include <numeric>

#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

std::vector<int64_t> ToVec(const at::Tensor& t) {
  at::Tensor c = t.to(at::kCPU, at::kLong).contiguous().reshape({-1});
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

int64_t NormAxis(int64_t axis, int64_t rank) {
  if (axis < 0) axis += rank;
  ORTB_ENFORCE_ARG(axis >= 0 && axis < rank, "axis out of range");
  return axis;
}

// LayerNormalization / SimplifiedLayerNormalization (RMS) with fp32 statistics.
void LayerNormImpl(Ctx& ctx, bool simplified) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const at::Tensor& scale = ctx.RequiredInput(1);
  const Node& n = ctx.node();
  const int64_t axis = NormAxis(n.attr_i("axis", -1), x.dim());
  const double eps = n.attr_f("epsilon", 1e-5f);
  std::vector<int64_t> dims;
  for (int64_t i = axis; i < x.dim(); ++i) dims.push_back(i);
  at::Tensor xf = x.to(at::kFloat);
  at::Tensor mean, inv;
  at::Tensor y;
  if (simplified) {
    at::Tensor ms = at::mean(xf * xf, dims, true);
    inv = at::rsqrt(ms + eps);
    y = xf * inv;
  } else {
    mean = at::mean(xf, dims, true);
    at::Tensor c = xf - mean;
    inv = at::rsqrt(at::mean(c * c, dims, true) + eps);
    y = c * inv;
  }
  y = y * scale.to(at::kFloat);
  if (!simplified && ctx.HasInput(2)) y = y + ctx.Input(2).to(at::kFloat);
  ctx.SetOutput(0, y.to(scale.scalar_type() == at::kFloat ? x.scalar_type() : scale.scalar_type()));
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1) && mean.defined()) ctx.SetOutput(1, mean);
  if (ctx.OutputCount() > 2 && ctx.OutputNeeded(2)) ctx.SetOutput(2, inv);
  if (simplified && ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, inv);
}

struct ConvAttrs {
  std::vector<int64_t> strides, dilations, pads_begin, pads_end, output_padding;
  int64_t group = 1;
};

ConvAttrs ParseConv(const Node& n, const at::Tensor& x, at::IntArrayRef kernel, bool transposed) {
  const int64_t nd = x.dim() - 2;
  ConvAttrs a;
  a.strides = n.attr_ints("strides");
  a.dilations = n.attr_ints("dilations");
  if (a.strides.empty()) a.strides.assign(nd, 1);
  if (a.dilations.empty()) a.dilations.assign(nd, 1);
  a.group = n.attr_i("group", 1);
  a.output_padding = n.attr_ints("output_padding");
  if (a.output_padding.empty()) a.output_padding.assign(nd, 0);
  std::vector<int64_t> pads = n.attr_ints("pads");
  const std::string auto_pad = n.attr_s("auto_pad", "NOTSET");
  a.pads_begin.assign(nd, 0);
  a.pads_end.assign(nd, 0);
  if (auto_pad == "NOTSET" || auto_pad.empty()) {
    if (!pads.empty()) {
      ORTB_ENFORCE_ARG(static_cast<int64_t>(pads.size()) == 2 * nd, "pads must have 2 * spatial rank entries");
      for (int64_t i = 0; i < nd; ++i) {
        a.pads_begin[i] = pads[i];
        a.pads_end[i] = pads[i + nd];
      }
    }
  } else if (auto_pad == "SAME_UPPER" || auto_pad == "SAME_LOWER") {
    for (int64_t i = 0; i < nd; ++i) {
      const int64_t in = x.size(2 + i);
      const int64_t eff_k = (kernel[i] - 1) * a.dilations[i] + 1;
      int64_t total;
      if (transposed) {
        total = std::max<int64_t>(0, eff_k - a.strides[i]);
      } else {
        const int64_t out = (in + a.strides[i] - 1) / a.strides[i];
        total = std::max<int64_t>(0, (out - 1) * a.strides[i] + eff_k - in);
      }
      const int64_t small = total / 2, big = total - small;
      a.pads_begin[i] = auto_pad == "SAME_UPPER" ? small : big;
      a.pads_end[i] = auto_pad == "SAME_UPPER" ? big : small;
    }
  }  // VALID: zeros
  return a;
}

bool Symmetric(const ConvAttrs& a) { return a.pads_begin == a.pads_end; }

at::Tensor PadSpatial(const at::Tensor& x, const ConvAttrs& a, double value) {
  std::vector<int64_t> tp;
  for (int64_t d = static_cast<int64_t>(a.pads_begin.size()) - 1; d >= 0; --d) {
    tp.push_back(a.pads_begin[d]);
    tp.push_back(a.pads_end[d]);
  }
  return at::constant_pad_nd(x, tp, value);
}

void ConvImpl(Ctx& ctx) {
  at::Tensor x = ctx.RequiredInput(0);
  const at::Tensor& w = ctx.RequiredInput(1);
  c10::optional<at::Tensor> bias;
  if (ctx.HasInput(2)) bias = ctx.Input(2);
  ConvAttrs a = ParseConv(ctx.node(), x, w.sizes().slice(2), false);
  std::vector<int64_t> pad = a.pads_begin;
  if (!Symmetric(a)) {
    x = PadSpatial(x, a, 0.0);
    pad.assign(pad.size(), 0);
  }
  ctx.SetOutput(0, at::convolution(x, w, bias, a.strides, pad, a.dilations, false, std::vector<int64_t>(pad.size(), 0), a.group));
}

// float convolution of already dequantised operands with the node's attributes
at::Tensor ConvFloat(const Node& node, at::Tensor x, const at::Tensor& w, const c10::optional<at::Tensor>& bias) {
  ConvAttrs a = ParseConv(node, x, w.sizes().slice(2), false);
  std::vector<int64_t> pad = a.pads_begin;
  if (!Symmetric(a)) {
    x = PadSpatial(x, a, 0.0);
    pad.assign(pad.size(), 0);
  }
  return at::convolution(x, w, bias, a.strides, pad, a.dilations, false, std::vector<int64_t>(pad.size(), 0), a.group);
}

// QLinearConv: x, x_scale, x_zp, w, w_scale (scalar or per output channel), w_zp, y_scale, y_zp, bias (int32, scale
// x_scale * w_scale).  ConvInteger: x, w, x_zp?, w_zp? -> int32.
void QLinearConvImpl(Ctx& ctx) {
  at::Tensor xf = (ctx.RequiredInput(0).to(at::kFloat) - ctx.RequiredInput(2).to(at::kFloat)) * ctx.RequiredInput(1).to(at::kFloat);
  const at::Tensor& w = ctx.RequiredInput(3);
  at::Tensor ws = ctx.RequiredInput(4).to(at::kFloat), wz = ctx.RequiredInput(5).to(at::kFloat);
  std::vector<int64_t> per_channel(w.dim(), 1);
  per_channel[0] = -1;
  if (ws.numel() > 1) ws = ws.reshape(per_channel);
  if (wz.numel() > 1) wz = wz.reshape(per_channel);
  at::Tensor wf = (w.to(at::kFloat) - wz) * ws;
  c10::optional<at::Tensor> bias;
  if (ctx.HasInput(8)) bias = ctx.Input(8).to(at::kFloat) * (ctx.RequiredInput(1).to(at::kFloat) * ctx.RequiredInput(4).to(at::kFloat).reshape({-1}));
  at::Tensor y = ConvFloat(ctx.node(), xf, wf, bias);
  const at::Tensor& yz = ctx.RequiredInput(7);
  const double lo = yz.scalar_type() == at::kChar ? -128 : 0, hi = yz.scalar_type() == at::kChar ? 127 : 255;
  ctx.SetOutput(0, at::clamp(at::round(y / ctx.RequiredInput(6).to(at::kFloat)) + yz.to(at::kFloat), lo, hi).to(yz.scalar_type()));
}

void ConvIntegerImpl(Ctx& ctx) {
  at::Tensor xf = ctx.RequiredInput(0).to(at::kFloat), wf = ctx.RequiredInput(1).to(at::kFloat);
  if (ctx.HasInput(2)) xf = xf - ctx.Input(2).to(at::kFloat);
  if (ctx.HasInput(3)) {
    at::Tensor wz = ctx.Input(3).to(at::kFloat);
    std::vector<int64_t> per_channel(wf.dim(), 1);
    per_channel[0] = -1;
    wf = wf - (wz.numel() > 1 ? wz.reshape(per_channel) : wz);
  }
  ctx.SetOutput(0, at::round(ConvFloat(ctx.node(), xf, wf, c10::nullopt)).to(at::kInt));
}

void ConvTransposeImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const at::Tensor& w = ctx.RequiredInput(1);
  c10::optional<at::Tensor> bias;
  if (ctx.HasInput(2)) bias = ctx.Input(2);
  const Node& n = ctx.node();
  ConvAttrs a = ParseConv(n, x, w.sizes().slice(2), true);
  const int64_t nd = x.dim() - 2;
  std::vector<int64_t> out_shape = n.attr_ints("output_shape");
  if (!out_shape.empty()) {
    // derive pads from the requested output shape
    const std::string auto_pad = n.attr_s("auto_pad", "NOTSET");
    for (int64_t i = 0; i < nd; ++i) {
      const int64_t eff_k = (w.size(2 + i) - 1) * a.dilations[i] + 1;
      const int64_t total = a.strides[i] * (x.size(2 + i) - 1) + a.output_padding[i] + eff_k - out_shape[out_shape.size() - nd + i];
      const int64_t t = std::max<int64_t>(total, 0);
      a.pads_begin[i] = auto_pad == "SAME_UPPER" ? t / 2 : t - t / 2;
      a.pads_end[i] = t - a.pads_begin[i];
    }
  }
  // torch takes symmetric padding; realise asymmetric pads by cropping an unpadded result
  std::vector<int64_t> zero(nd, 0);
  if (Symmetric(a)) {
    ctx.SetOutput(0, at::convolution(x, w, bias, a.strides, a.pads_begin, a.dilations, true, a.output_padding, a.group));
  } else {
    at::Tensor y = at::convolution(x, w, bias, a.strides, zero, a.dilations, true, a.output_padding, a.group);
    for (int64_t i = 0; i < nd; ++i) y = y.narrow(2 + i, a.pads_begin[i], y.size(2 + i) - a.pads_begin[i] - a.pads_end[i]);
    ctx.SetOutput(0, y.contiguous());
  }
}

void PoolImpl(Ctx& ctx, bool is_max) {
  at::Tensor x = ctx.RequiredInput(0);
  const Node& n = ctx.node();
  std::vector<int64_t> kernel = n.attr_ints("kernel_shape");
  const int64_t nd = x.dim() - 2;
  ORTB_ENFORCE_ARG(static_cast<int64_t>(kernel.size()) == nd, "kernel_shape rank mismatch");
  ConvAttrs a = ParseConv(n, x, kernel, false);
  const bool ceil_mode = n.attr_i("ceil_mode", 0) != 0;
  std::vector<int64_t> pad = a.pads_begin;
  const bool include_pad = n.attr_i("count_include_pad", 0) != 0;
  if (!Symmetric(a)) {
    ORTB_ENFORCE_ARG(is_max || include_pad, "AveragePool with asymmetric pads requires count_include_pad=1");
    x = PadSpatial(x, a, is_max ? -std::numeric_limits<double>::infinity() : 0.0);
    pad.assign(nd, 0);
  }
  if (is_max) {
    at::Tensor y, idx;
    if (nd == 1) std::tie(y, idx) = at::max_pool1d_with_indices(x, kernel, a.strides, pad, a.dilations, ceil_mode);
    else if (nd == 2) std::tie(y, idx) = at::max_pool2d_with_indices(x, kernel, a.strides, pad, a.dilations, ceil_mode);
    else if (nd == 3) std::tie(y, idx) = at::max_pool3d_with_indices(x, kernel, a.strides, pad, a.dilations, ceil_mode);
    else ORTB_NOT_IMPLEMENTED("MaxPool with ", nd, " spatial dims");
    ctx.SetOutput(0, y);
    if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) {
      // ONNX indices are flat over the whole (N, C, spatial) tensor
      int64_t plane = 1;
      for (int64_t i = 0; i < nd; ++i) plane *= ctx.RequiredInput(0).size(2 + i);
      at::Tensor nc = at::arange(x.size(0) * x.size(1), idx.options()).reshape({x.size(0), x.size(1)});
      std::vector<int64_t> vs = {x.size(0), x.size(1)};
      vs.insert(vs.end(), nd, 1);
      ctx.SetOutput(1, idx + nc.reshape(vs) * plane);
    }
  } else {
    at::Tensor y;
    if (nd == 1) y = at::avg_pool1d(x, kernel, a.strides, pad, ceil_mode, include_pad);
    else if (nd == 2) y = at::avg_pool2d(x, kernel, a.strides, pad, ceil_mode, include_pad);
    else if (nd == 3) y = at::avg_pool3d(x, kernel, a.strides, pad, ceil_mode, include_pad);
    else ORTB_NOT_IMPLEMENTED("AveragePool with ", nd, " spatial dims");
    ctx.SetOutput(0, y);
  }
}

void ResizeImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const Node& n = ctx.node();
  const int64_t rank = x.dim();
  std::vector<int64_t> out_size;
  std::vector<double> scales;
  const bool v10 = n.since_version < 11 || n.op_type == "Upsample";
  const int scales_idx = v10 ? 1 : 2, sizes_idx = 3;
  if (!v10 && ctx.HasInput(sizes_idx) && ctx.Input(sizes_idx).numel() > 0) {
    out_size = ToVec(ctx.Input(sizes_idx));
  } else if (ctx.HasInput(scales_idx) && ctx.Input(scales_idx).numel() > 0) {
    at::Tensor s = ctx.Input(scales_idx).to(at::kCPU, at::kDouble).contiguous();
    scales.assign(s.data_ptr<double>(), s.data_ptr<double>() + s.numel());
    for (int64_t i = 0; i < rank; ++i) out_size.push_back(static_cast<int64_t>(std::floor(x.size(i) * scales[i])));
  } else if (n.has_attr("scales")) {
    for (float f : n.attr_floats("scales")) scales.push_back(f);
    for (int64_t i = 0; i < rank; ++i) out_size.push_back(static_cast<int64_t>(std::floor(x.size(i) * scales[i])));
  } else {
    ORTB_THROW(INVALID_ARGUMENT, "Resize needs scales or sizes");
  }
  ORTB_ENFORCE_ARG(static_cast<int64_t>(out_size.size()) == rank, "Resize: sizes/scales must cover every dimension");
  ORTB_ENFORCE_ARG(rank >= 3 && out_size[0] == x.size(0) && out_size[1] == x.size(1),
                   "Resize supports resizing spatial dimensions of NCHW-style inputs only");
  std::vector<int64_t> spatial(out_size.begin() + 2, out_size.end());
  const std::string mode = n.attr_s("mode", "nearest");
  const std::string ctm = n.attr_s("coordinate_transformation_mode", v10 ? "asymmetric" : "half_pixel");
  const int64_t nd = rank - 2;
  at::Tensor y;
  if (mode == "nearest") {
    const std::string nm = n.attr_s("nearest_mode", "round_prefer_floor");
    const bool exact = (ctm == "half_pixel" || ctm == "pytorch_half_pixel") && nm != "floor";
    if (nd == 1) y = exact ? at::_upsample_nearest_exact1d(x, spatial) : at::upsample_nearest1d(x, spatial);
    else if (nd == 2) y = exact ? at::_upsample_nearest_exact2d(x, spatial) : at::upsample_nearest2d(x, spatial);
    else if (nd == 3) y = exact ? at::_upsample_nearest_exact3d(x, spatial) : at::upsample_nearest3d(x, spatial);
    else ORTB_NOT_IMPLEMENTED("Resize nearest with ", nd, " spatial dims");
  } else if (mode == "linear") {
    const bool align = ctm == "align_corners";
    ORTB_ENFORCE_ARG(align || ctm == "half_pixel" || ctm == "pytorch_half_pixel" || ctm == "asymmetric",
                     "Resize linear: unsupported coordinate_transformation_mode ", ctm);
    if (nd == 1) y = at::upsample_linear1d(x, spatial, align);
    else if (nd == 2) y = at::upsample_bilinear2d(x, spatial, align);
    else if (nd == 3) y = at::upsample_trilinear3d(x, spatial, align);
    else ORTB_NOT_IMPLEMENTED("Resize linear with ", nd, " spatial dims");
  } else if (mode == "cubic") {
    ORTB_ENFORCE_ARG(nd == 2, "Resize cubic supports 2 spatial dims");
    y = at::upsample_bicubic2d(x, spatial, ctm == "align_corners");
  } else {
    ORTB_THROW(INVALID_ARGUMENT, "Resize: unknown mode ", mode);
  }
  ctx.SetOutput(0, y);
}

at::Tensor BroadcastAlongAxis(const at::Tensor& p, int64_t axis, int64_t rank) {
  if (p.dim() != 1 || p.numel() == 1) return p;
  std::vector<int64_t> shape(rank, 1);
  shape[axis] = p.numel();
  return p.reshape(shape);
}

std::pair<double, double> QRange(at::ScalarType t) {
  switch (t) {
    case at::kByte: return {0, 255};
    case at::kChar: return {-128, 127};
    case at::kUInt16: return {0, 65535};
    case at::kShort: return {-32768, 32767};
    case at::kInt: return {-2147483648.0, 2147483647.0};
    default: return {0, 255};
  }
}

void QuantizeLinearImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const Node& n = ctx.node();
  // the axis only matters for per-axis parameters (a 1-D tensor quantised per tensor keeps the default axis 1)
  const int64_t axis = ctx.RequiredInput(1).numel() == 1 ? 0 : NormAxis(n.attr_i("axis", 1), std::max<int64_t>(x.dim(), 1));
  at::Tensor scale = BroadcastAlongAxis(ctx.RequiredInput(1).to(at::kFloat), axis, x.dim());
  at::ScalarType out_t = at::kByte;
  at::Tensor zp;
  if (ctx.HasInput(2)) {
    out_t = ctx.Input(2).scalar_type();
    zp = BroadcastAlongAxis(ctx.Input(2).to(at::kFloat), axis, x.dim());
  } else if (n.has_attr("output_dtype") && n.attr_i("output_dtype", 0) != 0) {
    out_t = ToTorchType(static_cast<int32_t>(n.attr_i("output_dtype", 2)));
  }
  at::Tensor q = x.to(at::kFloat) / scale;
  if (c10::isFloat8Type(out_t)) {
    ctx.SetOutput(0, q.to(out_t));
    return;
  }
  q = at::round(q);
  if (zp.defined()) q = q + zp;
  auto range = QRange(out_t);
  ctx.SetOutput(0, at::clamp(q, range.first, range.second).to(out_t));
}

void DequantizeLinearImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const Node& n = ctx.node();
  const at::Tensor& scale_in = ctx.RequiredInput(1);
  const int64_t axis = scale_in.numel() == 1 ? 0 : NormAxis(n.attr_i("axis", 1), std::max<int64_t>(x.dim(), 1));
  const int64_t block = n.attr_i("block_size", 0);
  at::Tensor xf = x.to(at::kFloat);
  at::Tensor scale = scale_in.to(at::kFloat);
  at::Tensor zp = ctx.HasInput(2) ? ctx.Input(2).to(at::kFloat) : at::Tensor();
  if (block > 0 && scale.dim() == x.dim()) {
    scale = scale.repeat_interleave(block, axis).narrow(axis, 0, x.size(axis));
    if (zp.defined()) zp = zp.repeat_interleave(block, axis).narrow(axis, 0, x.size(axis));
  } else {
    scale = BroadcastAlongAxis(scale, axis, x.dim());
    if (zp.defined()) zp = BroadcastAlongAxis(zp, axis, x.dim());
  }
  if (zp.defined()) xf = xf - zp;
  ctx.SetOutput(0, (xf * scale).to(scale_in.scalar_type()));
}

at::Tensor RotateHalfOrInterleaved(const at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin, bool interleaved) {
  // x: [..., rot]; cos/sin broadcastable to [..., rot/2]
  if (interleaved) {
    at::Tensor x1 = x.slice(-1, 0, c10::nullopt, 2), x2 = x.slice(-1, 1, c10::nullopt, 2);
    at::Tensor r1 = x1 * cos - x2 * sin, r2 = x2 * cos + x1 * sin;
    return at::stack({r1, r2}, -1).flatten(-2);
  }
  const int64_t half = x.size(-1) / 2;
  at::Tensor x1 = x.narrow(-1, 0, half), x2 = x.narrow(-1, half, half);
  return at::cat({x1 * cos - x2 * sin, x2 * cos + x1 * sin}, -1);
}

// ONNX-domain RotaryEmbedding (opset 23): X [B,N,S,H] or [B,S,hidden]; cos/sin caches [max_pos, rot/2]
// with position_ids [B,S], or already gathered [B,S,rot/2] without them.
void RotaryEmbedding23(Ctx& ctx) {
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor cos = ctx.RequiredInput(1), sin = ctx.RequiredInput(2);
  const Node& n = ctx.node();
  const bool interleaved = n.attr_i("interleaved", 0) != 0;
  int64_t num_heads = n.attr_i("num_heads", 0);
  at::Tensor x = x_in;
  const bool is3d = x.dim() == 3;
  if (is3d) {
    ORTB_ENFORCE_ARG(num_heads > 0, "RotaryEmbedding: num_heads is required for 3-D input");
    x = x.reshape({x.size(0), x.size(1), num_heads, x.size(2) / num_heads});  // B,S,N,H
  } else {
    x = x.permute({0, 2, 1, 3});  // B,N,S,H -> B,S,N,H
  }
  const int64_t H = x.size(3);
  int64_t rot = n.attr_i("rotary_embedding_dim", 0);
  if (rot == 0) rot = H;
  if (ctx.HasInput(3)) {
    at::Tensor pos = ctx.Input(3).to(at::kLong).to(cos.device());
    cos = cos.index({pos});
    sin = sin.index({pos});
  }
  cos = cos.unsqueeze(2).to(x.scalar_type());  // B,S,1,rot/2
  sin = sin.unsqueeze(2).to(x.scalar_type());
  at::Tensor xr = x.narrow(-1, 0, rot);
  at::Tensor y = RotateHalfOrInterleaved(xr, cos, sin, interleaved);
  if (rot < H) y = at::cat({y, x.narrow(-1, rot, H - rot)}, -1);
  if (is3d) ctx.SetOutput(0, y.reshape(x_in.sizes()));
  else ctx.SetOutput(0, y.permute({0, 2, 1, 3}).contiguous());
}

// ONNX-domain Attention (opset 23/24).
void Attention23(Ctx& ctx) {
  const Node& n = ctx.node();
  at::Tensor q = ctx.RequiredInput(0), k = ctx.RequiredInput(1), v = ctx.RequiredInput(2);
  const bool is3d = q.dim() == 3;
  const int64_t qh = n.attr_i("q_num_heads", 0), kvh = n.attr_i("kv_num_heads", 0);
  if (is3d) {
    ORTB_ENFORCE_ARG(qh > 0 && kvh > 0, "Attention: q_num_heads / kv_num_heads are required for 3-D inputs");
    q = q.reshape({q.size(0), q.size(1), qh, -1}).transpose(1, 2);
    k = k.reshape({k.size(0), k.size(1), kvh, -1}).transpose(1, 2);
    v = v.reshape({v.size(0), v.size(1), kvh, -1}).transpose(1, 2);
  }
  if (ctx.HasInput(4)) k = at::cat({ctx.Input(4), k}, 2);
  if (ctx.HasInput(5)) v = at::cat({ctx.Input(5), v}, 2);
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, k.contiguous());
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, v.contiguous());
  const int64_t N = q.size(1), Nk = k.size(1), S = q.size(2), T = k.size(2), H = q.size(3);
  at::Tensor kk = k, vv = v;
  if (N != Nk) {
    kk = k.repeat_interleave(N / Nk, 1);
    vv = v.repeat_interleave(N / Nk, 1);
  }
  const double scale = n.has_attr("scale") ? n.attr_f("scale", 1.f) : 1.0 / std::sqrt(static_cast<double>(H));
  at::Tensor s = at::matmul(q.to(at::kFloat), kk.to(at::kFloat).transpose(-1, -2)) * scale;
  const float softcap = n.attr_f("softcap", 0.f);
  if (softcap > 0.f) s = at::tanh(s / softcap) * softcap;
  if (n.attr_i("is_causal", 0)) {
    at::Tensor mask = at::ones({S, T}, s.options().dtype(at::kBool)).tril(T - S);
    s = s.masked_fill(mask.logical_not(), -std::numeric_limits<float>::infinity());
  }
  if (ctx.HasInput(3)) {
    const at::Tensor& m = ctx.Input(3);
    if (m.scalar_type() == at::kBool) s = s.masked_fill(m.logical_not(), -std::numeric_limits<float>::infinity());
    else s = s + m.to(at::kFloat);
  }
  at::Tensor p = at::softmax(s, -1);
  at::Tensor y = at::matmul(p, vv.to(at::kFloat)).to(q.scalar_type());
  if (is3d) y = y.transpose(1, 2).reshape({y.size(0), S, -1});
  ctx.SetOutput(0, y.contiguous());
}

}  // namespace

// Shared with the contrib operators that wrap a convolution or a pooling (FusedConv, NhwcConv, QLinearAveragePool ...)
at::Tensor ConvWithNodeAttrs(const Node& node, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias) {
  return ConvFloat(node, x, w, bias);
}

at::Tensor ConvTransposeWithNodeAttrs(const Node& node, const at::Tensor& x, const at::Tensor& w,
                                      const c10::optional<at::Tensor>& bias, const std::vector<int64_t>* pads_override) {
  std::vector<int64_t> kernel(w.sizes().slice(2).begin(), w.sizes().slice(2).end());
  ConvAttrs a = ParseConv(node, x, kernel, true);
  const int64_t nd = x.dim() - 2;
  if (pads_override != nullptr) {
    ORTB_ENFORCE_ARG(static_cast<int64_t>(pads_override->size()) == 2 * nd, "pads must have 2 * spatial rank entries");
    for (int64_t i = 0; i < nd; ++i) {
      a.pads_begin[i] = (*pads_override)[i];
      a.pads_end[i] = (*pads_override)[i + nd];
    }
  }
  // run without padding and crop: handles asymmetric pads uniformly
  at::Tensor y = at::convolution(x, w, bias, a.strides, std::vector<int64_t>(nd, 0), a.dilations, true, a.output_padding, a.group);
  for (int64_t i = 0; i < nd; ++i) {
    const int64_t len = y.size(2 + i) - a.pads_begin[i] - a.pads_end[i];
    ORTB_ENFORCE_ARG(len > 0, "ConvTranspose: pads remove the whole output");
    y = y.narrow(2 + i, a.pads_begin[i], len);
  }
  return y.contiguous();
}

at::Tensor PoolWithNodeAttrs(const Node& n, at::Tensor x, bool is_max) {
  std::vector<int64_t> kernel = n.attr_ints("kernel_shape");
  const int64_t nd = x.dim() - 2;
  ORTB_ENFORCE_ARG(static_cast<int64_t>(kernel.size()) == nd, "kernel_shape rank mismatch");
  ConvAttrs a = ParseConv(n, x, kernel, false);
  const bool ceil_mode = n.attr_i("ceil_mode", 0) != 0;
  const bool include_pad = n.attr_i("count_include_pad", 0) != 0;
  std::vector<int64_t> pad = a.pads_begin;
  if (!Symmetric(a)) {
    ORTB_ENFORCE_ARG(is_max || include_pad, "average pooling with asymmetric pads requires count_include_pad=1");
    x = PadSpatial(x, a, is_max ? -std::numeric_limits<double>::infinity() : 0.0);
    pad.assign(nd, 0);
  }
  if (is_max) {
    if (nd == 1) return std::get<0>(at::max_pool1d_with_indices(x, kernel, a.strides, pad, a.dilations, ceil_mode));
    if (nd == 2) return std::get<0>(at::max_pool2d_with_indices(x, kernel, a.strides, pad, a.dilations, ceil_mode));
    if (nd == 3) return std::get<0>(at::max_pool3d_with_indices(x, kernel, a.strides, pad, a.dilations, ceil_mode));
  } else {
    if (nd == 1) return at::avg_pool1d(x, kernel, a.strides, pad, ceil_mode, include_pad);
    if (nd == 2) return at::avg_pool2d(x, kernel, a.strides, pad, ceil_mode, include_pad);
    if (nd == 3) return at::avg_pool3d(x, kernel, a.strides, pad, ceil_mode, include_pad);
  }
  ORTB_NOT_IMPLEMENTED("pooling with ", nd, " spatial dims");
}

void RegisterNnKernels(KernelRegistry& r) {
  r.RegisterFn("", "LayerNormalization", 1, kMax, [](Ctx& ctx) { LayerNormImpl(ctx, false); });
  r.RegisterFn("", "SimplifiedLayerNormalization", 1, kMax, [](Ctx& ctx) { LayerNormImpl(ctx, true); });
  r.RegisterFn("", "RMSNormalization", 23, kMax, [](Ctx& ctx) { LayerNormImpl(ctx, true); });
  r.RegisterFn("", "InstanceNormalization", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::instance_norm(x, ctx.RequiredInput(1), ctx.RequiredInput(2), {}, {}, true, 0.0,
                                       ctx.node().attr_f("epsilon", 1e-5f), false));
  });
  r.RegisterFn("", "BatchNormalization", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ORTB_ENFORCE_ARG(ctx.node().attr_i("training_mode", 0) == 0, "BatchNormalization training mode is not supported");
    ctx.SetOutput(0, at::batch_norm(x, ctx.RequiredInput(1), ctx.RequiredInput(2), ctx.RequiredInput(3), ctx.RequiredInput(4),
                                    false, 0.0, ctx.node().attr_f("epsilon", 1e-5f), false));
  });
  r.RegisterFn("", "GroupNormalization", 18, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t groups = ctx.node().attr_i("num_groups", 1);
    at::Tensor scale = ctx.RequiredInput(1), bias = ctx.RequiredInput(2);
    if (scale.numel() == groups && x.size(1) != groups) {
      // opset 18 form: per-group scale/bias
      scale = scale.repeat_interleave(x.size(1) / groups);
      bias = bias.repeat_interleave(x.size(1) / groups);
    }
    ctx.SetOutput(0, at::group_norm(x, groups, scale, bias, ctx.node().attr_f("epsilon", 1e-5f), false));
  });
  r.RegisterFn("", "LpNormalization", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t axis = NormAxis(ctx.node().attr_i("axis", -1), x.dim());
    const int64_t p = ctx.node().attr_i("p", 2);
    at::Tensor norm = p == 1 ? at::sum(at::abs(x), {axis}, true) : at::sqrt(at::sum(x * x, {axis}, true));
    ctx.SetOutput(0, at::where(norm == 0, at::zeros_like(x), x / norm));
  });
  r.RegisterFn("", "LRN", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const Node& n = ctx.node();
    const int64_t size = n.attr_i("size", 1);
    const float alpha = n.attr_f("alpha", 1e-4f), beta = n.attr_f("beta", 0.75f), bias = n.attr_f("bias", 1.f);
    at::Tensor sq = (x * x).unsqueeze(1);
    const int64_t lo = (size - 1) / 2, hi = size - 1 - lo;
    std::vector<int64_t> pad(2 * (sq.dim() - 2), 0);
    pad[pad.size() - 2] = lo;
    pad[pad.size() - 1] = hi;
    at::Tensor padded = at::constant_pad_nd(sq, pad, 0);
    at::Tensor win = padded.unfold(2, size, 1).sum(-1).squeeze(1);
    ctx.SetOutput(0, x / at::pow(win * (alpha / size) + bias, beta));
  });
  r.RegisterFn("", "Conv", 1, kMax, ConvImpl);
  r.RegisterFn("", "ConvTranspose", 1, kMax, ConvTransposeImpl);
  r.RegisterFn("", "QLinearConv", 10, kMax, QLinearConvImpl);
  r.RegisterFn("", "ConvInteger", 10, kMax, ConvIntegerImpl);
  r.RegisterFn("", "MaxPool", 1, kMax, [](Ctx& ctx) { PoolImpl(ctx, true); });
  r.RegisterFn("", "AveragePool", 1, kMax, [](Ctx& ctx) { PoolImpl(ctx, false); });
  r.RegisterFn("", "GlobalAveragePool", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> dims;
    for (int64_t i = 2; i < x.dim(); ++i) dims.push_back(i);
    ctx.SetOutput(0, at::mean(x, dims, true));
  });
  r.RegisterFn("", "GlobalMaxPool", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> dims;
    for (int64_t i = 2; i < x.dim(); ++i) dims.push_back(i);
    ctx.SetOutput(0, at::amax(x, dims, true));
  });
  r.RegisterFn("", "Resize", 10, kMax, ResizeImpl, {1, 2, 3});
  r.RegisterFn("", "Upsample", 1, 9, ResizeImpl, {1});
  r.RegisterFn("", "GridSample", 16, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const std::string mode = n.attr_s("mode", "linear"), pm = n.attr_s("padding_mode", "zeros");
    const int64_t im = (mode == "nearest") ? 1 : (mode == "cubic" || mode == "bicubic") ? 2 : 0;
    const int64_t ip = pm == "border" ? 1 : pm == "reflection" ? 2 : 0;
    ctx.SetOutput(0, at::grid_sampler(ctx.RequiredInput(0), ctx.RequiredInput(1), im, ip, n.attr_i("align_corners", 0) != 0));
  });
  r.RegisterFn("", "QuantizeLinear", 10, kMax, QuantizeLinearImpl);
  r.RegisterFn("", "DequantizeLinear", 10, kMax, DequantizeLinearImpl);
  r.RegisterFn("", "DynamicQuantizeLinear", 11, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0).to(at::kFloat);
    at::Tensor mx = at::clamp_min(at::max(x), 0), mn = at::clamp_max(at::min(x), 0);
    at::Tensor scale = (mx - mn) / 255.0;
    at::Tensor safe = at::where(scale == 0, at::ones_like(scale), scale);
    at::Tensor zp = at::clamp(at::round(-mn / safe), 0, 255);
    ctx.SetOutput(0, at::clamp(at::round(x / safe) + zp, 0, 255).to(at::kByte));
    ctx.SetOutput(1, scale);
    ctx.SetOutput(2, zp.to(at::kByte));
  });
  auto random_like = [](bool normal, bool like) {
    return [normal, like](Ctx& ctx) {
      const Node& n = ctx.node();
      std::vector<int64_t> shape;
      at::ScalarType dt = at::kFloat;
      if (like) {
        const at::Tensor& x = ctx.RequiredInput(0);
        shape = x.sizes().vec();
        dt = x.scalar_type();
      } else {
        shape = n.attr_ints("shape");
      }
      if (n.has_attr("dtype")) dt = ToTorchType(static_cast<int32_t>(n.attr_i("dtype", 1)));
      c10::optional<at::Generator> gen;
      if (n.has_attr("seed")) {
        gen = at::detail::createCPUGenerator(static_cast<uint64_t>(n.attr_f("seed", 0.f)));
      }
      at::Tensor t = at::empty(shape, at::TensorOptions().dtype(at::kFloat));
      if (normal) t.normal_(n.attr_f("mean", 0.f), n.attr_f("scale", 1.f), gen);
      else t.uniform_(n.attr_f("low", 0.f), n.attr_f("high", 1.f), gen);
      ctx.SetOutput(0, t.to(dt).to(ctx.device()));
    };
  };
  r.RegisterFn("", "RandomNormal", 1, kMax, random_like(true, false));
  r.RegisterFn("", "RandomNormalLike", 1, kMax, random_like(true, true));
  r.RegisterFn("", "RandomUniform", 1, kMax, random_like(false, false));
  r.RegisterFn("", "RandomUniformLike", 1, kMax, random_like(false, true));
  r.RegisterFn("", "RotaryEmbedding", 23, kMax, RotaryEmbedding23);
  r.RegisterFn("", "Attention", 23, kMax, Attention23);
}

}  // namespace ortb
