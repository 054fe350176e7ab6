// ONNX operators: RoiAlign (opset 10 / 16), DeformConv (opset 19) and the numeric forms of ai.onnx.ml LabelEncoder.
// Reference kernels: onnxruntime/core/providers/cpu/object_detection/roialign.cc,
// core/providers/cpu/nn/deform_conv.cc, core/providers/cpu/ml/label_encoder.h.
#include <ATen/ATen.h>

#include <algorithm>
#include <cmath>
#include <limits>

#include "string_table.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

// Bilinear taps of the RoiAlign definition for sample coordinates ys [P], xs [Q] on an H x W map: samples further
// than one pixel outside contribute nothing, the rest are clamped to the border.
struct Taps {
  at::Tensor y0, y1, x0, x1, ly, lx, valid_y, valid_x;
};
Taps MakeTaps(at::Tensor ys, at::Tensor xs, int64_t H, int64_t W) {
  Taps t;
  t.valid_y = (ys >= -1.0) & (ys <= static_cast<double>(H));
  t.valid_x = (xs >= -1.0) & (xs <= static_cast<double>(W));
  ys = ys.clamp_min(0.0);
  xs = xs.clamp_min(0.0);
  t.y0 = at::floor(ys).to(at::kLong).clamp_max(H - 1);
  t.x0 = at::floor(xs).to(at::kLong).clamp_max(W - 1);
  t.y1 = (t.y0 + 1).clamp_max(H - 1);
  t.x1 = (t.x0 + 1).clamp_max(W - 1);
  ys = at::where(t.y0 >= H - 1, t.y0.to(ys.scalar_type()), ys);
  xs = at::where(t.x0 >= W - 1, t.x0.to(xs.scalar_type()), xs);
  t.ly = ys - t.y0.to(ys.scalar_type());
  t.lx = xs - t.x0.to(xs.scalar_type());
  return t;
}

void RoiAlignImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = x_in.to(at::kFloat);
  at::Tensor rois = ctx.RequiredInput(1).to(at::kCPU, at::kFloat).contiguous();
  at::Tensor bidx = ctx.RequiredInput(2).to(at::kCPU, at::kLong).contiguous();
  const int64_t C = x.size(1), H = x.size(2), W = x.size(3), R = rois.size(0);
  const int64_t oh = n.attr_i("output_height", 1), ow = n.attr_i("output_width", 1), sr = n.attr_i("sampling_ratio", 0);
  const float scale = n.attr_f("spatial_scale", 1.0f);
  const bool is_max = n.attr_s("mode", "avg") == "max";
  // the attribute exists from opset 16 on, where it defaults to half_pixel; before, the behaviour is output_half_pixel
  const bool half_pixel = n.attr_s("coordinate_transformation_mode", n.since_version >= 16 ? "half_pixel" : "output_half_pixel") == "half_pixel";
  auto fopt = at::TensorOptions().dtype(at::kFloat).device(x.device());
  at::Tensor out = at::zeros({R, C, oh, ow}, fopt);
  const float* rp = rois.data_ptr<float>();
  for (int64_t r = 0; r < R; ++r) {
    const float off = half_pixel ? 0.5f : 0.0f;
    const float x1 = rp[4 * r] * scale - off, y1 = rp[4 * r + 1] * scale - off;
    const float x2 = rp[4 * r + 2] * scale - off, y2 = rp[4 * r + 3] * scale - off;
    float rw = x2 - x1, rh = y2 - y1;
    if (!half_pixel) {
      rw = std::max(rw, 1.0f);
      rh = std::max(rh, 1.0f);
    }
    const float bh = rh / static_cast<float>(oh), bw = rw / static_cast<float>(ow);
    const int64_t gh = sr > 0 ? sr : static_cast<int64_t>(std::ceil(rh / static_cast<float>(oh)));
    const int64_t gw = sr > 0 ? sr : static_cast<int64_t>(std::ceil(rw / static_cast<float>(ow)));
    const int64_t gh1 = std::max<int64_t>(gh, 1), gw1 = std::max<int64_t>(gw, 1);
    // sample coordinates: bin p, sub-sample i -> y1 + p * bh + (i + 0.5) * bh / gh
    at::Tensor ys = (at::arange(oh, fopt).unsqueeze(1) * bh + (at::arange(gh1, fopt).unsqueeze(0) + 0.5) * (bh / gh1) + y1).reshape({-1});
    at::Tensor xs = (at::arange(ow, fopt).unsqueeze(1) * bw + (at::arange(gw1, fopt).unsqueeze(0) + 0.5) * (bw / gw1) + x1).reshape({-1});
    Taps t = MakeTaps(ys, xs, H, W);
    at::Tensor img = x[bidx[r].item<int64_t>()];                                    // [C, H, W]
    auto corner = [&](const at::Tensor& yi, const at::Tensor& xi) { return img.index_select(1, yi).index_select(2, xi); };
    at::Tensor hy = (1 - t.ly).reshape({1, -1, 1}), ly = t.ly.reshape({1, -1, 1});
    at::Tensor hx = (1 - t.lx).reshape({1, 1, -1}), lx = t.lx.reshape({1, 1, -1});
    at::Tensor valid = (t.valid_y.reshape({1, -1, 1}) & t.valid_x.reshape({1, 1, -1})).to(at::kFloat);
    at::Tensor v00 = corner(t.y0, t.x0) * hy * hx, v01 = corner(t.y0, t.x1) * hy * lx;
    at::Tensor v10 = corner(t.y1, t.x0) * ly * hx, v11 = corner(t.y1, t.x1) * ly * lx;
    at::Tensor pooled;
    if (is_max) {
      // the reference takes the largest weighted corner of a sample, then the largest sample of the bin
      at::Tensor s = at::maximum(at::maximum(v00, v01), at::maximum(v10, v11)) * valid;
      pooled = s.reshape({C, oh, gh1, ow, gw1}).amax({2, 4});
    } else {
      at::Tensor s = (v00 + v01 + v10 + v11) * valid;
      pooled = s.reshape({C, oh, gh1, ow, gw1}).sum({2, 4}) / static_cast<double>(gh1 * gw1);
    }
    out[r].copy_(pooled);
  }
  ctx.SetOutput(0, out.to(x_in.scalar_type()));
}

// DeformConv: every kernel tap samples the input at its regular position plus a learned offset (bilinear, zero
// outside), optionally scaled by a mask; then an ordinary (grouped) convolution over the sampled columns.
void DeformConvImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = x_in.to(at::kFloat);
  at::Tensor w = ctx.RequiredInput(1).to(at::kFloat);
  at::Tensor offset = ctx.RequiredInput(2).to(at::kFloat);
  const int64_t N = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3);
  const int64_t M = w.size(0), kh = w.size(2), kw = w.size(3), K = kh * kw;
  const int64_t group = n.attr_i("group", 1), og = n.attr_i("offset_group", 1);
  std::vector<int64_t> st = n.attr_ints("strides"), dil = n.attr_ints("dilations"), pads = n.attr_ints("pads");
  if (st.empty()) st = {1, 1};
  if (dil.empty()) dil = {1, 1};
  if (pads.empty()) pads = {0, 0, 0, 0};
  const int64_t oH = (H + pads[0] + pads[2] - dil[0] * (kh - 1) - 1) / st[0] + 1;
  const int64_t oW = (W + pads[1] + pads[3] - dil[1] * (kw - 1) - 1) / st[1] + 1;
  ORTB_ENFORCE_ARG(offset.size(1) == og * K * 2 && offset.size(2) == oH && offset.size(3) == oW, "DeformConv: offset shape mismatch");
  ORTB_ENFORCE_ARG(C % og == 0 && C % group == 0 && M % group == 0, "DeformConv: channels must divide into the groups");
  at::Tensor mask;
  if (ctx.HasInput(4)) mask = ctx.Input(4).to(at::kFloat).reshape({N, og, K, oH, oW});
  offset = offset.reshape({N, og, K, 2, oH, oW});
  auto fopt = x.options();
  at::Tensor base_y = (at::arange(oH, fopt) * static_cast<double>(st[0]) - static_cast<double>(pads[0])).reshape({1, oH, 1});
  at::Tensor base_x = (at::arange(oW, fopt) * static_cast<double>(st[1]) - static_cast<double>(pads[1])).reshape({1, 1, oW});
  const int64_t cg = C / og;
  at::Tensor cols = at::empty({N, C, K, oH, oW}, fopt);
  // grid_sample with align_corners addresses pixel centres: coordinate p maps to 2 p / (size - 1) - 1
  const double sx = W > 1 ? 2.0 / static_cast<double>(W - 1) : 0.0, sy = H > 1 ? 2.0 / static_cast<double>(H - 1) : 0.0;
  for (int64_t g = 0; g < og; ++g) {
    at::Tensor xg = x.narrow(1, g * cg, cg);
    for (int64_t k = 0; k < K; ++k) {
      const int64_t ky = k / kw, kx = k % kw;
      at::Tensor py = base_y + static_cast<double>(ky * dil[0]) + offset.select(1, g).select(1, k).select(1, 0);   // [N, oH, oW]
      at::Tensor px = base_x + static_cast<double>(kx * dil[1]) + offset.select(1, g).select(1, k).select(1, 1);
      at::Tensor grid = at::stack({px * sx - 1.0, py * sy - 1.0}, -1);                                           // [N, oH, oW, 2]
      at::Tensor sampled = at::grid_sampler(xg, grid, /*bilinear*/ 0, /*zeros*/ 0, /*align_corners*/ true);     // [N, cg, oH, oW]
      if (mask.defined()) sampled = sampled * mask.select(1, g).select(1, k).unsqueeze(1);
      cols.narrow(1, g * cg, cg).select(2, k).copy_(sampled);
    }
  }
  // grouped contraction: out[n, m, :] = sum over (c in group, k) of w[m, c, k] * cols[n, c, k, :]
  const int64_t cpg = C / group, mpg = M / group;
  at::Tensor colg = cols.reshape({N, group, cpg * K, oH * oW});
  at::Tensor wg = w.reshape({group, mpg, cpg * K});
  at::Tensor y = at::matmul(wg.unsqueeze(0), colg).reshape({N, M, oH, oW});
  if (ctx.HasInput(3)) y = y + ctx.Input(3).to(at::kFloat).reshape({1, M, 1, 1});
  ctx.SetOutput(0, y.to(x_in.scalar_type()));
}

// LabelEncoder: int64 / float / string keys and values (strings travel as ids of the string table).
void LabelEncoderImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  // strings are ids of the string table (one id per distinct string), so string keys / values are integer keys / values
  const bool str_keys = n.has_attr("keys_strings") || n.has_attr("classes_strings"), str_vals = n.has_attr("values_strings");
  ORTB_ENFORCE(str_keys == ctx.InputIsString(0), "LabelEncoder: string keys need a string input (and only then)");
  const at::Tensor& x = ctx.RequiredInput(0);
  const bool int_keys = n.has_attr("keys_int64s") || str_keys, int_vals = n.has_attr("values_int64s") || str_vals || n.has_attr("classes_strings");
  auto intern_all = [](const std::vector<std::string>& v) {
    std::vector<int64_t> ids;
    for (auto& s : v) ids.push_back(InternString(s));
    return ids;
  };
  at::Tensor keys, vals;
  if (n.has_attr("classes_strings")) {  // opset 1 form: string -> its position in classes_strings
    keys = at::tensor(intern_all(n.attr_strings("classes_strings")), at::TensorOptions().dtype(at::kLong));
    vals = at::arange(keys.numel(), at::TensorOptions().dtype(at::kLong));
  } else {
    if (str_keys) keys = at::tensor(intern_all(n.attr_strings("keys_strings")), at::TensorOptions().dtype(at::kLong));
    else if (int_keys) keys = at::tensor(n.attr_ints("keys_int64s"), at::TensorOptions().dtype(at::kLong));
    else keys = at::tensor(n.attr_floats("keys_floats"), at::TensorOptions().dtype(at::kFloat));
    if (str_vals) vals = at::tensor(intern_all(n.attr_strings("values_strings")), at::TensorOptions().dtype(at::kLong));
    else if (int_vals) vals = at::tensor(n.attr_ints("values_int64s"), at::TensorOptions().dtype(at::kLong));
    else vals = at::tensor(n.attr_floats("values_floats"), at::TensorOptions().dtype(at::kFloat));
  }
  ORTB_ENFORCE_ARG(keys.numel() == vals.numel() && keys.numel() > 0, "LabelEncoder: keys and values must have the same, non-zero length");
  at::Tensor order = at::argsort(keys);
  keys = keys.index_select(0, order).to(x.device());
  vals = vals.index_select(0, order).to(x.device());
  at::Tensor xq = x.to(keys.scalar_type()).reshape({-1});
  at::Tensor pos = at::searchsorted(keys, xq).clamp_max(keys.numel() - 1);
  at::Tensor hit = keys.index_select(0, pos).eq(xq);
  at::Tensor dflt = str_vals ? at::full({1}, InternString(n.attr_s("default_string", "_Unused")), vals.options())
                    : int_vals ? at::full({1}, n.attr_i("default_int64", -1), vals.options())
                               : at::full({1}, static_cast<double>(n.attr_f("default_float", -0.0f)), vals.options());
  at::Tensor y = at::where(hit, vals.index_select(0, pos), dflt).reshape(x.sizes());
  if (str_vals) ctx.SetOutputStrings(0, y);
  else ctx.SetOutput(0, y);
}

}  // namespace

void RegisterOnnxExtraKernels2(KernelRegistry& r) {
  r.RegisterFn("", "RoiAlign", 10, kMax, RoiAlignImpl);
  r.RegisterFn("", "DeformConv", 19, kMax, DeformConvImpl);
  r.RegisterFn("ai.onnx.ml", "LabelEncoder", 1, kMax, LabelEncoderImpl);
}

}  // namespace ortb
