// ONNX-domain operators beyond the core set, and the integer-quantised contrib operators, written against ATen
// (device-agnostic).  Semantics: the ONNX operator specifications; the reference's CPU kernels live under
// onnxruntime/core/providers/cpu/{quantization,rnn,signal,object_detection,tensor,nn}/ and
// onnxruntime/contrib_ops/cpu/quantization/.
#include <ATen/ATen.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <numeric>

#include "kernel.h"
#include "graph.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

std::vector<int64_t> HostInts(const at::Tensor& t) {
  at::Tensor c = t.to(at::kCPU, at::kLong).contiguous().reshape({-1});
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

// ----------------------------------------------------------------------------------------------- quantised helpers
at::Tensor Dequant(const at::Tensor& q, const at::Tensor& scale, const at::Tensor* zp, int64_t channel_axis = -1) {
  at::Tensor s = scale.to(at::kFloat), z = zp != nullptr ? zp->to(at::kFloat) : at::zeros({}, s.options());
  if (channel_axis >= 0 && s.numel() > 1) {
    std::vector<int64_t> shape(q.dim(), 1);
    shape[channel_axis] = s.numel();
    s = s.reshape(shape);
    if (z.numel() > 1) z = z.reshape(shape);
  }
  return (q.to(at::kFloat) - z) * s;
}

at::Tensor Requant(const at::Tensor& y, const at::Tensor& scale, const at::Tensor* zp, at::ScalarType fallback) {
  const at::ScalarType dt = zp != nullptr ? zp->scalar_type() : fallback;
  const double lo = dt == at::kChar ? -128 : 0, hi = dt == at::kChar ? 127 : 255;
  at::Tensor z = zp != nullptr ? zp->to(at::kFloat) : at::zeros({}, y.options());
  return at::clamp(at::round(y / scale.to(at::kFloat)) + z, lo, hi).to(dt);   // at::round is round-half-to-even
}

const at::Tensor* Opt(Ctx& ctx, int i, at::Tensor* slot) {
  if (!ctx.HasInput(i)) return nullptr;
  *slot = ctx.Input(i);
  return slot;
}

void QLinearMatMulImpl(Ctx& ctx) {
  at::Tensor za, zb, zy;
  at::Tensor a = Dequant(ctx.RequiredInput(0), ctx.RequiredInput(1), Opt(ctx, 2, &za), ctx.RequiredInput(1).numel() > 1 ? ctx.RequiredInput(0).dim() - 2 : -1);
  at::Tensor b = Dequant(ctx.RequiredInput(3), ctx.RequiredInput(4), Opt(ctx, 5, &zb), ctx.RequiredInput(4).numel() > 1 ? ctx.RequiredInput(3).dim() - 1 : -1);
  ctx.SetOutput(0, Requant(at::matmul(a, b), ctx.RequiredInput(6), Opt(ctx, 7, &zy), ctx.RequiredInput(0).scalar_type()));
}

void QLinearBinary(Ctx& ctx, bool mul) {
  at::Tensor za, zb, zc;
  at::Tensor a = Dequant(ctx.RequiredInput(0), ctx.RequiredInput(1), Opt(ctx, 2, &za));
  at::Tensor b = Dequant(ctx.RequiredInput(3), ctx.RequiredInput(4), Opt(ctx, 5, &zb));
  ctx.SetOutput(0, Requant(mul ? a * b : a + b, ctx.RequiredInput(6), Opt(ctx, 7, &zc), ctx.RequiredInput(0).scalar_type()));
}

// ----------------------------------------------------------------------------------------------- recurrent layers
at::Tensor Act(const std::string& name, const at::Tensor& x) {
  if (name == "Sigmoid") return at::sigmoid(x);
  if (name == "Tanh") return at::tanh(x);
  if (name == "Relu") return at::relu(x);
  ORTB_THROW(NOT_IMPLEMENTED, "recurrent activation ", name, " is not supported");
}

struct RnnCommon {
  int64_t S, B, H, D;
  bool batch_first;
  std::vector<std::string> acts;
  at::Tensor x;          // [S, B, I]
  at::Tensor lens;       // optional [B] long
};

RnnCommon ParseRnn(Ctx& ctx, int gates, const std::vector<std::string>& default_acts) {
  const Node& n = ctx.node();
  RnnCommon c;
  c.batch_first = n.attr_i("layout", 0) == 1;
  c.x = ctx.RequiredInput(0);
  if (c.batch_first) c.x = c.x.transpose(0, 1);
  c.S = c.x.size(0);
  c.B = c.x.size(1);
  const std::string dir = n.attr_s("direction", "forward");
  c.D = dir == "bidirectional" ? 2 : 1;
  c.H = n.attr_i("hidden_size", ctx.RequiredInput(2).size(2));
  c.acts = n.attr_strings("activations");
  if (c.acts.empty())
    for (int64_t d = 0; d < c.D; ++d) c.acts.insert(c.acts.end(), default_acts.begin(), default_acts.end());
  if (ctx.HasInput(4)) c.lens = ctx.Input(4).to(at::kLong);
  (void)gates;
  return c;
}

// runs `step(t, h_state...)` over time for one direction; `cell` maps (x_t, states) -> new states (first is h)
template <typename Cell>
void RunDirection(const RnnCommon& c, bool reverse, std::vector<at::Tensor>& states, at::Tensor& y_dir, Cell cell) {
  std::vector<at::Tensor> outs(c.S);
  for (int64_t i = 0; i < c.S; ++i) {
    const int64_t t = reverse ? c.S - 1 - i : i;
    std::vector<at::Tensor> next = cell(c.x.select(0, t), states);
    if (c.lens.defined()) {   // sequences shorter than t keep their state and emit zeros
      at::Tensor live = (c.lens > t).to(next[0].scalar_type()).unsqueeze(1);
      for (size_t k = 0; k < next.size(); ++k) next[k] = live * next[k] + (1 - live) * states[k];
      outs[t] = next[0] * live;
    } else {
      outs[t] = next[0];
    }
    states = next;
  }
  y_dir = at::stack(outs, 0);   // [S, B, H]
}

void FinishRnn(Ctx& ctx, const RnnCommon& c, const std::vector<at::Tensor>& ys, const std::vector<std::vector<at::Tensor>>& finals) {
  at::Tensor y = at::stack(ys, 1);   // [S, D, B, H]
  if (c.batch_first) y = y.permute({2, 0, 1, 3});   // [B, S, D, H]
  if (ctx.OutputCount() > 0) ctx.SetOutput(0, y.contiguous());
  for (size_t k = 0; k < finals[0].size(); ++k) {
    std::vector<at::Tensor> per_dir;
    for (auto& f : finals) per_dir.push_back(f[k]);
    at::Tensor s = at::stack(per_dir, 0);   // [D, B, H]
    if (c.batch_first) s = s.transpose(0, 1);
    if (ctx.OutputCount() > static_cast<int>(k + 1)) ctx.SetOutput(static_cast<int>(k + 1), s.contiguous());
  }
}

// W [D, 4H, I] (gate order i o f c), R [D, 4H, H]
void LstmWithWeights(Ctx& ctx, const at::Tensor& W, const at::Tensor& R) {
  RnnCommon c = ParseRnn(ctx, 4, {"Sigmoid", "Tanh", "Tanh"});
  c.H = R.size(2);
  const std::string dir = ctx.node().attr_s("direction", "forward");
  std::vector<at::Tensor> ys;
  std::vector<std::vector<at::Tensor>> finals;
  for (int64_t d = 0; d < c.D; ++d) {
    at::Tensor bias = ctx.HasInput(3) ? ctx.Input(3).select(0, d) : at::zeros({8 * c.H}, c.x.options());
    at::Tensor b = bias.narrow(0, 0, 4 * c.H) + bias.narrow(0, 4 * c.H, 4 * c.H);
    at::Tensor h0 = ctx.HasInput(5) ? (c.batch_first ? ctx.Input(5).transpose(0, 1) : ctx.Input(5)).select(0, d) : at::zeros({c.B, c.H}, c.x.options());
    at::Tensor c0 = ctx.HasInput(6) ? (c.batch_first ? ctx.Input(6).transpose(0, 1) : ctx.Input(6)).select(0, d) : at::zeros({c.B, c.H}, c.x.options());
    at::Tensor peep = ctx.HasInput(7) ? ctx.Input(7).select(0, d) : at::Tensor();   // [3H]: i o f
    at::Tensor Wd = W.select(0, d), Rd = R.select(0, d);
    const std::string f = c.acts[3 * d], g = c.acts[3 * d + 1], hact = c.acts[3 * d + 2];
    const int64_t H = c.H;
    std::vector<at::Tensor> st = {h0, c0};
    at::Tensor y;
    RunDirection(c, dir == "reverse" || d == 1, st, y, [&](const at::Tensor& xt, const std::vector<at::Tensor>& s) {
      at::Tensor z = at::matmul(xt, Wd.t()) + at::matmul(s[0], Rd.t()) + b;
      at::Tensor zi = z.narrow(1, 0, H), zo = z.narrow(1, H, H), zf = z.narrow(1, 2 * H, H), zc = z.narrow(1, 3 * H, H);
      if (peep.defined()) {
        zi = zi + peep.narrow(0, 0, H) * s[1];
        zf = zf + peep.narrow(0, 2 * H, H) * s[1];
      }
      at::Tensor it = Act(f, zi), ft = Act(f, zf), ct = ft * s[1] + it * Act(g, zc);
      if (peep.defined()) zo = zo + peep.narrow(0, H, H) * ct;
      at::Tensor ht = Act(f, zo) * Act(hact, ct);
      return std::vector<at::Tensor>{ht, ct};
    });
    ys.push_back(y);
    finals.push_back(st);
  }
  FinishRnn(ctx, c, ys, finals);
}

void LstmImpl(Ctx& ctx) { LstmWithWeights(ctx, ctx.RequiredInput(1), ctx.RequiredInput(2)); }

// DynamicQuantizeLSTM (contrib_ops/cpu/quantization/dynamic_quantize_lstm.cc): an LSTM whose W [D, I, 4H] and
// R [D, H, 4H] arrive as 8-bit integers with per-direction or per-column scales / zero points (inputs 8 - 11).
void DynamicQuantizeLstmImpl(Ctx& ctx) {
  auto dequant = [&](int wi, int si, int zi) {
    at::Tensor q = ctx.RequiredInput(wi).to(at::kFloat);            // [D, in, 4H]
    at::Tensor scale = ctx.RequiredInput(si).to(at::kFloat);
    at::Tensor zp = ctx.HasInput(zi) ? ctx.Input(zi).to(at::kFloat) : at::zeros_like(scale);
    auto shape_for = [&](const at::Tensor& t) {
      return t.dim() == 2 ? t.reshape({t.size(0), 1, t.size(1)}) : t.reshape({-1, 1, 1});
    };
    return ((q - shape_for(zp)) * shape_for(scale)).transpose(1, 2).contiguous();  // [D, 4H, in]
  };
  LstmWithWeights(ctx, dequant(1, 8, 9), dequant(2, 10, 11));
}

void GruImpl(Ctx& ctx) {
  RnnCommon c = ParseRnn(ctx, 3, {"Sigmoid", "Tanh"});
  const at::Tensor& W = ctx.RequiredInput(1);   // [D, 3H, I]  gate order z r h
  const at::Tensor& R = ctx.RequiredInput(2);
  const bool lbr = ctx.node().attr_i("linear_before_reset", 0) != 0;
  const std::string dir = ctx.node().attr_s("direction", "forward");
  std::vector<at::Tensor> ys;
  std::vector<std::vector<at::Tensor>> finals;
  for (int64_t d = 0; d < c.D; ++d) {
    const int64_t H = c.H;
    at::Tensor bias = ctx.HasInput(3) ? ctx.Input(3).select(0, d) : at::zeros({6 * H}, c.x.options());
    at::Tensor wb = bias.narrow(0, 0, 3 * H), rb = bias.narrow(0, 3 * H, 3 * H);
    at::Tensor h0 = ctx.HasInput(5) ? (c.batch_first ? ctx.Input(5).transpose(0, 1) : ctx.Input(5)).select(0, d) : at::zeros({c.B, H}, c.x.options());
    at::Tensor Wd = W.select(0, d), Rd = R.select(0, d);
    const std::string f = c.acts[2 * d], g = c.acts[2 * d + 1];
    std::vector<at::Tensor> st = {h0};
    at::Tensor y;
    RunDirection(c, dir == "reverse" || d == 1, st, y, [&](const at::Tensor& xt, const std::vector<at::Tensor>& s) {
      at::Tensor xw = at::matmul(xt, Wd.t()) + wb;                  // [B, 3H]
      at::Tensor hz = at::matmul(s[0], Rd.narrow(0, 0, 2 * H).t()) + rb.narrow(0, 0, 2 * H);
      at::Tensor zt = Act(f, xw.narrow(1, 0, H) + hz.narrow(1, 0, H));
      at::Tensor rt = Act(f, xw.narrow(1, H, H) + hz.narrow(1, H, H));
      at::Tensor Rh = Rd.narrow(0, 2 * H, H), rbh = rb.narrow(0, 2 * H, H);
      at::Tensor hh = lbr ? Act(g, xw.narrow(1, 2 * H, H) + rt * (at::matmul(s[0], Rh.t()) + rbh))
                          : Act(g, xw.narrow(1, 2 * H, H) + at::matmul(rt * s[0], Rh.t()) + rbh);
      return std::vector<at::Tensor>{(1 - zt) * hh + zt * s[0]};
    });
    ys.push_back(y);
    finals.push_back(st);
  }
  FinishRnn(ctx, c, ys, finals);
}

void RnnImpl(Ctx& ctx) {
  RnnCommon c = ParseRnn(ctx, 1, {"Tanh"});
  const at::Tensor& W = ctx.RequiredInput(1);
  const at::Tensor& R = ctx.RequiredInput(2);
  const std::string dir = ctx.node().attr_s("direction", "forward");
  std::vector<at::Tensor> ys;
  std::vector<std::vector<at::Tensor>> finals;
  for (int64_t d = 0; d < c.D; ++d) {
    const int64_t H = c.H;
    at::Tensor bias = ctx.HasInput(3) ? ctx.Input(3).select(0, d) : at::zeros({2 * H}, c.x.options());
    at::Tensor b = bias.narrow(0, 0, H) + bias.narrow(0, H, H);
    at::Tensor h0 = ctx.HasInput(5) ? (c.batch_first ? ctx.Input(5).transpose(0, 1) : ctx.Input(5)).select(0, d) : at::zeros({c.B, H}, c.x.options());
    at::Tensor Wd = W.select(0, d), Rd = R.select(0, d);
    const std::string f = c.acts[d];
    std::vector<at::Tensor> st = {h0};
    at::Tensor y;
    RunDirection(c, dir == "reverse" || d == 1, st, y, [&](const at::Tensor& xt, const std::vector<at::Tensor>& s) {
      return std::vector<at::Tensor>{Act(f, at::matmul(xt, Wd.t()) + at::matmul(s[0], Rd.t()) + b)};
    });
    ys.push_back(y);
    finals.push_back(st);
  }
  FinishRnn(ctx, c, ys, finals);
}

// ----------------------------------------------------------------------------------------------- misc
void UniqueImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  const bool sorted = n.attr_i("sorted", 1) != 0;
  at::Tensor y, inverse, counts;
  int64_t axis = 0;
  at::Tensor flat;
  if (n.has_attr("axis")) {
    axis = n.attr_i("axis", 0);
    if (axis < 0) axis += x.dim();
    std::tie(y, inverse, counts) = at::unique_dim(x, axis, true, true, true);
  } else {
    flat = x.reshape({-1});
    std::tie(y, inverse, counts) = at::_unique2(flat, true, true, true);
  }
  const int64_t k = counts.numel(), total = inverse.numel();
  at::Tensor pos = at::arange(total, inverse.options());
  at::Tensor first = at::full({k}, total, inverse.options()).scatter_reduce(0, inverse, pos, "amin");
  if (!sorted) {   // order of first appearance
    at::Tensor order = at::argsort(first);
    y = y.index_select(n.has_attr("axis") ? axis : 0, order);
    counts = counts.index_select(0, order);
    first = first.index_select(0, order);
    at::Tensor rank = at::empty_like(order).scatter_(0, order, at::arange(k, order.options()));
    inverse = rank.index_select(0, inverse);
  }
  ctx.SetOutput(0, y);
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, first);
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, inverse);
  if (ctx.OutputCount() > 3) ctx.SetOutput(3, counts);
}

void NonMaxSuppressionImpl(Ctx& ctx) {
  at::Tensor boxes = ctx.RequiredInput(0).to(at::kCPU, at::kFloat).contiguous();    // [B, N, 4]
  at::Tensor scores = ctx.RequiredInput(1).to(at::kCPU, at::kFloat).contiguous();  // [B, C, N]
  const int64_t max_out = ctx.HasInput(2) ? HostInts(ctx.Input(2)).at(0) : 0;
  const float iou_thr = ctx.HasInput(3) ? ctx.Input(3).cpu().to(at::kFloat).item<float>() : 0.f;
  const bool has_score_thr = ctx.HasInput(4);
  const float score_thr = has_score_thr ? ctx.Input(4).cpu().to(at::kFloat).item<float>() : 0.f;
  const bool center = ctx.node().attr_i("center_point_box", 0) != 0;
  const int64_t B = boxes.size(0), N = boxes.size(1), C = scores.size(1);
  const float* bp = boxes.data_ptr<float>();
  const float* sp = scores.data_ptr<float>();
  auto corners = [&](const float* b, float& x1, float& y1, float& x2, float& y2) {
    if (center) {
      x1 = b[0] - b[2] / 2; x2 = b[0] + b[2] / 2; y1 = b[1] - b[3] / 2; y2 = b[1] + b[3] / 2;
    } else {   // [y1, x1, y2, x2], corners in any order
      y1 = std::min(b[0], b[2]); y2 = std::max(b[0], b[2]); x1 = std::min(b[1], b[3]); x2 = std::max(b[1], b[3]);
    }
  };
  std::vector<int64_t> out;
  if (max_out > 0) {
    for (int64_t b = 0; b < B; ++b) {
      for (int64_t c = 0; c < C; ++c) {
        const float* s = sp + (b * C + c) * N;
        std::vector<int64_t> order;
        for (int64_t i = 0; i < N; ++i)
          if (!has_score_thr || s[i] > score_thr) order.push_back(i);
        std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t d) { return s[a] > s[d]; });
        std::vector<int64_t> kept;
        for (int64_t i : order) {
          if (static_cast<int64_t>(kept.size()) >= max_out) break;
          float ax1, ay1, ax2, ay2;
          corners(bp + (b * N + i) * 4, ax1, ay1, ax2, ay2);
          bool ok = true;
          for (int64_t j : kept) {
            float bx1, by1, bx2, by2;
            corners(bp + (b * N + j) * 4, bx1, by1, bx2, by2);
            const float iw = std::min(ax2, bx2) - std::max(ax1, bx1), ih = std::min(ay2, by2) - std::max(ay1, by1);
            const float inter = iw > 0 && ih > 0 ? iw * ih : 0.f;
            const float uni = (ax2 - ax1) * (ay2 - ay1) + (bx2 - bx1) * (by2 - by1) - inter;
            if (uni > 0 && inter / uni > iou_thr) { ok = false; break; }
          }
          if (ok) kept.push_back(i);
        }
        for (int64_t i : kept) { out.push_back(b); out.push_back(c); out.push_back(i); }
      }
    }
  }
  at::Tensor t = at::tensor(out, at::kLong).reshape({static_cast<int64_t>(out.size() / 3), 3});
  ctx.SetOutput(0, t.to(ctx.RequiredInput(0).device()));
}

at::Tensor WindowImpl(Ctx& ctx, int kind) {
  const int64_t size = HostInts(ctx.RequiredInput(0)).at(0);
  const bool periodic = ctx.node().attr_i("periodic", 1) != 0;
  const at::ScalarType dt = ToTorchType(static_cast<int32_t>(ctx.node().attr_i("output_datatype", 1)));
  auto opt = at::TensorOptions().dtype(at::kDouble);
  at::Tensor w = kind == 0 ? at::hann_window(size, periodic, opt)
                           : kind == 1 ? (25.0 / 46.0 - 21.0 / 46.0 * at::cos(2 * M_PI * at::arange(size, opt) / static_cast<double>(periodic ? size : size - 1)))
                                       : at::blackman_window(size, periodic, opt);
  return w.to(dt);
}

void DftImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);    // [..., signal..., 1 or 2]
  const bool inverse = n.attr_i("inverse", 0) != 0, onesided = n.attr_i("onesided", 0) != 0;
  int64_t axis = n.since_version >= 20 ? (ctx.HasInput(2) ? HostInts(ctx.Input(2)).at(0) : -2) : n.attr_i("axis", 1);
  if (axis < 0) axis += x.dim();
  c10::optional<int64_t> len;
  if (ctx.HasInput(1)) len = HostInts(ctx.Input(1)).at(0);
  const bool real_in = x.size(-1) == 1;
  at::Tensor c = real_in ? at::complex(x.squeeze(-1).to(at::kFloat), at::zeros_like(x.squeeze(-1), at::kFloat))
                         : at::view_as_complex(x.to(at::kFloat).contiguous());
  at::Tensor y;
  if (inverse) {
    y = at::fft_ifft(c, len, axis);
    if (onesided) {   // inverse of a one-sided transform yields a real signal
      y = at::fft_irfft(c, len, axis);
      ctx.SetOutput(0, y.unsqueeze(-1).to(x.scalar_type()));
      return;
    }
  } else if (onesided && real_in) {
    y = at::fft_rfft(at::real(c), len, axis);
  } else {
    y = at::fft_fft(c, len, axis);
  }
  ctx.SetOutput(0, at::view_as_real(y).to(x.scalar_type()));
}

void LossImpl(Ctx& ctx, bool softmax) {
  const Node& n = ctx.node();
  at::Tensor scores = ctx.RequiredInput(0);      // [N, C, d1...]
  const at::Tensor& target = ctx.RequiredInput(1);
  const std::string reduction = n.attr_s("reduction", "mean");
  const int64_t ignore = n.has_attr("ignore_index") ? n.attr_i("ignore_index", -100) : std::numeric_limits<int64_t>::min();
  at::Tensor logp = softmax ? at::log_softmax(scores.to(at::kFloat), 1) : scores.to(at::kFloat);
  c10::optional<at::Tensor> w;
  if (ctx.HasInput(2)) w = ctx.Input(2).to(at::kFloat);
  const int64_t red = reduction == "none" ? 0 : reduction == "mean" ? 1 : 2;
  at::Tensor loss = at::nll_loss_nd(logp, target.to(at::kLong), w, red, ignore);
  ctx.SetOutput(0, loss.to(scores.scalar_type()));
  if (softmax && ctx.OutputCount() > 1) ctx.SetOutput(1, logp.to(scores.scalar_type()));
}

}  // namespace

void RegisterOnnxExtraKernels(KernelRegistry& r) {
  // ---- integer-quantised linear algebra
  r.RegisterFn("", "QLinearMatMul", 10, kMax, QLinearMatMulImpl);
  r.RegisterFn(MS, "QLinearAdd", 1, kMax, [](Ctx& ctx) { QLinearBinary(ctx, false); });
  r.RegisterFn(MS, "QLinearMul", 1, kMax, [](Ctx& ctx) { QLinearBinary(ctx, true); });
  auto qunary = [](int kind) {
    return [kind](Ctx& ctx) {
      at::Tensor zx, zy;
      at::Tensor x = Dequant(ctx.RequiredInput(0), ctx.RequiredInput(1), Opt(ctx, 2, &zx));
      at::Tensor y = kind == 0 ? at::sigmoid(x) : at::leaky_relu(x, ctx.node().attr_f("alpha", 0.01f));
      ctx.SetOutput(0, Requant(y, ctx.RequiredInput(3), Opt(ctx, 4, &zy), ctx.RequiredInput(0).scalar_type()));
    };
  };
  r.RegisterFn(MS, "QLinearSigmoid", 1, kMax, qunary(0));
  r.RegisterFn(MS, "QLinearLeakyRelu", 1, kMax, qunary(1));
  r.RegisterFn(MS, "MatMulIntegerToFloat", 1, kMax, [](Ctx& ctx) {
    // A, B, a_scale, b_scale, a_zero_point?, b_zero_point?, bias?
    at::Tensor za, zb;
    const at::Tensor& B = ctx.RequiredInput(1);
    at::Tensor a = Dequant(ctx.RequiredInput(0), ctx.RequiredInput(2), Opt(ctx, 4, &za));
    at::Tensor b = Dequant(B, ctx.RequiredInput(3), Opt(ctx, 5, &zb), ctx.RequiredInput(3).numel() > 1 ? B.dim() - 1 : -1);
    at::Tensor y = at::matmul(a, b);
    if (ctx.HasInput(6)) y = y + ctx.Input(6);
    ctx.SetOutput(0, y);
  });
  r.RegisterFn(MS, "DynamicQuantizeMatMul", 1, kMax, [](Ctx& ctx) {
    // A (float) is quantised to uint8 on the fly as DynamicQuantizeLinear does; B, b_scale, b_zero_point?, bias?
    at::Tensor x = ctx.RequiredInput(0).to(at::kFloat);
    at::Tensor mx = at::clamp_min(at::max(x), 0), mn = at::clamp_max(at::min(x), 0);
    at::Tensor scale = (mx - mn) / 255.0;
    at::Tensor safe = at::where(scale == 0, at::ones_like(scale), scale);
    at::Tensor zp = at::clamp(at::round(-mn / safe), 0, 255);
    at::Tensor a = (at::clamp(at::round(x / safe) + zp, 0, 255) - zp) * scale;
    at::Tensor zb;
    const at::Tensor& B = ctx.RequiredInput(1);
    at::Tensor b = Dequant(B, ctx.RequiredInput(2), Opt(ctx, 3, &zb), ctx.RequiredInput(2).numel() > 1 ? B.dim() - 1 : -1);
    at::Tensor y = at::matmul(a, b);
    if (ctx.HasInput(4)) y = y + ctx.Input(4);
    ctx.SetOutput(0, y);
  });
  r.RegisterFn(MS, "QGemm", 1, kMax, [](Ctx& ctx) {
    // A, a_scale, a_zp, B, b_scale, b_zp, C? (int32, scale a_scale * b_scale), y_scale?, y_zp?
    const Node& n = ctx.node();
    at::Tensor za, zb, zy;
    at::Tensor a = Dequant(ctx.RequiredInput(0), ctx.RequiredInput(1), Opt(ctx, 2, &za));
    const at::Tensor& B = ctx.RequiredInput(3);
    const bool tb = n.attr_i("transB", 0) != 0;
    at::Tensor b = Dequant(B, ctx.RequiredInput(4), Opt(ctx, 5, &zb), ctx.RequiredInput(4).numel() > 1 ? (tb ? 0 : 1) : -1);
    if (n.attr_i("transA", 0)) a = a.t();
    if (tb) b = b.t();
    at::Tensor y = at::matmul(a, b) * n.attr_f("alpha", 1.f);
    if (ctx.HasInput(6)) y = y + ctx.Input(6).to(at::kFloat) * (ctx.RequiredInput(1).to(at::kFloat) * ctx.RequiredInput(4).to(at::kFloat).reshape({-1}));
    if (ctx.HasInput(7)) ctx.SetOutput(0, Requant(y, ctx.Input(7), Opt(ctx, 8, &zy), ctx.RequiredInput(0).scalar_type()));
    else ctx.SetOutput(0, y);
  });

  // ---- recurrent layers
  r.RegisterFn("", "LSTM", 7, kMax, LstmImpl);
  r.RegisterFn(kMSDomain, "DynamicQuantizeLSTM", 1, kMax, DynamicQuantizeLstmImpl);
  r.RegisterFn("", "GRU", 7, kMax, GruImpl);
  r.RegisterFn("", "RNN", 7, kMax, RnnImpl);

  // ---- signal
  r.RegisterFn("", "HannWindow", 17, kMax, [](Ctx& ctx) { ctx.SetOutput(0, WindowImpl(ctx, 0)); }, {0});
  r.RegisterFn("", "HammingWindow", 17, kMax, [](Ctx& ctx) { ctx.SetOutput(0, WindowImpl(ctx, 1)); }, {0});
  r.RegisterFn("", "BlackmanWindow", 17, kMax, [](Ctx& ctx) { ctx.SetOutput(0, WindowImpl(ctx, 2)); }, {0});
  r.RegisterFn("", "DFT", 17, kMax, DftImpl, {1, 2});

  // ---- pooling / normalisation / linear algebra
  auto lp_pool = [](bool global) {
    return [global](Ctx& ctx) {
      const Node& n = ctx.node();
      const at::Tensor& x = ctx.RequiredInput(0);
      const double p = static_cast<double>(n.attr_i("p", 2));
      const int64_t nd = x.dim() - 2;
      at::Tensor xp = at::pow(at::abs(x.to(at::kFloat)), p);
      at::Tensor s;
      if (global) {
        std::vector<int64_t> dims;
        for (int64_t i = 2; i < x.dim(); ++i) dims.push_back(i);
        s = at::sum(xp, dims, true);
      } else {
        std::vector<int64_t> k = n.attr_ints("kernel_shape"), st = n.attr_ints("strides"), pads = n.attr_ints("pads");
        if (st.empty()) st.assign(nd, 1);
        if (pads.empty()) pads.assign(2 * nd, 0);
        std::vector<int64_t> pb(pads.begin(), pads.begin() + nd);
        int64_t ksize = 1;
        for (int64_t v : k) ksize *= v;
        const bool ceil_mode = n.attr_i("ceil_mode", 0) != 0;
        at::Tensor avg = nd == 1   ? at::avg_pool1d(xp, k, st, pb, ceil_mode, true)
                         : nd == 2 ? at::avg_pool2d(xp, k, st, pb, ceil_mode, true)
                                   : at::avg_pool3d(xp, k, st, pb, ceil_mode, true);
        s = avg * static_cast<double>(ksize);
      }
      ctx.SetOutput(0, at::pow(s, 1.0 / p).to(x.scalar_type()));
    };
  };
  r.RegisterFn("", "LpPool", 1, kMax, lp_pool(false));
  r.RegisterFn("", "GlobalLpPool", 1, kMax, lp_pool(true));
  r.RegisterFn("", "Det", 11, kMax, [](Ctx& ctx) { ctx.SetOutput(0, at::linalg_det(ctx.RequiredInput(0))); });
  r.RegisterFn("", "MeanVarianceNormalization", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    std::vector<int64_t> axes = ctx.node().attr_ints("axes");
    if (axes.empty()) axes = {0, 2, 3};
    at::Tensor xf = x.to(at::kFloat);
    at::Tensor mean = at::mean(xf, axes, true);
    at::Tensor var = at::mean(at::pow(xf - mean, 2), axes, true);
    ctx.SetOutput(0, ((xf - mean) / (at::sqrt(var) + 1e-9)).to(x.scalar_type()));
  });
  r.RegisterFn("", "Col2Im", 18, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);
    const std::vector<int64_t> image = HostInts(ctx.RequiredInput(1)), block = HostInts(ctx.RequiredInput(2));
    ORTB_ENFORCE(image.size() == 2, "Col2Im: only two spatial dimensions are supported");
    std::vector<int64_t> dil = n.attr_ints("dilations"), pads = n.attr_ints("pads"), st = n.attr_ints("strides");
    if (dil.empty()) dil = {1, 1};
    if (st.empty()) st = {1, 1};
    if (pads.empty()) pads = {0, 0, 0, 0};
    ORTB_ENFORCE(pads[0] == pads[2] && pads[1] == pads[3], "Col2Im: asymmetric pads are not supported");
    ctx.SetOutput(0, at::col2im(x, image, block, dil, {pads[0], pads[1]}, st));
  }, {1, 2});
  r.RegisterFn("", "CenterCropPad", 18, kMax, [](Ctx& ctx) {
    at::Tensor y = ctx.RequiredInput(0);
    const std::vector<int64_t> shape = HostInts(ctx.RequiredInput(1));
    std::vector<int64_t> axes = ctx.node().attr_ints("axes");
    if (axes.empty()) for (int64_t i = 0; i < y.dim(); ++i) axes.push_back(i);
    for (size_t i = 0; i < axes.size(); ++i) {
      const int64_t ax = axes[i] < 0 ? axes[i] + y.dim() : axes[i], have = y.size(ax), want = shape[i];
      if (want < have) {
        y = y.narrow(ax, (have - want) / 2, want);
      } else if (want > have) {
        std::vector<int64_t> sz = y.sizes().vec();
        sz[ax] = want;
        at::Tensor out = at::zeros(sz, y.options());
        out.narrow(ax, (want - have) / 2, have).copy_(y);
        y = out;
      }
    }
    ctx.SetOutput(0, y.contiguous());
  }, {1});
  r.RegisterFn("", "MaxUnpool", 9, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);
    const at::Tensor& idx = ctx.RequiredInput(1);
    const int64_t nd = x.dim() - 2;
    std::vector<int64_t> out_shape;
    if (ctx.HasInput(2)) {
      out_shape = HostInts(ctx.Input(2));
    } else {
      std::vector<int64_t> k = n.attr_ints("kernel_shape"), st = n.attr_ints("strides"), pads = n.attr_ints("pads");
      if (st.empty()) st.assign(nd, 1);
      if (pads.empty()) pads.assign(2 * nd, 0);
      out_shape = {x.size(0), x.size(1)};
      for (int64_t i = 0; i < nd; ++i) out_shape.push_back((x.size(2 + i) - 1) * st[i] - pads[i] - pads[nd + i] + k[i]);
    }
    int64_t total = 1;
    for (int64_t v : out_shape) total *= v;
    at::Tensor out = at::zeros({total}, x.options());
    out.index_put_({idx.reshape({-1}).to(at::kLong)}, x.reshape({-1}));   // indices address the flattened output
    ctx.SetOutput(0, out.reshape(out_shape));
  }, {2});
  r.RegisterFn("", "AffineGrid", 20, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::affine_grid_generator(ctx.RequiredInput(0), HostInts(ctx.RequiredInput(1)), ctx.node().attr_i("align_corners", 0) != 0));
  }, {1});

  // ---- losses
  r.RegisterFn("", "NegativeLogLikelihoodLoss", 12, kMax, [](Ctx& ctx) { LossImpl(ctx, false); });
  r.RegisterFn("", "SoftmaxCrossEntropyLoss", 12, kMax, [](Ctx& ctx) { LossImpl(ctx, true); });

  // ---- random
  r.RegisterFn("", "Bernoulli", 15, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);
    c10::optional<at::Generator> gen;
    if (n.has_attr("seed")) {
      gen = at::detail::createCPUGenerator(static_cast<uint64_t>(n.attr_f("seed", 0.f)));
    }
    at::Tensor y = at::bernoulli(x.to(at::kCPU, at::kFloat), gen);
    const at::ScalarType dt = n.has_attr("dtype") ? ToTorchType(static_cast<int32_t>(n.attr_i("dtype", 1))) : x.scalar_type();
    ctx.SetOutput(0, y.to(x.device(), dt));
  });
  r.RegisterFn("", "Multinomial", 7, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);   // unnormalised log-probabilities [batch, classes]
    c10::optional<at::Generator> gen;
    if (n.has_attr("seed")) gen = at::detail::createCPUGenerator(static_cast<uint64_t>(n.attr_f("seed", 0.f)));
    at::Tensor p = at::softmax(x.to(at::kCPU, at::kFloat), 1);
    at::Tensor y = at::multinomial(p, n.attr_i("sample_size", 1), true, gen);
    ctx.SetOutput(0, y.to(x.device(), ToTorchType(static_cast<int32_t>(n.attr_i("dtype", 6)))));
  });

  // ---- selection
  r.RegisterFn("", "Unique", 11, kMax, UniqueImpl);
  r.RegisterFn("", "NonMaxSuppression", 10, kMax, NonMaxSuppressionImpl, {2, 3, 4});
  r.RegisterFn("", "TensorScatter", 24, kMax, [](Ctx& ctx) {
    // KV-cache update: update [B, ..., T, ...] is written into past_cache along `axis` starting at write_indices[b]
    const Node& n = ctx.node();
    at::Tensor out = ctx.RequiredInput(0).clone();
    const at::Tensor& upd = ctx.RequiredInput(1);
    int64_t axis = n.attr_i("axis", -2);
    if (axis < 0) axis += out.dim();
    const bool circular = n.attr_s("mode", "linear") == "circular";
    const int64_t B = out.size(0), T = upd.size(axis), cap = out.size(axis);
    std::vector<int64_t> start(B, 0);
    if (ctx.HasInput(2)) start = HostInts(ctx.Input(2));
    for (int64_t b = 0; b < B; ++b) {
      for (int64_t t = 0; t < T; ++t) {
        int64_t pos = start[b] + t;
        if (circular) pos %= cap;
        ORTB_ENFORCE(pos >= 0 && pos < cap, "TensorScatter: write position out of range");
        out.select(0, b).select(axis - 1, pos).copy_(upd.select(0, b).select(axis - 1, t));
      }
    }
    ctx.SetOutput(0, out);
  }, {2});
}

}  // namespace ortb
