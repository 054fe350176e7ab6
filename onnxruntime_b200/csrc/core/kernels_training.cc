// Training operators of the com.microsoft domain: the backward halves that a gradient graph is made of, loss
// functions in their training form, gradient accumulation and the optimizers.  Semantics follow the schemas in
// orttraining/orttraining/core/graph/training_op_defs.cc and the CPU kernels under
// orttraining/orttraining/training_ops/cpu (activation_grad, layer_norm, loss, optimizer/adamw, optimizer/sgd,
// optimizer/clip_grad_norm, tensor/gather_grad, tensor/slice_grad, nn/conv_grad, nn/dropout_grad).  Every kernel is
// a composition of tensor-library calls, so it runs on the device its inputs live on; optimizer state is updated in
// place, the way the reference aliases its sequence inputs to its outputs.
#include <ATen/ATen.h>
#include <c10/core/GradMode.h>

#include <cmath>

#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
const char* const MS = "com.microsoft";

int64_t NormAxis(int64_t axis, int64_t rank) { return axis < 0 ? axis + rank : axis; }

std::vector<int64_t> HostInts(const at::Tensor& t) {
  at::Tensor c = t.to(at::kCPU, at::kLong).contiguous().reshape({-1});
  return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
}

const std::vector<at::Tensor>& SeqInput(Ctx& ctx, int i, const char* what) {
  ORTB_ENFORCE_ARG(i < ctx.InputCount() && ctx.InputValue(i).seq != nullptr, ctx.node().op_type, ": input '", what,
                   "' must be a sequence of tensors");
  return *ctx.InputValue(i).seq;
}

// ---- activations --------------------------------------------------------------------------------------------------
void ReluGrad(Ctx& ctx) { ctx.SetOutput(0, ctx.RequiredInput(0) * (ctx.RequiredInput(1) > 0).to(ctx.Input(0).scalar_type())); }

void GeluGrad(Ctx& ctx) {  // exact (erf) form; input 1 is X
  const at::Tensor& dy = ctx.RequiredInput(0);
  at::Tensor x = ctx.RequiredInput(1).to(at::kFloat);
  at::Tensor cdf = 0.5 * (1.0 + at::erf(x * M_SQRT1_2));
  at::Tensor pdf = at::exp(-0.5 * x * x) * (1.0 / std::sqrt(2.0 * M_PI));
  ctx.SetOutput(0, (dy.to(at::kFloat) * (cdf + x * pdf)).to(dy.scalar_type()));
}

at::Tensor TanhGeluDerivative(const at::Tensor& x) {
  const double a = std::sqrt(2.0 / M_PI), b = 0.044715;
  at::Tensor u = a * (x + b * x * x * x);
  at::Tensor t = at::tanh(u);
  return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * a * (1.0 + 3.0 * b * x * x);
}

void FastGeluGrad(Ctx& ctx) {
  const at::Tensor& dy = ctx.RequiredInput(0);
  ctx.SetOutput(0, (dy.to(at::kFloat) * TanhGeluDerivative(ctx.RequiredInput(1).to(at::kFloat))).to(dy.scalar_type()));
}

void BiasGeluGradDx(Ctx& ctx, bool fast) {  // (dY, X, B): derivative at X + B
  const at::Tensor& dy = ctx.RequiredInput(0);
  at::Tensor x = (ctx.RequiredInput(1) + ctx.RequiredInput(2)).to(at::kFloat);
  at::Tensor d;
  if (fast) {
    d = TanhGeluDerivative(x);
  } else {
    d = 0.5 * (1.0 + at::erf(x * M_SQRT1_2)) + x * at::exp(-0.5 * x * x) * (1.0 / std::sqrt(2.0 * M_PI));
  }
  ctx.SetOutput(0, (dy.to(at::kFloat) * d).to(dy.scalar_type()));
}

void QuickGeluGrad(Ctx& ctx) {
  const double alpha = ctx.node().attr_f("alpha", 1.702f);
  const at::Tensor& dy = ctx.RequiredInput(0);
  at::Tensor x = ctx.RequiredInput(1).to(at::kFloat);
  at::Tensor s = at::sigmoid(alpha * x);
  ctx.SetOutput(0, (dy.to(at::kFloat) * (s + alpha * x * s * (1.0 - s))).to(dy.scalar_type()));
}

void SigmoidGrad(Ctx& ctx) {  // input 1 is Y
  const at::Tensor& y = ctx.RequiredInput(1);
  ctx.SetOutput(0, ctx.RequiredInput(0) * y * (1.0 - y));
}

void TanhGrad(Ctx& ctx) {
  const at::Tensor& y = ctx.RequiredInput(1);
  ctx.SetOutput(0, ctx.RequiredInput(0) * (1.0 - y * y));
}

void LeakyReluGrad(Ctx& ctx) {  // input 1 is Y (its sign is X's sign for alpha > 0)
  const double alpha = ctx.node().attr_f("alpha", 0.01f);
  const at::Tensor& dy = ctx.RequiredInput(0);
  ctx.SetOutput(0, at::where(ctx.RequiredInput(1) > 0, dy, dy * alpha));
}

// ---- softmax family -----------------------------------------------------------------------------------------------
// The opset-13 forms reduce over `axis` only; the older forms flatten [axis, rank) into one dimension.
void SoftmaxGradImpl(Ctx& ctx, bool log_form, bool opset13) {
  const at::Tensor& dy = ctx.RequiredInput(0);
  const at::Tensor& y = ctx.RequiredInput(1);
  const int64_t axis = NormAxis(ctx.node().attr_i("axis", opset13 ? -1 : 1), y.dim());
  at::Tensor dy2 = dy.to(at::kFloat), y2 = y.to(at::kFloat);
  std::vector<int64_t> dims;
  if (opset13) {
    dims = {axis};
  } else {
    for (int64_t d = axis; d < y.dim(); ++d) dims.push_back(d);
  }
  at::Tensor dx = log_form ? dy2 - at::exp(y2) * dy2.sum(dims, true) : y2 * (dy2 - (dy2 * y2).sum(dims, true));
  ctx.SetOutput(0, dx.to(dy.scalar_type()));
}

// ---- normalisation ------------------------------------------------------------------------------------------------
void LayerNormGrad(Ctx& ctx, bool simplified) {
  const at::Tensor& dy = ctx.RequiredInput(0);
  const at::Tensor& x = ctx.RequiredInput(1);
  const at::Tensor& scale = ctx.RequiredInput(2);
  const int64_t axis = NormAxis(ctx.node().attr_i("axis", -1), x.dim());
  at::Tensor inv = ctx.RequiredInput(simplified ? 3 : 4).to(at::kFloat);
  std::vector<int64_t> norm_dims, batch_dims;
  for (int64_t d = 0; d < x.dim(); ++d) (d < axis ? batch_dims : norm_dims).push_back(d);
  std::vector<int64_t> stat_shape = x.sizes().vec();
  for (int64_t d = axis; d < x.dim(); ++d) stat_shape[static_cast<size_t>(d)] = 1;
  inv = inv.reshape(stat_shape);
  at::Tensor xf = x.to(at::kFloat), dyf = dy.to(at::kFloat);
  at::Tensor xhat = simplified ? xf * inv : (xf - ctx.RequiredInput(3).to(at::kFloat).reshape(stat_shape)) * inv;
  at::Tensor g = dyf * scale.to(at::kFloat);
  at::Tensor dx;
  if (simplified) {
    dx = inv * (g - xhat * (g * xhat).mean(norm_dims, true));
  } else {
    dx = inv * (g - g.mean(norm_dims, true) - xhat * (g * xhat).mean(norm_dims, true));
  }
  ctx.SetOutput(0, dx.to(x.scalar_type()));
  at::Tensor dscale = dyf * xhat, dbias = dyf;
  if (!batch_dims.empty()) {
    dscale = dscale.sum(batch_dims);
    dbias = dbias.sum(batch_dims);
  }
  ctx.SetOutput(1, dscale.reshape(scale.sizes()).to(scale.scalar_type()));
  if (!simplified && ctx.OutputCount() > 2) ctx.SetOutput(2, dbias.reshape(scale.sizes()).to(scale.scalar_type()));
}

void BatchNormGrad(Ctx& ctx) {  // (dY, X, scale, saved mean, saved variance) over [N, C, ...]
  const double eps = ctx.node().attr_f("epsilon", 1e-5f);
  at::Tensor dy = ctx.RequiredInput(0).to(at::kFloat), x = ctx.RequiredInput(1).to(at::kFloat);
  const at::Tensor& scale = ctx.RequiredInput(2);
  std::vector<int64_t> dims{0}, cshape(static_cast<size_t>(x.dim()), 1);
  for (int64_t d = 2; d < x.dim(); ++d) dims.push_back(d);
  cshape[1] = x.size(1);
  at::Tensor mean = ctx.RequiredInput(3).to(at::kFloat).reshape(cshape);
  at::Tensor inv = at::rsqrt(ctx.RequiredInput(4).to(at::kFloat).reshape(cshape) + eps);
  at::Tensor xhat = (x - mean) * inv;
  at::Tensor g = dy * scale.to(at::kFloat).reshape(cshape);
  at::Tensor dx = inv * (g - g.mean(dims, true) - xhat * (g * xhat).mean(dims, true));
  ctx.SetOutput(0, dx.to(ctx.Input(1).scalar_type()));
  ctx.SetOutput(1, (dy * xhat).sum(dims).to(scale.scalar_type()));
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, dy.sum(dims).to(scale.scalar_type()));
}

// ---- losses -------------------------------------------------------------------------------------------------------
// logits [N, C, d1..], labels [N, d1..].  Returns the per-element weights (class weight, zero where ignored).
at::Tensor SceWeights(const at::Tensor& labels, const at::Tensor& weight, int64_t ignore_index, bool has_ignore,
                      at::Tensor* safe_labels) {
  at::Tensor keep = has_ignore ? labels != ignore_index : at::ones_like(labels, at::kBool);
  *safe_labels = at::where(keep, labels, at::zeros_like(labels));
  at::Tensor w = weight.defined() ? weight.to(at::kFloat).index({*safe_labels}) : at::ones(labels.sizes(), labels.options().dtype(at::kFloat));
  return w * keep.to(at::kFloat);
}

void SceInternal(Ctx& ctx) {  // (scores, labels, weights?, ignore_index?) -> (loss, log_prob)
  const at::Tensor& scores = ctx.RequiredInput(0);
  at::Tensor labels = ctx.RequiredInput(1).to(at::kLong);
  const std::string reduction = ctx.node().attr_s("reduction", "mean");
  at::Tensor weight = ctx.HasInput(2) ? ctx.Input(2) : at::Tensor();
  const bool has_ignore = ctx.HasInput(3);
  const int64_t ignore = has_ignore ? ctx.Input(3).item<int64_t>() : 0;
  at::Tensor logp = at::log_softmax(scores.to(at::kFloat), 1);
  at::Tensor safe;
  at::Tensor w = SceWeights(labels, weight, ignore, has_ignore, &safe);
  at::Tensor picked = -logp.gather(1, safe.unsqueeze(1)).squeeze(1) * w;
  at::Tensor loss = picked;
  if (reduction == "mean") {
    loss = picked.sum() / at::clamp_min(w.sum(), 1e-12);
  } else if (reduction == "sum") {
    loss = picked.sum();
  }
  ctx.SetOutput(0, loss.to(scores.scalar_type()));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, logp.to(scores.scalar_type()));
}

// (dY, log_prob, label, weight?, ignore_index?, bias?) -> d_logits; `ignore_from_attr` is the ONNX-attribute form
void SceGrad(Ctx& ctx, bool ignore_from_attr) {
  const at::Tensor& dy = ctx.RequiredInput(0);
  const at::Tensor& logp_in = ctx.RequiredInput(1);
  at::Tensor labels = ctx.RequiredInput(2).to(at::kLong);
  at::Tensor weight = ctx.HasInput(3) ? ctx.Input(3) : at::Tensor();
  const std::string reduction = ctx.node().attr_s("reduction", "mean");
  bool has_ignore;
  int64_t ignore = 0;
  if (ignore_from_attr) {
    has_ignore = ctx.node().has_attr("ignore_index");
    ignore = ctx.node().attr_i("ignore_index", 0);
  } else {
    has_ignore = ctx.HasInput(4);
    if (has_ignore) ignore = ctx.Input(4).item<int64_t>();
  }
  at::Tensor logp = logp_in.to(at::kFloat);
  at::Tensor safe;
  at::Tensor w = SceWeights(labels, weight, ignore, has_ignore, &safe);
  at::Tensor onehot = at::zeros_like(logp).scatter_(1, safe.unsqueeze(1), 1.0);
  at::Tensor g = (at::exp(logp) - onehot) * w.unsqueeze(1);
  at::Tensor dyf = dy.to(at::kFloat);
  if (reduction == "mean") {
    g = g * (dyf / at::clamp_min(w.sum(), 1e-12));
  } else if (reduction == "sum") {
    g = g * dyf;
  } else {
    g = g * dyf.unsqueeze(1);
  }
  if (!ignore_from_attr && ctx.HasInput(5)) g = g + ctx.Input(5).to(at::kFloat);
  ctx.SetOutput(0, g.to(logp_in.scalar_type()));
}

// ---- gradients of data movement ---------------------------------------------------------------------------------
void GatherGrad(Ctx& ctx) {  // (shape, indices, dY; axis)
  std::vector<int64_t> shape = HostInts(ctx.RequiredInput(0));
  const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), static_cast<int64_t>(shape.size()));
  at::Tensor idx = ctx.RequiredInput(1).to(at::kLong).reshape({-1});
  const at::Tensor& dy = ctx.RequiredInput(2);
  idx = at::where(idx < 0, idx + shape[static_cast<size_t>(axis)], idx);
  std::vector<int64_t> mid = shape;
  mid[static_cast<size_t>(axis)] = idx.numel();
  ctx.SetOutput(0, at::zeros(shape, dy.options()).index_add_(axis, idx, dy.reshape(mid)));
}

void GatherElementsGrad(Ctx& ctx) {  // (dY, shape, indices; axis)
  const at::Tensor& dy = ctx.RequiredInput(0);
  std::vector<int64_t> shape = HostInts(ctx.RequiredInput(1));
  const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), static_cast<int64_t>(shape.size()));
  at::Tensor idx = ctx.RequiredInput(2).to(at::kLong);
  idx = at::where(idx < 0, idx + shape[static_cast<size_t>(axis)], idx);
  ctx.SetOutput(0, at::zeros(shape, dy.options()).scatter_add_(axis, idx, dy));
}

void GatherNDGrad(Ctx& ctx) {  // (shape, indices [B.., M.., k], update; batch_dims)
  std::vector<int64_t> shape = HostInts(ctx.RequiredInput(0));
  at::Tensor idx = ctx.RequiredInput(1).to(at::kLong);
  const at::Tensor& upd = ctx.RequiredInput(2);
  const int64_t b = ctx.node().attr_i("batch_dims", 0), k = idx.size(-1);
  int64_t batch = 1, span = 1, rest = 1;
  for (int64_t d = 0; d < b; ++d) batch *= shape[static_cast<size_t>(d)];
  for (int64_t d = b; d < b + k; ++d) span *= shape[static_cast<size_t>(d)];
  for (size_t d = static_cast<size_t>(b + k); d < shape.size(); ++d) rest *= shape[d];
  at::Tensor flat = idx.reshape({batch, -1, k});
  at::Tensor lin = at::zeros({batch, flat.size(1)}, flat.options());
  int64_t stride = span;
  for (int64_t j = 0; j < k; ++j) {
    const int64_t dim = shape[static_cast<size_t>(b + j)];
    stride /= dim;
    at::Tensor col = flat.select(2, j);
    lin = lin + at::where(col < 0, col + dim, col) * stride;
  }
  lin = lin + at::arange(batch, flat.options()).unsqueeze(1) * span;
  at::Tensor out = at::zeros({batch * span, rest}, upd.options()).index_add_(0, lin.reshape({-1}), upd.reshape({-1, rest}));
  ctx.SetOutput(0, out.reshape(shape));
}

// Positions of a slice: the same slice is taken of a tensor that holds every element's own flat offset.
void SliceGrad(Ctx& ctx) {  // (dY, shape, starts, ends, axes?, steps?)
  const at::Tensor& dy = ctx.RequiredInput(0);
  std::vector<int64_t> shape = HostInts(ctx.RequiredInput(1));
  std::vector<int64_t> starts = HostInts(ctx.RequiredInput(2)), ends = HostInts(ctx.RequiredInput(3));
  std::vector<int64_t> axes, steps;
  if (ctx.HasInput(4)) axes = HostInts(ctx.Input(4));
  if (ctx.HasInput(5)) steps = HostInts(ctx.Input(5));
  int64_t total = 1;
  for (int64_t d : shape) total *= d;
  at::Tensor pos = at::arange(total, dy.options().dtype(at::kLong)).reshape(shape);
  for (size_t i = 0; i < starts.size(); ++i) {
    const int64_t axis = NormAxis(axes.empty() ? static_cast<int64_t>(i) : axes[i], static_cast<int64_t>(shape.size()));
    const int64_t dim = shape[static_cast<size_t>(axis)], step = steps.empty() ? 1 : steps[i];
    ORTB_ENFORCE_ARG(step != 0, "SliceGrad: a step of 0");
    int64_t s = starts[i] < 0 ? starts[i] + dim : starts[i], e = ends[i] < 0 ? ends[i] + dim : ends[i];
    std::vector<int64_t> picks;
    if (step > 0) {
      s = std::min(std::max<int64_t>(s, 0), dim);
      e = std::min(std::max<int64_t>(e, 0), dim);
      for (int64_t p = s; p < e; p += step) picks.push_back(p);
    } else {
      s = std::min(std::max<int64_t>(s, 0), dim - 1);
      e = std::min(std::max<int64_t>(e, -1), dim - 1);
      for (int64_t p = s; p > e; p += step) picks.push_back(p);
    }
    pos = pos.index_select(axis, at::tensor(picks, pos.options()));
  }
  at::Tensor out = at::zeros({total}, dy.options());
  out.index_put_({pos.reshape({-1})}, dy.reshape({-1}));
  ctx.SetOutput(0, out.reshape(shape));
}

void ConvGrad(Ctx& ctx) {  // (dY, X, W) -> (dX, dW, dB)
  const Node& n = ctx.node();
  const at::Tensor& dy = ctx.RequiredInput(0);
  const at::Tensor& x = ctx.RequiredInput(1);
  const at::Tensor& w = ctx.RequiredInput(2);
  const size_t sp = static_cast<size_t>(x.dim() - 2);
  std::vector<int64_t> strides = n.attr_ints("strides"), dil = n.attr_ints("dilations"), pads = n.attr_ints("pads");
  if (strides.empty()) strides.assign(sp, 1);
  if (dil.empty()) dil.assign(sp, 1);
  if (pads.empty()) pads.assign(2 * sp, 0);
  const std::string auto_pad = n.attr_s("auto_pad", "NOTSET");
  ORTB_ENFORCE_ARG(auto_pad == "NOTSET" || auto_pad == "VALID", "ConvGrad: auto_pad ", auto_pad, " is not supported");
  std::vector<int64_t> padding(sp);
  for (size_t d = 0; d < sp; ++d) {
    ORTB_ENFORCE_ARG(pads[d] == pads[d + sp], "ConvGrad: pads must be the same on both sides of a dimension");
    padding[d] = pads[d];
  }
  std::vector<int64_t> out_pad(sp, 0);
  auto grads = at::convolution_backward(dy, x, w, std::vector<int64_t>{w.size(0)}, strides, padding, dil, false, out_pad,
                                        n.attr_i("group", 1),
                                        {ctx.OutputNeeded(0), ctx.OutputNeeded(1), ctx.OutputCount() > 2 && ctx.OutputNeeded(2)});
  if (ctx.OutputNeeded(0)) ctx.SetOutput(0, std::get<0>(grads));
  if (ctx.OutputNeeded(1)) ctx.SetOutput(1, std::get<1>(grads));
  if (ctx.OutputCount() > 2 && ctx.OutputNeeded(2)) ctx.SetOutput(2, std::get<2>(grads));
}

void DropoutGrad(Ctx& ctx) {  // (dy, mask, ratio?, training_mode?)
  const at::Tensor& dy = ctx.RequiredInput(0);
  const double ratio = ctx.HasInput(2) ? ctx.Input(2).item<double>() : 0.5;
  const bool training = !ctx.HasInput(3) || ctx.Input(3).item<bool>();
  if (!training || ratio == 0.0) {
    ctx.SetOutput(0, dy);
  } else {
    ctx.SetOutput(0, dy * ctx.RequiredInput(1).to(dy.scalar_type()) * (1.0 / (1.0 - ratio)));
  }
}

void DivGrad(Ctx& ctx) {  // (dY, A, B) -> (dA, dB)
  const at::Tensor& dy = ctx.RequiredInput(0);
  const at::Tensor& a = ctx.RequiredInput(1);
  const at::Tensor& b = ctx.RequiredInput(2);
  if (ctx.OutputNeeded(0)) ctx.SetOutput(0, at::sum_to(dy / b, a.sizes()));
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, at::sum_to(-dy * a / (b * b), b.sizes()));
}

void SumToShape(Ctx& ctx) { ctx.SetOutput(0, at::sum_to(ctx.RequiredInput(0), ctx.RequiredInput(1).sizes()).contiguous()); }

void ReduceSumTraining(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  std::vector<int64_t> axes = ctx.HasInput(1) ? HostInts(ctx.Input(1)) : std::vector<int64_t>{};
  const bool keep = ctx.node().attr_i("keepdims", 1) != 0;
  if (axes.empty()) {
    if (ctx.node().attr_i("noop_with_empty_axes", 0) != 0) {
      ctx.SetOutput(0, x);
      return;
    }
    for (int64_t d = 0; d < x.dim(); ++d) axes.push_back(d);
  }
  ctx.SetOutput(0, axes.empty() ? x : x.sum(axes, keep));
}

void BroadcastGradientArgs(Ctx& ctx) {  // axes of the broadcast result over which each operand's gradient is summed
  std::vector<int64_t> a = HostInts(ctx.RequiredInput(0)), b = HostInts(ctx.RequiredInput(1));
  const size_t rank = std::max(a.size(), b.size());
  std::vector<int64_t> ra, rb;
  for (size_t d = 0; d < rank; ++d) {
    const int64_t da = d + a.size() >= rank ? a[d + a.size() - rank] : 1, db = d + b.size() >= rank ? b[d + b.size() - rank] : 1;
    ORTB_ENFORCE_ARG(da == db || da == 1 || db == 1, "BroadcastGradientArgs: shapes do not broadcast");
    if (da == 1 && (db != 1 || d + a.size() < rank)) ra.push_back(static_cast<int64_t>(d));
    if (db == 1 && (da != 1 || d + b.size() < rank)) rb.push_back(static_cast<int64_t>(d));
  }
  auto opts = at::TensorOptions().dtype(at::kLong);
  if (ctx.OutputNeeded(0)) ctx.SetOutput(0, at::tensor(ra, opts));
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, at::tensor(rb, opts));
}

void SplitTraining(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), x.dim());
  std::vector<at::Tensor> parts = ctx.HasInput(1) ? x.split_with_sizes(HostInts(ctx.Input(1)), axis)
                                                  : x.chunk(ctx.OutputCount(), axis);
  ORTB_ENFORCE_ARG(static_cast<int>(parts.size()) == ctx.OutputCount(), "SplitTraining: ", parts.size(), " parts for ", ctx.OutputCount(), " outputs");
  for (int i = 0; i < ctx.OutputCount(); ++i) ctx.SetOutput(i, parts[static_cast<size_t>(i)].contiguous());
}

void ConcatTraining(Ctx& ctx) {
  std::vector<at::Tensor> in;
  std::vector<int64_t> lens;
  const int64_t axis = NormAxis(ctx.node().attr_i("axis", 0), ctx.RequiredInput(0).dim());
  for (int i = 0; i < ctx.InputCount(); ++i) {
    in.push_back(ctx.RequiredInput(i));
    lens.push_back(in.back().size(axis));
  }
  ctx.SetOutput(0, at::cat(in, axis));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, at::tensor(lens, at::TensorOptions().dtype(at::kLong)));
}

// ---- accumulation, optimizers, scaling ----------------------------------------------------------------------------
void InPlaceAccumulatorV2(Ctx& ctx) {  // (buffer, value, overwrite?) -> (updated flag, buffer)
  c10::NoGradGuard no_grad;
  at::Tensor buf = ctx.RequiredInput(0);
  const at::Tensor& v = ctx.RequiredInput(1);
  if (ctx.HasInput(2) && ctx.Input(2).item<bool>()) {
    buf.copy_(v);
  } else {
    buf.add_(v.to(buf.scalar_type()));
  }
  ctx.SetOutput(0, at::ones({1}, at::TensorOptions().dtype(at::kBool)));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, buf);
}

void InPlaceAccumulator(Ctx& ctx) {  // (old_sum, value, update_signal?) -> new_sum
  c10::NoGradGuard no_grad;
  at::Tensor buf = ctx.RequiredInput(0);
  if (!ctx.HasInput(2) || ctx.Input(2).item<bool>()) buf.add_(ctx.RequiredInput(1).to(buf.scalar_type()));
  ctx.SetOutput(0, buf);
}

void ZeroGradient(Ctx& ctx) {
  c10::NoGradGuard no_grad;
  at::Tensor g = ctx.RequiredInput(0);
  g.zero_();
  ctx.SetOutput(0, g);
}

bool UpdateAllowed(Ctx& ctx, int signal_input) { return !ctx.HasInput(signal_input) || ctx.Input(signal_input).item<bool>(); }

void SgdOptimizerV2(Ctx& ctx) {  // (lr, weights, gradients, update_signal?) -> (flag, weights)
  c10::NoGradGuard no_grad;
  const double lr = ctx.RequiredInput(0).item<double>();
  const auto& w = SeqInput(ctx, 1, "weights");
  const auto& g = SeqInput(ctx, 2, "gradients");
  ORTB_ENFORCE_ARG(w.size() == g.size(), "SGDOptimizerV2: ", w.size(), " weights and ", g.size(), " gradients");
  const bool go = UpdateAllowed(ctx, 3);
  if (go) {
    for (size_t i = 0; i < w.size(); ++i) const_cast<at::Tensor&>(w[i]).add_(g[i].to(w[i].scalar_type()), -lr);
  }
  ctx.SetOutput(0, at::full({1}, go, at::TensorOptions().dtype(at::kBool)));
  if (ctx.OutputCount() > 1) ctx.SetOutputSeq(1, w);
}

void AdamWOptimizer(Ctx& ctx) {  // (lr, step, weights, gradients, m1, m2, update_signal?) -> (flag, weights, m1, m2)
  c10::NoGradGuard no_grad;
  const Node& n = ctx.node();
  const double alpha = n.attr_f("alpha", 0.9f), beta = n.attr_f("beta", 0.999f), eps = n.attr_f("epsilon", 1e-8f);
  const double decay = n.attr_f("weight_decay", 0.f);
  const int64_t mode = n.attr_i("adam_mode", 0);
  ORTB_ENFORCE_ARG(mode == 0 || mode == 1, "AdamWOptimizer: adam_mode must be 0 or 1");
  const double lr = ctx.RequiredInput(0).item<double>();
  const int64_t step = ctx.RequiredInput(1).item<int64_t>();
  const auto& w = SeqInput(ctx, 2, "weights");
  const auto& g = SeqInput(ctx, 3, "gradients");
  const auto& m1 = SeqInput(ctx, 4, "momentums_1");
  const auto& m2 = SeqInput(ctx, 5, "momentums_2");
  ORTB_ENFORCE_ARG(w.size() == g.size() && w.size() == m1.size() && w.size() == m2.size(),
                   "AdamWOptimizer: the four sequences differ in length");
  const bool go = UpdateAllowed(ctx, 6);
  if (go) {
    double ac = 1.0, bc = 1.0, lr_corrected = lr;
    if (n.attr_i("correct_bias", 1) == 1) {
      ac = 1.0 - std::pow(alpha, static_cast<double>(step));
      bc = 1.0 - std::pow(beta, static_cast<double>(step));
      lr_corrected *= std::sqrt(bc) / ac;
    }
    for (size_t i = 0; i < w.size(); ++i) {
      at::Tensor& wi = const_cast<at::Tensor&>(w[i]);
      at::Tensor& a = const_cast<at::Tensor&>(m1[i]);
      at::Tensor& b = const_cast<at::Tensor&>(m2[i]);
      at::Tensor gi = g[i].to(a.scalar_type());
      if (mode == 0) wi.mul_(1.0 - lr * decay);                 // decay first: the torch.optim.AdamW order
      a.mul_(alpha).add_(gi, 1.0 - alpha);
      b.mul_(beta).addcmul_(gi, gi, 1.0 - beta);
      if (mode == 0) {
        wi.addcdiv_(a.to(wi.scalar_type()), ((b / bc).sqrt() + eps).to(wi.scalar_type()), -lr / ac);
      } else {
        wi.addcdiv_(a.to(wi.scalar_type()), (b.sqrt() + eps).to(wi.scalar_type()), -lr_corrected);
        wi.mul_(1.0 - lr * decay);                              // decay last: the transformers-library order
      }
    }
  }
  ctx.SetOutput(0, at::full({1}, go, at::TensorOptions().dtype(at::kBool)));
  if (ctx.OutputCount() > 1) ctx.SetOutputSeq(1, w);
  if (ctx.OutputCount() > 2) ctx.SetOutputSeq(2, m1);
  if (ctx.OutputCount() > 3) ctx.SetOutputSeq(3, m2);
}

void InplaceClipGradNorm(Ctx& ctx) {
  c10::NoGradGuard no_grad;
  const auto& g = SeqInput(ctx, 0, "gradients");
  const double max_norm = ctx.node().attr_f("max_norm", 1.f);
  ORTB_ENFORCE_ARG(ctx.node().attr_s("norm_type", "fro") == "fro", "InplaceClipGradNorm: only the Frobenius norm");
  at::Tensor total = at::zeros({}, at::TensorOptions().dtype(at::kFloat));
  for (const at::Tensor& t : g) total = total + t.to(at::kFloat).pow(2).sum().cpu();
  const double coef = max_norm / (std::sqrt(total.item<double>()) + 1e-6);
  if (coef < 1.0) {
    for (const at::Tensor& t : g) const_cast<at::Tensor&>(t).mul_(coef);
  }
  ctx.SetOutputSeq(0, g);
}

void ReduceAllL2(Ctx& ctx) {
  at::Tensor total;
  for (int i = 0; i < ctx.InputCount(); ++i) {
    at::Tensor s = ctx.RequiredInput(i).to(at::kFloat).pow(2).sum();
    total = total.defined() ? total + s : s;
  }
  ctx.SetOutput(0, total.sqrt().reshape({1}).to(ctx.Input(0).scalar_type()));
}

void MixedPrecisionScale(Ctx& ctx) {  // (S, X...) -> X * S cast to `to` (one tensor per input, or one fused vector)
  const at::Tensor& s = ctx.RequiredInput(0);
  const at::ScalarType to = ToTorchType(static_cast<int32_t>(ctx.node().attr_i("to", 1)));
  std::vector<at::Tensor> out;
  for (int i = 1; i < ctx.InputCount(); ++i) out.push_back((ctx.RequiredInput(i).to(at::kFloat) * s.to(at::kFloat)).to(to));
  if (ctx.node().attr_i("fuse_outputs", 0) != 0) {
    for (at::Tensor& t : out) t = t.reshape({-1});
    ctx.SetOutput(0, at::cat(out, 0));
  } else {
    for (size_t i = 0; i < out.size(); ++i) ctx.SetOutput(static_cast<int>(i), out[i]);
  }
}

void ScaleOp(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  at::Tensor s = ctx.RequiredInput(1).to(at::kFloat);
  at::Tensor y = ctx.node().attr_i("scale_down", 0) != 0 ? x.to(at::kFloat) / s : x.to(at::kFloat) * s;
  ctx.SetOutput(0, y.to(x.scalar_type()));
}

void ScaledSum(Ctx& ctx) {
  const Node& n = ctx.node();
  at::Tensor y = ctx.RequiredInput(0) * static_cast<double>(n.attr_f("scale_0", 1.f)) +
                 ctx.RequiredInput(1) * static_cast<double>(n.attr_f("scale_1", 1.f));
  if (ctx.HasInput(2)) y = y + ctx.Input(2) * static_cast<double>(n.attr_f("scale_2", 1.f));
  ctx.SetOutput(0, y);
}

void BatchScale(Ctx& ctx) {
  static const char* const kNames[3] = {"scale_0", "scale_1", "scale_2"};
  for (int i = 0; i < ctx.OutputCount() && i < 3; ++i)
    ctx.SetOutput(i, ctx.RequiredInput(0) * static_cast<double>(ctx.node().attr_f(kNames[i], 1.f)));
}

void FakeQuant(Ctx& ctx) {  // (input, scale, zero_point) -> (output, mask of values inside the range)
  const at::Tensor& x = ctx.RequiredInput(0);
  const double lo = static_cast<double>(ctx.node().attr_i("quant_min", 0)), hi = static_cast<double>(ctx.node().attr_i("quant_max", 255));
  at::Tensor scale = ctx.RequiredInput(1).to(at::kFloat), zp = ctx.RequiredInput(2).to(at::kFloat);
  at::Tensor q = at::round(x.to(at::kFloat) / scale + zp);
  ctx.SetOutput(0, ((at::clamp(q, lo, hi) - zp) * scale).to(x.scalar_type()));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, at::logical_and(q >= lo, q <= hi));
}

void ViewOp(Ctx& ctx) {  // (input, shape_1 .. shape_n) -> consecutive pieces of the input's storage in those shapes
  at::Tensor flat = ctx.RequiredInput(0).reshape({-1});
  int64_t at_elem = 0;
  for (int i = 0; i < ctx.OutputCount(); ++i) {
    std::vector<int64_t> shape = HostInts(ctx.RequiredInput(i + 1));
    int64_t count = 1;
    for (int64_t d : shape) count *= d;
    ctx.SetOutput(i, flat.narrow(0, at_elem, count).reshape(shape));
    at_elem += count;
  }
}

}  // namespace

void RegisterTrainingKernels(KernelRegistry& r) {
  r.RegisterFn(MS, "ReluGrad", 1, kMax, ReluGrad);
  r.RegisterFn(MS, "GeluGrad", 1, kMax, GeluGrad);
  r.RegisterFn(MS, "FastGeluGrad", 1, kMax, FastGeluGrad);
  r.RegisterFn(MS, "BiasGeluGrad_dX", 1, kMax, [](Ctx& c) { BiasGeluGradDx(c, false); });
  r.RegisterFn(MS, "BiasFastGeluGrad_dX", 1, kMax, [](Ctx& c) { BiasGeluGradDx(c, true); });
  r.RegisterFn(MS, "QuickGeluGrad", 1, kMax, QuickGeluGrad);
  r.RegisterFn(MS, "SigmoidGrad", 1, kMax, SigmoidGrad);
  r.RegisterFn(MS, "TanhGrad", 1, kMax, TanhGrad);
  r.RegisterFn(MS, "LeakyReluGrad", 1, kMax, LeakyReluGrad);
  r.RegisterFn(MS, "SoftmaxGrad", 1, kMax, [](Ctx& c) { SoftmaxGradImpl(c, false, false); });
  r.RegisterFn(MS, "SoftmaxGrad_13", 1, kMax, [](Ctx& c) { SoftmaxGradImpl(c, false, true); });
  r.RegisterFn(MS, "LogSoftmaxGrad", 1, kMax, [](Ctx& c) { SoftmaxGradImpl(c, true, false); });
  r.RegisterFn(MS, "LogSoftmaxGrad_13", 1, kMax, [](Ctx& c) { SoftmaxGradImpl(c, true, true); });
  r.RegisterFn(MS, "LayerNormalizationGrad", 1, kMax, [](Ctx& c) { LayerNormGrad(c, false); });
  r.RegisterFn(MS, "SimplifiedLayerNormalizationGrad", 1, kMax, [](Ctx& c) { LayerNormGrad(c, true); });
  r.RegisterFn(MS, "BatchNormalizationGrad", 1, kMax, BatchNormGrad);
  r.RegisterFn(MS, "SoftmaxCrossEntropyLossInternal", 1, kMax, SceInternal, {3});
  r.RegisterFn(MS, "SoftmaxCrossEntropyLossInternalGrad", 1, kMax, [](Ctx& c) { SceGrad(c, false); }, {4});
  r.RegisterFn(MS, "SoftmaxCrossEntropyLossGrad", 1, kMax, [](Ctx& c) { SceGrad(c, true); });
  r.RegisterFn(MS, "GatherGrad", 1, kMax, GatherGrad, {0});
  r.RegisterFn(MS, "GatherElementsGrad", 1, kMax, GatherElementsGrad, {1});
  r.RegisterFn(MS, "GatherNDGrad", 1, kMax, GatherNDGrad, {0});
  r.RegisterFn(MS, "SliceGrad", 1, kMax, SliceGrad, {1, 2, 3, 4, 5});
  r.RegisterFn(MS, "ConvGrad", 1, kMax, ConvGrad);
  r.RegisterFn(MS, "DropoutGrad", 1, kMax, DropoutGrad, {2, 3});
  r.RegisterFn(MS, "DivGrad", 1, kMax, DivGrad);
  r.RegisterFn("com.ortb200", "SumToShape", 1, kMax, SumToShape);
  r.RegisterFn(MS, "ReduceSumTraining", 1, kMax, ReduceSumTraining, {1});
  r.RegisterFn(MS, "BroadcastGradientArgs", 1, kMax, BroadcastGradientArgs, {0, 1});
  r.RegisterFn(MS, "SplitTraining", 1, kMax, SplitTraining, {1});
  r.RegisterFn(MS, "ConcatTraining", 1, kMax, ConcatTraining);
  r.RegisterFn(MS, "InPlaceAccumulatorV2", 1, kMax, InPlaceAccumulatorV2, {2});
  r.RegisterFn(MS, "InPlaceAccumulator", 1, kMax, InPlaceAccumulator, {2});
  r.RegisterFn(MS, "ZeroGradient", 1, kMax, ZeroGradient);
  r.RegisterFn(MS, "SGDOptimizerV2", 1, kMax, SgdOptimizerV2, {0, 3});
  r.RegisterFn(MS, "AdamWOptimizer", 1, kMax, AdamWOptimizer, {0, 1, 6});
  r.RegisterFn(MS, "InplaceClipGradNorm", 1, kMax, InplaceClipGradNorm);
  r.RegisterFn(MS, "ReduceAllL2", 1, kMax, ReduceAllL2);
  r.RegisterFn(MS, "MixedPrecisionScale", 1, kMax, MixedPrecisionScale);
  r.RegisterFn(MS, "Scale", 1, kMax, ScaleOp);
  r.RegisterFn(MS, "ScaledSum", 1, kMax, ScaledSum);
  r.RegisterFn(MS, "BatchScale", 1, kMax, BatchScale);
  r.RegisterFn(MS, "FakeQuant", 1, kMax, FakeQuant);
  r.RegisterFn(MS, "FakeQuantGrad", 1, kMax, [](Ctx& c) { c.SetOutput(0, c.RequiredInput(0) * c.RequiredInput(1).to(c.Input(0).scalar_type())); });
  r.RegisterFn(MS, "View", 1, kMax, ViewOp);
  r.RegisterFn(MS, "IsFinite", 1, kMax, [](Ctx& c) { c.SetOutput(0, at::isfinite(c.RequiredInput(0))); });
  r.RegisterFn(MS, "All", 1, kMax, [](Ctx& c) { c.SetOutput(0, c.RequiredInput(0).all().reshape({1})); });
  r.RegisterFn(MS, "Group", 1, kMax, [](Ctx& c) { c.SetOutput(0, at::ones({1}, at::TensorOptions().dtype(at::kBool))); });
  r.RegisterFn(MS, "PassThrough", 1, kMax, [](Ctx& c) {
    for (int i = 0; i < c.OutputCount() && i < c.InputCount(); ++i) c.SetOutput(i, c.Input(i));
  });
}

}  // namespace ortb
