// Element-wise ONNX operators written against ATen.  Device-agnostic: they are
// the CPU execution provider and the GPU provider's long tail (the reference
// splits these between core/providers/cpu/math + activation and
// core/providers/cuda/math/{unary,binary,variadic}_elementwise_ops_impl.cu).
#include <ATen/ATen.h>

#include <cmath>
#include <limits>

#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

at::Tensor CastTo(const at::Tensor& x, int32_t onnx_type) {
  const at::ScalarType st = ToTorchType(onnx_type);
  if (x.scalar_type() == st) return x;
  if (st == at::kBool) return x.ne(0);
  if (c10::isIntegralType(st, false) && c10::isFloatingType(x.scalar_type())) {
    // float -> int truncates toward zero; go through int64 for unsigned targets
    return at::trunc(x.to(at::kDouble)).to(at::kLong).to(st);
  }
  return x.to(st);
}

at::Tensor VariadicReduce(Ctx& ctx, const std::function<at::Tensor(const at::Tensor&, const at::Tensor&)>& f) {
  at::Tensor acc = ctx.RequiredInput(0);
  for (int i = 1; i < ctx.InputCount(); ++i)
    if (ctx.HasInput(i)) acc = f(acc, ctx.Input(i));
  return acc;
}

at::Tensor Gelu(const at::Tensor& x, bool tanh_approx) { return at::gelu(x, tanh_approx ? "tanh" : "none"); }

}  // namespace

#define ORTB_UNARY(NAME, SINCE, EXPR)                                                   \
  r.RegisterFn("", NAME, SINCE, kMax, [](Ctx& ctx) {                                    \
    const at::Tensor& x = ctx.RequiredInput(0);                                         \
    ctx.SetOutput(0, (EXPR));                                                           \
  })
#define ORTB_BINARY(NAME, SINCE, EXPR)                                                  \
  r.RegisterFn("", NAME, SINCE, kMax, [](Ctx& ctx) {                                    \
    const at::Tensor& a = ctx.RequiredInput(0);                                         \
    const at::Tensor& b = ctx.RequiredInput(1);                                         \
    ctx.SetOutput(0, (EXPR));                                                           \
  })

void RegisterElementwiseKernels(KernelRegistry& r) {
  ORTB_UNARY("Abs", 1, at::abs(x));
  ORTB_UNARY("Neg", 1, at::neg(x));
  ORTB_UNARY("Floor", 1, at::floor(x));
  ORTB_UNARY("Ceil", 1, at::ceil(x));
  ORTB_UNARY("Round", 1, at::round(x));  // half to even, as ONNX specifies
  ORTB_UNARY("Sqrt", 1, at::sqrt(x));
  ORTB_UNARY("Reciprocal", 1, at::reciprocal(x));
  ORTB_UNARY("Exp", 1, at::exp(x));
  ORTB_UNARY("Log", 1, at::log(x));
  ORTB_UNARY("Sin", 1, at::sin(x));
  ORTB_UNARY("Cos", 1, at::cos(x));
  ORTB_UNARY("Tan", 1, at::tan(x));
  ORTB_UNARY("Asin", 1, at::asin(x));
  ORTB_UNARY("Acos", 1, at::acos(x));
  ORTB_UNARY("Atan", 1, at::atan(x));
  ORTB_UNARY("Sinh", 1, at::sinh(x));
  ORTB_UNARY("Cosh", 1, at::cosh(x));
  ORTB_UNARY("Tanh", 1, at::tanh(x));
  ORTB_UNARY("Asinh", 1, at::asinh(x));
  ORTB_UNARY("Acosh", 1, at::acosh(x));
  ORTB_UNARY("Atanh", 1, at::atanh(x));
  ORTB_UNARY("Erf", 1, at::erf(x));
  ORTB_UNARY("Sigmoid", 1, at::sigmoid(x));
  ORTB_UNARY("Relu", 1, at::relu(x));
  ORTB_UNARY("Sign", 1, at::sign(x));
  ORTB_UNARY("Not", 1, at::logical_not(x));
  ORTB_UNARY("IsNaN", 1, at::isnan(x));
  ORTB_UNARY("Softsign", 1, x / (at::abs(x) + 1));
  ORTB_UNARY("Identity", 1, x);
  ORTB_UNARY("Mish", 1, x * at::tanh(at::softplus(x)));
  ORTB_UNARY("BitwiseNot", 1, at::bitwise_not(x));
  ORTB_UNARY("Softplus", 1, at::softplus(x));

  r.RegisterFn("", "IsInf", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const bool neg = ctx.node().attr_i("detect_negative", 1) != 0, pos = ctx.node().attr_i("detect_positive", 1) != 0;
    at::Tensor out = at::zeros_like(x, x.options().dtype(at::kBool));
    if (pos) out = out.logical_or(at::isposinf(x));
    if (neg) out = out.logical_or(at::isneginf(x));
    ctx.SetOutput(0, out);
  });
  r.RegisterFn("", "LeakyRelu", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::leaky_relu(ctx.RequiredInput(0), ctx.node().attr_f("alpha", 0.01f)));
  });
  r.RegisterFn("", "Elu", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::elu(ctx.RequiredInput(0), ctx.node().attr_f("alpha", 1.0f)));
  });
  r.RegisterFn("", "Celu", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::celu(ctx.RequiredInput(0), ctx.node().attr_f("alpha", 1.0f)));
  });
  r.RegisterFn("", "Selu", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const float alpha = ctx.node().attr_f("alpha", 1.67326319217681884765625f);
    const float gamma = ctx.node().attr_f("gamma", 1.05070102214813232421875f);
    ctx.SetOutput(0, at::where(x > 0, x * gamma, (at::exp(x) - 1) * (alpha * gamma)).to(x.scalar_type()));
  });
  r.RegisterFn("", "HardSigmoid", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::clamp(x * ctx.node().attr_f("alpha", 0.2f) + ctx.node().attr_f("beta", 0.5f), 0, 1));
  });
  r.RegisterFn("", "HardSwish", 14, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x * at::clamp(x * (1.0 / 6.0) + 0.5, 0, 1));
  });
  r.RegisterFn("", "ThresholdedRelu", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::where(x > ctx.node().attr_f("alpha", 1.0f), x, at::zeros_like(x)));
  });
  r.RegisterFn("", "Shrink", 9, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const float bias = ctx.node().attr_f("bias", 0.f), lambd = ctx.node().attr_f("lambd", 0.5f);
    ctx.SetOutput(0, at::where(x < -lambd, x + bias, at::where(x > lambd, x - bias, at::zeros_like(x))));
  });
  r.RegisterFn("", "Gelu", 20, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, Gelu(ctx.RequiredInput(0), ctx.node().attr_s("approximate", "none") == "tanh"));
  });
  r.RegisterFn("", "Swish", 24, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x * at::sigmoid(x * ctx.node().attr_f("alpha", 1.0f)));
  });
  r.RegisterFn("", "Clip", 1, 10, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::clamp(x, ctx.node().attr_f("min", -std::numeric_limits<float>::max()),
                               ctx.node().attr_f("max", std::numeric_limits<float>::max())));
  });
  r.RegisterFn("", "Clip", 11, kMax, [](Ctx& ctx) {
    at::Tensor x = ctx.RequiredInput(0);
    if (ctx.HasInput(1)) x = at::maximum(x, ctx.Input(1).to(x.device()));
    if (ctx.HasInput(2)) x = at::minimum(x, ctx.Input(2).to(x.device()));
    ctx.SetOutput(0, x);
  });
  r.RegisterFn("", "Cast", 1, kMax, [](Ctx& ctx) {
    const int32_t to = static_cast<int32_t>(ctx.node().attr_i("to", 1));
    if (CastWithStrings(ctx, to)) return;
    ctx.SetOutput(0, CastTo(ctx.RequiredInput(0), to));
  });
  r.RegisterFn("", "CastLike", 15, kMax, [](Ctx& ctx) {
    const int32_t to = ctx.InputIsString(1) ? static_cast<int32_t>(pb::STRING) : ToOnnxType(ctx.RequiredInput(1).scalar_type());
    if (CastWithStrings(ctx, to)) return;
    ctx.SetOutput(0, CastTo(ctx.RequiredInput(0), to));
  });
  r.RegisterFn("", "Dropout", 1, kMax, [](Ctx& ctx) {
    // inference: identity, mask of ones
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x);
    if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ctx.SetOutput(1, at::ones_like(x, x.options().dtype(at::kBool)));
  });

  ORTB_BINARY("Add", 1, at::add(a, b));
  ORTB_BINARY("Sub", 1, at::sub(a, b));
  ORTB_BINARY("Mul", 1, at::mul(a, b));
  ORTB_BINARY("Div", 1, c10::isIntegralType(a.scalar_type(), true) ? at::div(a, b, "trunc") : at::div(a, b));
  ORTB_BINARY("Pow", 1, at::pow(a, b.scalar_type() == a.scalar_type() ? b : b.to(at::result_type(a, b))).to(a.scalar_type()));
  ORTB_BINARY("And", 1, at::logical_and(a, b));
  ORTB_BINARY("Or", 1, at::logical_or(a, b));
  ORTB_BINARY("Xor", 1, at::logical_xor(a, b));
  ORTB_BINARY("Equal", 1, at::eq(a, b));
  ORTB_BINARY("Less", 1, at::lt(a, b));
  ORTB_BINARY("Greater", 1, at::gt(a, b));
  ORTB_BINARY("LessOrEqual", 12, at::le(a, b));
  ORTB_BINARY("GreaterOrEqual", 12, at::ge(a, b));
  ORTB_BINARY("BitwiseAnd", 18, at::bitwise_and(a, b));
  ORTB_BINARY("BitwiseOr", 18, at::bitwise_or(a, b));
  ORTB_BINARY("BitwiseXor", 18, at::bitwise_xor(a, b));
  ORTB_BINARY("PRelu", 1, at::where(a < 0, a * b, a));
  r.RegisterFn("", "Mod", 10, kMax, [](Ctx& ctx) {
    const at::Tensor& a = ctx.RequiredInput(0);
    const at::Tensor& b = ctx.RequiredInput(1);
    ctx.SetOutput(0, ctx.node().attr_i("fmod", 0) ? at::fmod(a, b) : at::remainder(a, b));
  });
  r.RegisterFn("", "BitShift", 11, kMax, [](Ctx& ctx) {
    const at::Tensor& a = ctx.RequiredInput(0);
    const at::Tensor& b = ctx.RequiredInput(1);
    ctx.SetOutput(0, ctx.node().attr_s("direction", "LEFT") == "LEFT" ? at::bitwise_left_shift(a, b)
                                                                         : at::bitwise_right_shift(a, b));
  });
  r.RegisterFn("", "Where", 9, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::where(ctx.RequiredInput(0), ctx.RequiredInput(1), ctx.RequiredInput(2)));
  });
  r.RegisterFn("", "Sum", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, VariadicReduce(ctx, [](const at::Tensor& a, const at::Tensor& b) { return at::add(a, b); }));
  });
  r.RegisterFn("", "Max", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, VariadicReduce(ctx, [](const at::Tensor& a, const at::Tensor& b) { return at::maximum(a, b); }));
  });
  r.RegisterFn("", "Min", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, VariadicReduce(ctx, [](const at::Tensor& a, const at::Tensor& b) { return at::minimum(a, b); }));
  });
  r.RegisterFn("", "Mean", 1, kMax, [](Ctx& ctx) {
    int n = 0;
    for (int i = 0; i < ctx.InputCount(); ++i) n += ctx.HasInput(i) ? 1 : 0;
    at::Tensor s = VariadicReduce(ctx, [](const at::Tensor& a, const at::Tensor& b) { return at::add(a, b); });
    ctx.SetOutput(0, s / n);
  });
}

}  // namespace ortb
