// The QOrdered* family (int8 tensors with a cuBLASLt "order" attribute) for the orders that are plain memory layouts:
// activations and outputs in ORDER_ROW, weights in ORDER_ROW or ORDER_COL (ORDER_COL: the buffer holds the transpose).
// The tiled orders (COL32, COL4_4R2_8C, COL32_2R_4R4) are private layouts of one GEMM library and are rejected.
// Reference kernels: onnxruntime/contrib_ops/cuda/quantization/qordered_ops/ (qordered_qdq.cc, qordered_matmul.cc,
// qordered_layer_norm.cc, qordered_unary_ops.cc, qordered_attention.cc, qordered_longformer_attention.cc);
// semantics follow docs/ContribOperators.md of the reference and its tests (test/contrib_ops/qordered_*_test.cc).
#include <ATen/ATen.h>

#include <cmath>

#include "contrib_math.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = "com.microsoft";
enum Order : int64_t { kCol = 0, kRow = 1 };

void RequireRow(const Node& n, const char* attr) {
  if (!n.has_attr(attr)) return;
  ORTB_ENFORCE(n.attr_i(attr, kRow) == kRow, n.op_type, ": ", attr, " = ", n.attr_i(attr, kRow),
               " is not supported (activations and outputs must be ORDER_ROW = 1)");
}

// weight declared as [rows, cols]; ORDER_COL means the buffer holds it column by column
at::Tensor LogicalWeight(const Node& n, const at::Tensor& w, const char* attr) {
  const int64_t order = n.attr_i(attr, kRow);
  ORTB_ENFORCE(order == kRow || order == kCol, n.op_type, ": ", attr, " = ", order, " is not supported (ORDER_ROW = 1 or ORDER_COL = 0)");
  ORTB_ENFORCE_ARG(w.dim() == 2, n.op_type, ": weights must be 2-D");
  if (order == kRow) return w;
  return w.contiguous().reshape({w.size(1), w.size(0)}).t();
}

at::Tensor Scale(const Ctx& ctx, int i) { return ctx.RequiredInput(i).to(at::kFloat); }

at::Tensor QuantizeS8(const at::Tensor& x, const at::Tensor& scale) {
  return at::clamp(at::round(x.to(at::kFloat) / scale), -128, 127).to(at::kChar);
}

void QuantizeWithOrderImpl(Ctx& ctx) {
  RequireRow(ctx.node(), "order_input");
  RequireRow(ctx.node(), "order_output");
  ctx.SetOutput(0, QuantizeS8(ctx.RequiredInput(0), Scale(ctx, 1)));
}

void DequantizeWithOrderImpl(Ctx& ctx) {
  RequireRow(ctx.node(), "order_input");
  RequireRow(ctx.node(), "order_output");
  const int64_t to = ctx.node().attr_i("to", 1);
  ORTB_ENFORCE_ARG(to == 1 || to == 10, "DequantizeWithOrder: `to` must be 1 (float) or 10 (float16)");
  at::Tensor y = ctx.RequiredInput(0).to(at::kFloat) * Scale(ctx, 1);
  ctx.SetOutput(0, to == 10 ? y.to(at::kHalf) : y);
}

void QOrderedGeluImpl(Ctx& ctx) {
  RequireRow(ctx.node(), "order_X");
  RequireRow(ctx.node(), "order_Y");
  at::Tensor x = ctx.RequiredInput(0).to(at::kFloat) * Scale(ctx, 1);
  ctx.SetOutput(0, QuantizeS8(at::gelu(x), Scale(ctx, 2)));
}

void QOrderedLayerNormImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  RequireRow(n, "order_X");
  RequireRow(n, "order_Y");
  at::Tensor x = ctx.RequiredInput(0).to(at::kFloat) * Scale(ctx, 1);
  int64_t axis = n.attr_i("axis", -1);
  if (axis < 0) axis += x.dim();
  ORTB_ENFORCE_ARG(axis == x.dim() - 1, "QOrderedLayerNormalization: normalises the last axis only");
  at::Tensor gamma = ctx.RequiredInput(2).to(at::kFloat);
  c10::optional<at::Tensor> beta = ctx.HasInput(3) ? c10::optional<at::Tensor>(ctx.Input(3).to(at::kFloat)) : c10::nullopt;
  at::Tensor y = at::layer_norm(x, {x.size(-1)}, gamma, beta, n.attr_f("epsilon", 1e-5f));
  ctx.SetOutput(0, QuantizeS8(y, Scale(ctx, 4)));
}

// Y = saturate(round((sA * sB / sY) * A @ B + bias / sY + (sC / sY) * C))
void QOrderedMatMulImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  RequireRow(n, "order_A");
  RequireRow(n, "order_Y");
  const at::Tensor& A = ctx.RequiredInput(0);
  at::Tensor B = LogicalWeight(n, ctx.RequiredInput(2), "order_B").to(at::kFloat);  // [K, N]
  ORTB_ENFORCE_ARG(A.size(-1) == B.size(0), "QOrderedMatMul: inner dimensions differ");
  at::Tensor sB = Scale(ctx, 3).reshape({-1});                                       // scalar or one per column of B
  at::Tensor sY = Scale(ctx, 4);
  // int8 products summed in fp32 would round above 2^24: accumulate in double (exact for any K in reach)
  at::Tensor acc = at::matmul(A.to(at::kDouble), B.to(at::kDouble)).to(at::kFloat);
  at::Tensor y = acc * (Scale(ctx, 1) * sB / sY);
  if (ctx.HasInput(5)) y = y + ctx.Input(5).to(at::kFloat) / sY;
  if (ctx.HasInput(6)) {
    ORTB_ENFORCE_ARG(ctx.HasInput(7), "QOrderedMatMul: C needs scale_C");
    at::Tensor C = ctx.Input(6).to(at::kFloat);
    if (C.dim() == 2 && y.dim() == 3) C = C.unsqueeze(0);
    y = y + C * (ctx.Input(7).to(at::kFloat) / sY);
  }
  ctx.SetOutput(0, at::clamp(at::round(y), -128, 127).to(at::kChar));
}

// value -> int8 grid of `scale` -> value (what the next integer GEMM sees)
at::Tensor FakeQuant(const at::Tensor& x, const at::Tensor& scale) { return at::clamp(at::round(x / scale), -128, 127) * scale; }

// Self attention whose three projections, probabilities and output live on int8 grids:
//   Q = q8((x sx) (Wq swq) + bq; sQ) (K, V alike), P = q8(softmax(q8(Q K^T; s_qk) / sqrt(H) + mask); s_softmax), out = q8(P V; s_out)
void QOrderedAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  RequireRow(n, "order_input");
  RequireRow(n, "order_output");
  ORTB_ENFORCE(!ctx.HasInput(18) && !ctx.HasInput(19), "QOrderedAttention: past and attention_bias are not supported (as in the reference)");
  const at::Tensor& in = ctx.RequiredInput(0);
  ORTB_ENFORCE_ARG(in.dim() == 3, "QOrderedAttention: input must be [batch, sequence, hidden]");
  const int64_t B = in.size(0), S = in.size(1), N = n.attr_i("num_heads", 1);
  at::Tensor x = in.to(at::kFloat) * Scale(ctx, 1);
  auto project = [&](int w_idx, int ws_idx, int b_idx, int s_idx) {
    at::Tensor w = LogicalWeight(n, ctx.RequiredInput(w_idx), "order_weight").to(at::kFloat) * Scale(ctx, ws_idx).reshape({1, -1});
    at::Tensor g = at::matmul(x, w) + ctx.RequiredInput(b_idx).to(at::kFloat);
    g = FakeQuant(g, Scale(ctx, s_idx));
    return g.reshape({B, S, N, g.size(-1) / N}).transpose(1, 2);  // [B, N, S, H]
  };
  at::Tensor q = project(5, 8, 11, 2), k = project(6, 9, 12, 3), v = project(7, 10, 13, 4);
  const int64_t H = q.size(-1);
  // the raw products sit on the int8 grid of scale_QKT_gemm; 1 / sqrt(H) belongs to the softmax step
  at::Tensor scores = at::matmul(q, k.transpose(-1, -2));
  if (ctx.HasInput(14)) scores = FakeQuant(scores, Scale(ctx, 14));
  scores = scores / std::sqrt(static_cast<double>(H));
  if (ctx.HasInput(17)) scores = scores + contrib::AttentionMaskBias(ctx.Input(17), B, S, S, -10000.f, scores.device());
  if (n.attr_i("unidirectional", 0) != 0) {
    at::Tensor causal = at::ones({S, S}, scores.options().dtype(at::kBool)).tril();
    scores = scores.masked_fill(causal.logical_not(), -std::numeric_limits<float>::infinity());
  }
  at::Tensor p = at::softmax(scores, -1);
  if (ctx.HasInput(15)) p = FakeQuant(p, Scale(ctx, 15));
  at::Tensor out = at::matmul(p, v).transpose(1, 2).reshape({B, S, N * H});
  ctx.SetOutput(0, QuantizeS8(out, Scale(ctx, 16)));
}

void QOrderedLongformerImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  RequireRow(n, "order_input");
  RequireRow(n, "order_output");
  at::Tensor x = ctx.RequiredInput(0).to(at::kFloat) * Scale(ctx, 1);
  auto project = [&](int w_idx, int ws_idx, int b_idx, const char* order_attr, int s_idx) {
    at::Tensor w = LogicalWeight(n, ctx.RequiredInput(w_idx), order_attr).to(at::kFloat) * Scale(ctx, ws_idx).reshape({1, -1});
    at::Tensor bias = ctx.RequiredInput(b_idx).to(at::kFloat);
    if (b_idx == 4) bias = bias * Scale(ctx, 5);  // the local projection's bias carries its own scale
    return FakeQuant(at::matmul(x, w) + bias, Scale(ctx, s_idx));
  };
  at::Tensor qkv = project(2, 3, 4, "order_weight", 6);
  at::Tensor gqkv = project(8, 9, 10, "order_global_weight", 11);
  at::Tensor y = contrib::LongformerCore(qkv, gqkv, ctx.RequiredInput(7), ctx.RequiredInput(12), n.attr_i("num_heads", 1), n.attr_i("window", 1));
  ctx.SetOutput(0, QuantizeS8(y, Scale(ctx, 13)));
}

}  // namespace

void RegisterQOrderedKernels(KernelRegistry& r) {
  r.RegisterFn(MS, "QuantizeWithOrder", 1, kMax, QuantizeWithOrderImpl);
  r.RegisterFn(MS, "DequantizeWithOrder", 1, kMax, DequantizeWithOrderImpl);
  r.RegisterFn(MS, "QOrderedGelu", 1, kMax, QOrderedGeluImpl);
  r.RegisterFn(MS, "QOrderedLayerNormalization", 1, kMax, QOrderedLayerNormImpl);
  r.RegisterFn(MS, "QOrderedMatMul", 1, kMax, QOrderedMatMulImpl);
  r.RegisterFn(MS, "QOrderedAttention", 1, kMax, QOrderedAttentionImpl);
  r.RegisterFn(MS, "QOrderedLongformerAttention", 1, kMax, QOrderedLongformerImpl);
}

}  // namespace ortb
