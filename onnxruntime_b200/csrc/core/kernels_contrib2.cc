// More com.microsoft contrib operators written against ATen (device-agnostic: the same code serves the CPU
// provider and, on CUDA tensors, the GPU provider).  Semantics follow docs/ContribOperators.md of the reference and
// the kernels named beside each operator.
#include <ATen/ATen.h>

#include <algorithm>
#include <cmath>
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

// RemovePadding (onnxruntime/contrib_ops/cuda/bert/bert_padding.cu): rows of real tokens first, in batch order.
// token_offset lists the flat [batch, sequence] index of every real token, then of every padding token.
void RemovePaddingImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const int64_t B = x.size(0), S = x.size(1);
  const std::vector<int64_t> counts = HostInts(ctx.RequiredInput(1));
  ORTB_ENFORCE(static_cast<int64_t>(counts.size()) == B, "RemovePadding: sequence_token_count must have batch_size entries");
  std::vector<int32_t> offsets, pads, cum(B + 1, 0);
  int64_t max_len = 0;
  for (int64_t b = 0; b < B; ++b) {
    ORTB_ENFORCE(counts[b] >= 0 && counts[b] <= S, "RemovePadding: token count out of range");
    for (int64_t s = 0; s < S; ++s) (s < counts[b] ? offsets : pads).push_back(static_cast<int32_t>(b * S + s));
    cum[b + 1] = cum[b] + static_cast<int32_t>(counts[b]);
    max_len = std::max(max_len, counts[b]);
  }
  const int64_t total = static_cast<int64_t>(offsets.size());
  offsets.insert(offsets.end(), pads.begin(), pads.end());
  at::Tensor off = at::tensor(offsets, at::kInt);
  at::Tensor idx = off.narrow(0, 0, total).to(x.device(), at::kLong);
  ctx.SetOutput(0, x.reshape({B * S, x.size(2)}).index_select(0, idx));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, off.reshape({B, S}).to(x.device()));
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, at::tensor(cum, at::kInt).to(x.device()));
  if (ctx.OutputCount() > 3) ctx.SetOutput(3, at::tensor({static_cast<int32_t>(max_len)}, at::kInt).to(x.device()));
}

void RestorePaddingImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);          // [total_tokens, hidden]
  const at::Tensor& off = ctx.RequiredInput(1);        // [B, S]
  const int64_t B = off.size(0), S = off.size(1), T = x.size(0);
  at::Tensor out = at::zeros({B * S, x.size(1)}, x.options());
  out.index_copy_(0, off.reshape({-1}).narrow(0, 0, T).to(x.device(), at::kLong), x);
  ctx.SetOutput(0, out.reshape({B, S, x.size(1)}));
}

// RelativePositionBias (contrib_ops/cuda/bert/relative_attn_bias_impl.cu, buildRelativeAttentionBias): T5 buckets.
// The table is read as [num_heads, num_buckets] in memory.
void RelativePositionBiasImpl(Ctx& ctx) {
  const at::Tensor& table = ctx.RequiredInput(0);
  const int64_t qlen = HostInts(ctx.RequiredInput(1)).at(0), klen = HostInts(ctx.RequiredInput(2)).at(0);
  const int64_t max_distance = ctx.node().attr_i("max_distance", 128);
  const bool bidir = ctx.node().attr_i("is_bidirectional", 0) != 0;
  const int64_t num_buckets = table.size(0), heads = table.size(1);
  auto lopt = at::TensorOptions().dtype(at::kLong).device(table.device());
  at::Tensor rel = at::arange(klen, lopt).unsqueeze(0) - at::arange(qlen, lopt).unsqueeze(1);   // key - query
  at::Tensor bucket = at::zeros_like(rel);
  int64_t nb = num_buckets;
  at::Tensor n;
  if (bidir) {
    nb /= 2;
    bucket = bucket + (rel > 0).to(at::kLong) * nb;
    n = rel.abs();
  } else {
    n = (-rel).clamp_min(0);
  }
  const int64_t max_exact = nb / 2;
  at::Tensor large = max_exact + (at::log(n.to(at::kFloat) / static_cast<double>(max_exact)) /
                                  std::log(static_cast<double>(max_distance) / max_exact) * static_cast<double>(nb - max_exact))
                                     .to(at::kLong);
  large = large.clamp_max(nb - 1);
  bucket = bucket + at::where(n < max_exact, n, large);
  at::Tensor t2 = table.contiguous().reshape({heads, num_buckets});
  ctx.SetOutput(0, t2.index_select(1, bucket.reshape({-1})).reshape({1, heads, qlen, klen}));
}

// NGramRepeatBlock (contrib_ops/cuda/bert/ngram_repeat_block_impl.cu): ban the token that would complete an n-gram
// already present in input_ids.
void NGramRepeatBlockImpl(Ctx& ctx) {
  const int64_t n = ctx.node().attr_i("ngram_size", 0);
  ORTB_ENFORCE(n > 0, "NGramRepeatBlock: ngram_size must be positive");
  at::Tensor ids = ctx.RequiredInput(0).to(at::kCPU, at::kLong).contiguous();
  at::Tensor scores = ctx.RequiredInput(1).clone();
  const int64_t B = ids.size(0), L = ids.size(1), V = scores.size(1);
  const int64_t* p = ids.data_ptr<int64_t>();
  std::vector<int64_t> rows, cols;
  for (int64_t b = 0; b < B; ++b) {
    const int64_t* s = p + b * L;
    if (L + 1 < n) continue;
    for (int64_t i = 0; i + n <= L; ++i) {   // n-gram s[i .. i+n-1]; its prefix must equal the last n-1 tokens
      bool same = true;
      for (int64_t k = 0; k < n - 1 && same; ++k) same = s[i + k] == s[L - (n - 1) + k];
      if (same && s[i + n - 1] >= 0 && s[i + n - 1] < V) {
        rows.push_back(b);
        cols.push_back(s[i + n - 1]);
      }
    }
  }
  if (!rows.empty()) {
    at::Tensor r = at::tensor(rows, at::kLong).to(scores.device()), c = at::tensor(cols, at::kLong).to(scores.device());
    scores.index_put_({r, c}, -std::numeric_limits<float>::infinity());
  }
  ctx.SetOutput(0, scores);
}

// SkipGroupNorm (contrib_ops/cuda/diffusion/group_norm.cc): s = x + skip + bias; y = GroupNorm(s) (+ SiLU); also s.
void SkipGroupNormImpl(Ctx& ctx) {
  const Node& node = ctx.node();
  const at::Tensor& x = ctx.RequiredInput(0);
  const bool nhwc = node.attr_i("channels_last", 1) != 0;
  at::Tensor skip = ctx.RequiredInput(3);
  const int64_t C = nhwc ? x.size(3) : x.size(1);
  auto shape_like = [&](const at::Tensor& t) {   // (N, C) and (N, 1, 1, C) broadcast over the spatial dims
    if (t.dim() == 2) return nhwc ? t.reshape({t.size(0), 1, 1, C}) : t.reshape({t.size(0), C, 1, 1});
    return t;
  };
  at::Tensor s = x + shape_like(skip);
  if (ctx.HasInput(4)) s = s + (nhwc ? ctx.Input(4).reshape({1, 1, 1, C}) : ctx.Input(4).reshape({1, C, 1, 1}));
  at::Tensor nchw = nhwc ? s.permute({0, 3, 1, 2}) : s;
  at::Tensor y = at::group_norm(nchw.to(at::kFloat), node.attr_i("groups", 32), ctx.RequiredInput(1).to(at::kFloat),
                                ctx.RequiredInput(2).to(at::kFloat), node.attr_f("epsilon", 1e-5f), false);
  if (node.attr_i("activation", 0) == 1) y = y * at::sigmoid(y);
  if (nhwc) y = y.permute({0, 2, 3, 1}).contiguous();
  ctx.SetOutput(0, y.to(x.scalar_type()));
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, s);
}

// 4-bit bitsandbytes tables (contrib_ops/cpu/quantization/blockwise_quant_block_bnb4.h): code -> value in [-1, 1]
const float kFp4[16] = {0.f, 0.0052083333f, 0.66666667f, 1.f, 0.33333333f, 0.5f, 0.16666667f, 0.25f,
                        -0.f, -0.0052083333f, -0.66666667f, -1.f, -0.33333333f, -0.5f, -0.16666667f, -0.25f};
const float kNf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f, -0.28444138169288635f,
                        -0.18477343022823334f, -0.09105003625154495f, 0.0f, 0.07958029955625534f, 0.16093020141124725f,
                        0.24611230194568634f, 0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                        0.7229568362236023f, 1.0f};

// MatMulBnb4 (contrib_ops/cuda/quantization/matmul_bnb4.cc): B holds N*K codes, two per byte (first in the high
// nibble), blocks of block_size consecutive elements of the flattened [N, K] matrix share one absmax.
void MatMulBnb4Impl(Ctx& ctx) {
  const Node& node = ctx.node();
  const int64_t K = node.attr_i("K", 0), N = node.attr_i("N", 0), bs = node.attr_i("block_size", 64);
  const int64_t qt = node.attr_i("quant_type", 1);   // 0 = FP4, 1 = NF4
  const bool trans_b = node.attr_i("transB", 1) != 0;
  const at::Tensor& a = ctx.RequiredInput(0);
  at::Tensor packed = ctx.RequiredInput(1).reshape({-1});
  at::Tensor absmax = ctx.RequiredInput(2).reshape({-1}).to(at::kFloat);
  at::Tensor table = at::from_blob(const_cast<float*>(qt == 0 ? kFp4 : kNf4), {16}, at::kFloat).clone().to(a.device());
  at::Tensor codes = at::stack({packed.bitwise_right_shift(4), packed.bitwise_and(15)}, 1).reshape({-1}).narrow(0, 0, N * K);
  at::Tensor w = table.index_select(0, codes.to(at::kLong));
  const int64_t blocks = (N * K + bs - 1) / bs;
  at::Tensor scale = absmax.narrow(0, 0, blocks).repeat_interleave(bs).narrow(0, 0, N * K);
  w = (w * scale).reshape({N, K}).to(a.scalar_type());
  ctx.SetOutput(0, at::matmul(a, trans_b ? w.t() : w));
}

// MatMulBlockQuantizedFp8Weight (contrib_ops/cuda/math/matmul_block_scaled_fp8.cc): fp8 e4m3 weight [N, K], one fp32
// scale per block_size values along K; optional static fp8 quantise / dequantise of the activation.
at::Tensor DequantBlockFp8(const at::Tensor& b, const at::Tensor& scale, int64_t bs, at::ScalarType to) {
  const int64_t N = b.size(0), K = b.size(1);
  at::Tensor s = scale.to(at::kFloat).repeat_interleave(bs, 1).narrow(1, 0, K);
  return (b.to(at::kFloat) * s).to(to).reshape({N, K});
}

void MatMulBlockFp8Impl(Ctx& ctx) {
  const int64_t bs = ctx.node().attr_i("block_size", 128);
  at::Tensor a = ctx.RequiredInput(0);
  const at::Tensor& b = ctx.RequiredInput(1);
  ORTB_ENFORCE(b.scalar_type() == at::kFloat8_e4m3fn && b.dim() == 2, "MatMulBlockQuantizedFp8Weight: B must be fp8 e4m3 [N, K]");
  if (ctx.HasInput(3)) {
    at::Tensor sc = ctx.Input(3).to(at::kFloat).reshape({});
    a = ((a.to(at::kFloat) / sc).clamp(-448.f, 448.f).to(at::kFloat8_e4m3fn).to(at::kFloat) * sc).to(a.scalar_type());
  }
  at::Tensor w = DequantBlockFp8(b, ctx.RequiredInput(2), bs, a.scalar_type());
  at::Tensor y = at::matmul(a, w.t());
  if (ctx.HasInput(4)) y = y + ctx.Input(4);
  ctx.SetOutput(0, y);
}

// DynamicTimeWarping (contrib_ops/cpu/dynamic_time_warping.cc): lowest-cost monotone path through a cost matrix.
void DynamicTimeWarpingImpl(Ctx& ctx) {
  at::Tensor cost = ctx.RequiredInput(0).to(at::kCPU, at::kFloat).contiguous();
  if (cost.dim() == 3) cost = cost.squeeze(0);
  const int64_t M = cost.size(0), N = cost.size(1);
  const float* c = cost.data_ptr<float>();
  const float inf = std::numeric_limits<float>::infinity();
  std::vector<float> acc((M + 1) * (N + 1), inf);
  std::vector<int8_t> trace((M + 1) * (N + 1), -1);
  acc[0] = 0.f;
  for (int64_t i = 1; i <= M; ++i) {
    for (int64_t j = 1; j <= N; ++j) {
      const float diag = acc[(i - 1) * (N + 1) + j - 1], up = acc[(i - 1) * (N + 1) + j], left = acc[i * (N + 1) + j - 1];
      float best = diag;
      int8_t t = 0;
      if (up < best) { best = up; t = 1; }
      if (left < best) { best = left; t = 2; }
      acc[i * (N + 1) + j] = c[(i - 1) * N + j - 1] + best;
      trace[i * (N + 1) + j] = t;
    }
  }
  for (int64_t j = 0; j <= N; ++j) trace[j] = 2;
  for (int64_t i = 0; i <= M; ++i) trace[i * (N + 1)] = 1;
  std::vector<int32_t> rows, cols;
  int64_t i = M, j = N;
  while (i > 0 || j > 0) {
    rows.push_back(static_cast<int32_t>(i - 1));
    cols.push_back(static_cast<int32_t>(j - 1));
    const int8_t t = trace[i * (N + 1) + j];
    if (t == 0) { --i; --j; } else if (t == 1) { --i; } else { --j; }
    if (i == 0 && j == 0) break;
  }
  std::reverse(rows.begin(), rows.end());
  std::reverse(cols.begin(), cols.end());
  const int64_t L = static_cast<int64_t>(rows.size());
  at::Tensor out = at::empty({2, L}, at::kInt);
  std::copy(rows.begin(), rows.end(), out.data_ptr<int32_t>());
  std::copy(cols.begin(), cols.end(), out.data_ptr<int32_t>() + L);
  ctx.SetOutput(0, out.to(ctx.RequiredInput(0).device()));
}

at::Tensor AsComplex(const at::Tensor& t) { return at::view_as_complex(t.to(at::kFloat).contiguous()); }

// GatedRMSNorm: Y = X * rsqrt(mean(X^2 over groups of C) + eps) * scale * SiLU(gate), all in fp32.
void GatedRmsNormImpl(Ctx& ctx) {
  const at::Tensor& x = ctx.RequiredInput(0);
  const at::Tensor& scale = ctx.RequiredInput(1);
  const at::Tensor& gate = ctx.RequiredInput(2);
  const int64_t C = scale.numel();
  ORTB_ENFORCE(C > 0 && x.size(-1) % C == 0, "GatedRMSNorm: last dimension must be a multiple of the scale length");
  std::vector<int64_t> grouped(x.sizes().begin(), x.sizes().end());
  grouped.back() = x.size(-1) / C;
  grouped.push_back(C);
  at::Tensor xf = x.to(at::kFloat).reshape(grouped);
  at::Tensor gf = gate.to(at::kFloat).reshape(grouped);
  at::Tensor y = xf * at::rsqrt(xf.pow(2).mean(-1, true) + ctx.node().attr_f("epsilon", 1e-6f)) * scale.to(at::kFloat) * (gf * at::sigmoid(gf));
  ctx.SetOutput(0, y.reshape(x.sizes()).to(x.scalar_type()));
}

// PackedMultiHeadAttention / PackedAttention (contrib_ops/cuda/bert/packed_multihead_attention.cc, packed_attention.cc):
// attention over sequences stored back to back without padding; sequence b owns rows [cum[b], cum[b + 1]).
at::Tensor PackedSdpa(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const std::vector<int64_t>& cum, int64_t heads,
                      float scale, const at::Tensor* bias) {
  // q, k [T, N * H]; v [T, N * Hv]
  const int64_t T = q.size(0), H = q.size(1) / heads, Hv = v.size(1) / heads;
  at::Tensor out = at::empty({T, heads * Hv}, q.options());
  const float sc = scale != 0.f ? scale : 1.f / std::sqrt(static_cast<float>(H));
  for (size_t b = 0; b + 1 < cum.size(); ++b) {
    const int64_t lo = cum[b], len = cum[b + 1] - cum[b];
    if (len <= 0) continue;
    at::Tensor qb = q.narrow(0, lo, len).reshape({len, heads, H}).transpose(0, 1).to(at::kFloat);
    at::Tensor kb = k.narrow(0, lo, len).reshape({len, heads, H}).transpose(0, 1).to(at::kFloat);
    at::Tensor vb = v.narrow(0, lo, len).reshape({len, heads, Hv}).transpose(0, 1).to(at::kFloat);
    at::Tensor s = at::matmul(qb, kb.transpose(1, 2)) * sc;
    if (bias != nullptr) {
      at::Tensor bb = bias->size(0) == 1 ? bias->select(0, 0) : bias->select(0, static_cast<int64_t>(b));
      s = s + bb.narrow(-2, 0, len).narrow(-1, 0, len).to(at::kFloat);
    }
    at::Tensor o = at::matmul(at::softmax(s, -1), vb).transpose(0, 1).reshape({len, heads * Hv});
    out.narrow(0, lo, len).copy_(o.to(q.scalar_type()));
  }
  return out;
}

void PackedMhaImpl(Ctx& ctx) {
  const Node& node = ctx.node();
  const int64_t heads = node.attr_i("num_heads", 0);
  ORTB_ENFORCE(heads > 0, "PackedMultiHeadAttention: num_heads is required");
  at::Tensor q = ctx.RequiredInput(0), k, v;
  const std::vector<int64_t> cum = HostInts(ctx.RequiredInput(5));
  if (q.dim() == 4) {   // packed [T, N, 3, H]
    const int64_t T = q.size(0), H = q.size(3);
    at::Tensor qkv = q;
    if (ctx.HasInput(3)) qkv = qkv + ctx.Input(3).reshape({1, heads, 3, H});
    k = qkv.select(2, 1).reshape({T, heads * H});
    v = qkv.select(2, 2).reshape({T, heads * H});
    q = qkv.select(2, 0).reshape({T, heads * H});
  } else {
    k = ctx.RequiredInput(1);
    v = ctx.RequiredInput(2);
    if (ctx.HasInput(3)) {
      const at::Tensor& bias = ctx.Input(3);
      const int64_t dq = q.size(1), dk = k.size(1), dv = v.size(1);
      q = q + bias.narrow(0, 0, dq);
      k = k + bias.narrow(0, dq, dk);
      v = v + bias.narrow(0, dq + dk, dv);
    }
  }
  at::Tensor bias_t;
  const at::Tensor* bias = nullptr;
  if (ctx.HasInput(6)) {
    bias_t = ctx.Input(6);
    bias = &bias_t;
  }
  ctx.SetOutput(0, PackedSdpa(q, k, v, cum, heads, node.attr_f("scale", 0.f), bias));
}

void PackedAttentionImpl(Ctx& ctx) {
  // input [T, in], weights [in, 3 * hidden], bias [3 * hidden], token_offset, cumulative_sequence_length, attention_bias
  const Node& node = ctx.node();
  const int64_t heads = node.attr_i("num_heads", 0);
  ORTB_ENFORCE(heads > 0, "PackedAttention: num_heads is required");
  at::Tensor qkv = at::matmul(ctx.RequiredInput(0), ctx.RequiredInput(1)) + ctx.RequiredInput(2);
  std::vector<int64_t> sizes = node.attr_ints("qkv_hidden_sizes");
  if (sizes.size() != 3) sizes = {qkv.size(1) / 3, qkv.size(1) / 3, qkv.size(1) / 3};
  at::Tensor q = qkv.narrow(1, 0, sizes[0]), k = qkv.narrow(1, sizes[0], sizes[1]), v = qkv.narrow(1, sizes[0] + sizes[1], sizes[2]);
  at::Tensor bias_t;
  const at::Tensor* bias = nullptr;
  if (ctx.HasInput(5)) {
    bias_t = ctx.Input(5);
    bias = &bias_t;
  }
  ctx.SetOutput(0, PackedSdpa(q, k, v, HostInts(ctx.RequiredInput(4)), heads, node.attr_f("scale", 0.f), bias));
}

}  // namespace

void RegisterContribKernels2(KernelRegistry& r) {
  r.RegisterFn(MS, "RemovePadding", 1, kMax, RemovePaddingImpl, {1});
  r.RegisterFn(MS, "RestorePadding", 1, kMax, RestorePaddingImpl);
  r.RegisterFn(MS, "RelativePositionBias", 1, kMax, RelativePositionBiasImpl, {1, 2});
  r.RegisterFn(MS, "NGramRepeatBlock", 1, kMax, NGramRepeatBlockImpl, {0});
  r.RegisterFn(MS, "SkipGroupNorm", 1, kMax, SkipGroupNormImpl);
  r.RegisterFn(MS, "MatMulBnb4", 1, kMax, MatMulBnb4Impl);
  r.RegisterFn(MS, "MatMulBlockQuantizedFp8Weight", 1, kMax, MatMulBlockFp8Impl);
  r.RegisterFn(MS, "DynamicTimeWarping", 1, kMax, DynamicTimeWarpingImpl, {0});
  r.RegisterFn(MS, "GatedRMSNorm", 1, kMax, GatedRmsNormImpl);
  r.RegisterFn(MS, "PackedMultiHeadAttention", 1, kMax, PackedMhaImpl, {5});
  r.RegisterFn(MS, "PackedAttention", 1, kMax, PackedAttentionImpl, {4});
  r.RegisterFn(MS, "GatedAdd", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x + (ctx.RequiredInput(1) * ctx.RequiredInput(2)).to(x.scalar_type()));
  });
  r.RegisterFn(MS, "GemmaRotaryEmbedding", 1, kMax, [](Ctx& ctx) {
    // emb [B, S, D] fp32; q, q_rot, k, k_rot [B, N, S, D] (contrib_ops/cuda/bert/gemma_rotary_emb.cc)
    const at::Tensor& emb = ctx.RequiredInput(0);
    const at::Tensor& q = ctx.RequiredInput(1);
    at::Tensor sin = at::sin(emb).to(q.scalar_type()).unsqueeze(1), cos = at::cos(emb).to(q.scalar_type()).unsqueeze(1);
    ctx.SetOutput(0, q * cos + ctx.RequiredInput(2) * sin);
    ctx.SetOutput(1, ctx.RequiredInput(3) * cos + ctx.RequiredInput(4) * sin);
  });
  // BiasDropout / BitmaskDropout at inference (training_mode false or absent): no element is dropped
  r.RegisterFn(MS, "BiasDropout", 1, kMax, [](Ctx& ctx) {
    const bool training = ctx.HasInput(4) && ctx.Input(4).cpu().item<bool>();
    ORTB_ENFORCE(!training, "BiasDropout: training mode is not supported by this inference engine");
    at::Tensor y = ctx.RequiredInput(0) + ctx.RequiredInput(1);
    if (ctx.HasInput(2)) y = y + ctx.Input(2);
    ctx.SetOutput(0, y);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, at::ones(y.sizes(), y.options().dtype(at::kBool)));
  }, {4});
  r.RegisterFn(MS, "BitmaskDropout", 1, kMax, [](Ctx& ctx) {
    const bool training = ctx.HasInput(2) && ctx.Input(2).cpu().item<bool>();
    ORTB_ENFORCE(!training, "BitmaskDropout: training mode is not supported by this inference engine");
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, x);
    if (ctx.OutputCount() > 1) {   // every element kept: all bits set (the last word only up to the element count)
      const int64_t n = x.numel(), words = (n + 31) / 32;
      at::Tensor m = at::full({words}, static_cast<int64_t>(0xffffffffLL), x.options().dtype(at::kLong));
      if (n % 32 != 0) m[words - 1] = static_cast<int64_t>((1LL << (n % 32)) - 1);
      ctx.SetOutput(1, m.to(at::kUInt32));
    }
  }, {2});
  r.RegisterFn(MS, "UnfoldTensor", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    const at::Tensor& x = ctx.RequiredInput(0);
    int64_t dim = n.attr_i("dim", -1);
    if (dim < 0) dim += x.dim();
    ctx.SetOutput(0, x.unfold(dim, n.attr_i("size", 1), n.attr_i("step", 1)).contiguous());
  });
  r.RegisterFn(MS, "Rfft", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t nd = ctx.node().attr_i("signal_ndim", 1);
    std::vector<int64_t> dims;
    for (int64_t i = nd; i >= 1; --i) dims.push_back(x.dim() - i);
    at::Tensor y = at::fft_rfftn(x.to(at::kFloat), c10::nullopt, dims);
    ctx.SetOutput(0, at::view_as_real(y).to(x.scalar_type()));
  });
  r.RegisterFn(MS, "Irfft", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);   // [..., n / 2 + 1, 2]
    const int64_t nd = ctx.node().attr_i("signal_ndim", 1);
    at::Tensor c = AsComplex(x);
    std::vector<int64_t> dims;
    for (int64_t i = nd; i >= 1; --i) dims.push_back(c.dim() - i);
    std::vector<int64_t> sizes;
    for (int64_t d : dims) sizes.push_back(c.size(d));
    sizes.back() = (c.size(-1) - 1) * 2;
    ctx.SetOutput(0, at::fft_irfftn(c, sizes, dims).to(x.scalar_type()));
  });
  r.RegisterFn(MS, "ComplexMul", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& a = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::view_as_real(AsComplex(a) * AsComplex(ctx.RequiredInput(1))).to(a.scalar_type()));
  });
  r.RegisterFn(MS, "ComplexMulConj", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& a = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::view_as_real(AsComplex(a) * at::conj(AsComplex(ctx.RequiredInput(1)))).to(a.scalar_type()));
  });
  // legacy ONNX-domain experimental operators the reference still registers (contrib_ops/cpu/cpu_contrib_kernels.cc)
  r.RegisterFn("", "Affine", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, ctx.RequiredInput(0) * ctx.node().attr_f("alpha", 1.f) + ctx.node().attr_f("beta", 0.f));
  });
  r.RegisterFn("", "ParametricSoftplus", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ctx.SetOutput(0, at::softplus(x * ctx.node().attr_f("beta", 1.f)) * ctx.node().attr_f("alpha", 1.f));
  });
  r.RegisterFn("", "ScaledTanh", 1, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::tanh(ctx.RequiredInput(0) * ctx.node().attr_f("beta", 1.f)) * ctx.node().attr_f("alpha", 1.f));
  });
  r.RegisterFn("", "ImageScaler", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);   // NCHW
    at::Tensor y = x * ctx.node().attr_f("scale", 1.f);
    const std::vector<float> bias = ctx.node().attr_floats("bias");
    if (!bias.empty()) y = y + at::tensor(bias, at::kFloat).to(x.device(), x.scalar_type()).reshape({1, -1, 1, 1});
    ctx.SetOutput(0, y);
  });
  r.RegisterFn("", "Crop", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);   // NCHW; border = left, top, right, bottom
    const std::vector<int64_t> border = ctx.node().attr_ints("border");
    ORTB_ENFORCE(border.size() == 4, "Crop: border must have 4 values");
    const std::vector<int64_t> scale = ctx.node().attr_ints("scale");
    const int64_t H = x.size(2), W = x.size(3);
    const int64_t top = border[1], left = border[0];
    const int64_t h = scale.size() == 2 ? scale[0] : H - top - border[3];
    const int64_t w = scale.size() == 2 ? scale[1] : W - left - border[2];
    ctx.SetOutput(0, x.narrow(2, top, h).narrow(3, left, w).contiguous());
  });
  r.RegisterFn("", "DynamicSlice", 1, kMax, [](Ctx& ctx) {
    at::Tensor y = ctx.RequiredInput(0);
    const std::vector<int64_t> starts = HostInts(ctx.RequiredInput(1)), ends = HostInts(ctx.RequiredInput(2));
    std::vector<int64_t> axes;
    if (ctx.HasInput(3)) axes = HostInts(ctx.Input(3));
    else for (size_t i = 0; i < starts.size(); ++i) axes.push_back(static_cast<int64_t>(i));
    for (size_t i = 0; i < axes.size(); ++i) {
      const int64_t ax = axes[i] < 0 ? axes[i] + y.dim() : axes[i], n = y.size(ax);
      int64_t s = starts[i] < 0 ? starts[i] + n : starts[i], e = ends[i] < 0 ? ends[i] + n : ends[i];
      s = std::min(std::max<int64_t>(s, 0), n);
      e = std::min(std::max<int64_t>(e, s), n);
      y = y.narrow(ax, s, e - s);
    }
    ctx.SetOutput(0, y.contiguous());
  }, {1, 2, 3});
}

}  // namespace ortb
