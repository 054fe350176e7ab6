// com.microsoft contrib operators, fifth group: fused MatMulNBits projections (gated MLP, QKV with RMS norm),
// DecoderAttention (sequence-first self / cross attention with runtime switches) and BifurcationDetector.
#include <ATen/ATen.h>

#include <limits>

#include <algorithm>
#include <cctype>
#include <cmath>

#include "contrib_math.h"
#include "kernel.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;

at::Tensor OptT(Ctx& ctx, int i) { return ctx.HasInput(i) ? ctx.Input(i) : at::Tensor(); }

bool HostBool(const at::Tensor& t) { return t.to(at::kCPU).reshape({-1})[0].item<bool>(); }

// x [.., K] @ dequant(B [N, blocks, block * bits / 8], scales)^T + bias; symmetric zero point (2^(bits-1))
at::Tensor NBitsProject(const at::Tensor& x, const at::Tensor& B, const at::Tensor& scales, const at::Tensor& bias,
                        int64_t N, int64_t K, int64_t bits, int64_t block) {
  at::Tensor w = contrib::DequantizeNBits(B, scales, at::Tensor(), N, K, bits, block, at::kFloat);   // [N, K]
  at::Tensor y = at::matmul(x.to(at::kFloat), w.t());
  if (bias.defined()) y = y + bias.to(at::kFloat);
  return y;
}

// optional (Skip)SimplifiedLayerNormalization in front of the projections; returns the normalised activation and
// sets *sum to input + skip when a skip input is present
at::Tensor MaybeRmsNorm(const at::Tensor& a, const at::Tensor& skip, const at::Tensor& gamma, float eps, at::Tensor* sum) {
  at::Tensor x = a.to(at::kFloat);
  if (skip.defined()) {
    x = x + skip.to(at::kFloat);
    *sum = x;
  }
  if (!gamma.defined()) return x;
  at::Tensor rstd = at::rsqrt(x.pow(2).mean(-1, true) + static_cast<double>(eps));
  return x * rstd * gamma.to(at::kFloat);
}

at::Tensor GateActivation(const at::Tensor& x, std::string name) {
  std::transform(name.begin(), name.end(), name.begin(), [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
  if (name == "silu" || name == "swish") return at::silu(x);
  if (name == "gelu") return at::gelu(x);
  if (name == "gelu_tanh" || name == "fastgelu" || name == "fast_gelu") return at::gelu(x, "tanh");
  if (name == "relu") return at::relu(x);
  if (name == "sigmoid") return at::sigmoid(x);
  if (name == "identity" || name == "none") return x;
  ORTB_THROW(INVALID_ARGUMENT, "MatMulNBitsMlp: unknown activation '", name, "'");
}

// MatMulNBitsMlp: Y = act(A' gate_W^T + gate_b) * (A' up_W^T + up_b), A' = A or RMSNorm(A (+ skip))
void NBitsMlpImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& a = ctx.RequiredInput(0);
  const int64_t K = n.attr_i("K", 0), N = n.attr_i("N", 0), bits = n.attr_i("bits", 4), block = n.attr_i("block_size", 32);
  at::Tensor sum;
  at::Tensor x = MaybeRmsNorm(a, OptT(ctx, 1), OptT(ctx, 2), n.attr_f("epsilon", 1e-5f), &sum);
  at::Tensor gate = NBitsProject(x, ctx.RequiredInput(3), ctx.RequiredInput(4), OptT(ctx, 5), N, K, bits, block);
  at::Tensor up = NBitsProject(x, ctx.RequiredInput(6), ctx.RequiredInput(7), OptT(ctx, 8), N, K, bits, block);
  ctx.SetOutput(0, (GateActivation(gate, n.attr_s("activation", "silu")) * up).to(a.scalar_type()));
  if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) {
    ORTB_ENFORCE_ARG(sum.defined(), "MatMulNBitsMlp: the residual-sum output needs the skip input");
    ctx.SetOutput(1, sum.to(a.scalar_type()));
  }
}

// MatMulNBitsQkv: RMSNorm(A (+ skip)) projected three times
void NBitsQkvImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& a = ctx.RequiredInput(0);
  const int64_t K = n.attr_i("K", 0), Nq = n.attr_i("Nq", 0), Nkv = n.attr_i("Nkv", 0);
  const int64_t bits = n.attr_i("bits", 4), block = n.attr_i("block_size", 32);
  at::Tensor sum;
  at::Tensor x = MaybeRmsNorm(a, OptT(ctx, 1), ctx.RequiredInput(2), n.attr_f("epsilon", 1e-5f), &sum);
  ctx.SetOutput(0, NBitsProject(x, ctx.RequiredInput(3), ctx.RequiredInput(4), OptT(ctx, 5), Nq, K, bits, block).to(a.scalar_type()));
  ctx.SetOutput(1, NBitsProject(x, ctx.RequiredInput(6), ctx.RequiredInput(7), OptT(ctx, 8), Nkv, K, bits, block).to(a.scalar_type()));
  ctx.SetOutput(2, NBitsProject(x, ctx.RequiredInput(9), ctx.RequiredInput(10), OptT(ctx, 11), Nkv, K, bits, block).to(a.scalar_type()));
  if (ctx.OutputCount() > 3 && ctx.OutputNeeded(3)) {
    ORTB_ENFORCE_ARG(sum.defined(), "MatMulNBitsQkv: the residual-sum output needs the skip input");
    ctx.SetOutput(3, sum.to(a.scalar_type()));
  }
}

// DecoderAttention (contrib_ops/cuda/bert/decoder_attention.cc).  query [S, B, hidden], key [T, B, hidden].
//   first step (no layer state or use_past false): keys / values are projected from `query` (self attention) or
//     from `key` (static_kv: cross attention);
//   later steps: self attention appends the projection of `query` to the caches, cross attention reuses the caches.
void DecoderAttentionImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& query = ctx.RequiredInput(0);
  const at::Tensor& key = ctx.RequiredInput(1);
  const at::Tensor& qw = ctx.RequiredInput(2);
  const at::Tensor& kvw = ctx.RequiredInput(3);
  const at::Tensor& bias = ctx.RequiredInput(4);
  const bool static_kv = HostBool(ctx.RequiredInput(8)), use_past = HostBool(ctx.RequiredInput(9));
  const bool has_state = HostBool(ctx.RequiredInput(10)), has_mask = HostBool(ctx.RequiredInput(11));
  const int64_t S = query.size(0), B = query.size(1), hidden = query.size(2), N = n.attr_i("num_heads", 1), H = hidden / N;
  auto heads = [&](const at::Tensor& t) {  // [L, B, hidden] -> [B, N, L, H]
    return t.reshape({t.size(0), B, N, H}).permute({1, 2, 0, 3});
  };
  at::Tensor q = heads((at::matmul(query, qw) + bias.narrow(0, 0, hidden)).to(at::kFloat));
  auto project_kv = [&](const at::Tensor& src) {
    at::Tensor kv = (at::matmul(src, kvw) + bias.narrow(0, hidden, 2 * hidden)).to(at::kFloat);
    return std::make_pair(heads(kv.narrow(2, 0, hidden)), heads(kv.narrow(2, hidden, hidden)));
  };
  at::Tensor k, v;
  if (!has_state || !use_past) {
    std::tie(k, v) = project_kv(static_kv ? key : query);
  } else {
    ORTB_ENFORCE_ARG(ctx.HasInput(6) && ctx.HasInput(7), "DecoderAttention: use_past needs key_cache and value_cache");
    k = ctx.Input(6).to(at::kFloat);
    v = ctx.Input(7).to(at::kFloat);
    if (!static_kv) {
      auto kv = project_kv(query);
      k = at::cat({k, kv.first}, 2);
      v = at::cat({v, kv.second}, 2);
    }
  }
  const int64_t T = k.size(2);
  at::Tensor s = at::matmul(q, k.transpose(-1, -2)) / std::sqrt(static_cast<double>(H));
  if (has_mask && ctx.HasInput(5)) {
    at::Tensor masked = ctx.Input(5).to(s.device()).to(at::kBool).reshape({B, 1, 1, T});   // true = padding
    s = s.masked_fill(masked, n.attr_f("mask_filter_value", -10000.f));
  }
  at::Tensor y = at::matmul(at::softmax(s, -1), v);                                         // [B, N, S, H]
  ctx.SetOutput(0, y.permute({2, 0, 1, 3}).reshape({S, B, hidden}).to(query.scalar_type()).contiguous());
  if (ctx.OutputCount() > 1) ctx.SetOutput(1, k.to(query.scalar_type()).contiguous());
  if (ctx.OutputCount() > 2) ctx.SetOutput(2, v.to(query.scalar_type()).contiguous());
}

// BifurcationDetector (contrib_ops/cpu/bert/bifurcation_detector.h), used by aggressive decoding.
//  1. tokens = cur_tokens ++ pred_tokens[0 .. d], d = first index where pred_tokens leaves src_tokens[prev_idx + .]
//  2. for n = min_ngram .. max_ngram: look the last n tokens up in src_tokens; none -> stop with the previous answer;
//     exactly one occurrence -> answer = position just behind it (stop if that is the end of src_tokens); more than
//     one -> answer = -1; then try the next n.
void BifurcationDetectorImpl(Ctx& ctx) {
  auto host = [](const at::Tensor& t) {
    at::Tensor c = t.to(at::kCPU, at::kLong).contiguous();
    ORTB_ENFORCE_ARG(c.dim() == 1, "BifurcationDetector: token inputs must be 1-D");
    return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
  };
  const std::vector<int64_t> src = host(ctx.RequiredInput(0)), cur = host(ctx.RequiredInput(1));
  const at::Tensor& prev_t = ctx.RequiredInput(2);
  ORTB_ENFORCE_ARG(prev_t.numel() == 1, "BifurcationDetector: prev_suffix_match_idx must hold one value");
  const int64_t prev = prev_t.to(at::kCPU, at::kLong).reshape({-1})[0].item<int64_t>();
  std::vector<int64_t> tokens = cur;
  if (ctx.HasInput(3)) {
    const std::vector<int64_t> pred = host(ctx.Input(3));
    const int64_t n_src = static_cast<int64_t>(src.size());
    ORTB_ENFORCE_ARG(prev >= 0 && prev <= n_src, "BifurcationDetector: prev_suffix_match_idx out of range");
    ORTB_ENFORCE_ARG(static_cast<int64_t>(pred.size()) == n_src + 1 - prev, "BifurcationDetector: pred_tokens must hold ",
                     n_src + 1 - prev, " tokens");
    int64_t d = 0;
    while (d < n_src - prev && pred[d] == src[d + prev]) ++d;
    tokens.insert(tokens.end(), pred.begin(), pred.begin() + d + 1);
  }
  const int64_t min_n = ctx.node().attr_i("min_ngram_size", 1), max_n = ctx.node().attr_i("max_ngram_size", 3);
  int64_t answer = -1;
  for (int64_t g = min_n; g <= max_n && g <= static_cast<int64_t>(tokens.size()); ++g) {
    auto gram_begin = tokens.end() - g;
    auto first = std::search(src.begin(), src.end(), gram_begin, tokens.end());
    if (first == src.end()) break;
    answer = (first - src.begin()) + g;
    if (answer >= static_cast<int64_t>(src.size())) break;
    if (std::search(first + 1, src.end(), gram_begin, tokens.end()) != src.end()) answer = -1;
  }
  auto lopt = at::TensorOptions().dtype(at::kLong);
  ctx.SetOutput(0, at::tensor(tokens, lopt).to(ctx.RequiredInput(1).device()));
  ctx.SetOutput(1, at::full(prev_t.sizes(), answer, lopt).to(prev_t.device()));
}

}  // namespace

// WordConvEmbedding (contrib_ops/cpu/word_conv_embedding.cc): every word (a row of character ids, 0 or out-of-range ids
// = padding) -> character embeddings (padding contributes zero vectors) -> convolution over the characters with window
// W.shape[2] and stride 1 -> tanh -> maximum over the max(length - window + 1, 1) positions that lie inside the word.
void WordConvEmbeddingImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& seq = ctx.RequiredInput(0);
  const at::Tensor& W = ctx.RequiredInput(1);
  const at::Tensor& B = ctx.RequiredInput(2);
  const at::Tensor& C = ctx.RequiredInput(3);
  ORTB_ENFORCE_ARG(seq.dim() > 1, "WordConvEmbedding: Sequence input must have rank greater than 1");
  ORTB_ENFORCE_ARG(W.dim() == 4 && W.size(1) == 1 && C.dim() == 2, "WordConvEmbedding: W must be [filters, 1, window, char_embedding], C [chars, char_embedding]");
  const int64_t F = W.size(0), window = W.size(2), E = W.size(3), WL = seq.size(-1);
  ORTB_ENFORCE_ARG(C.size(1) == E, "WordConvEmbedding: char embedding size of C (", C.size(1), ") and of W (", E, ") differ");
  ORTB_ENFORCE_ARG(B.numel() >= F, "WordConvEmbedding: bias has fewer entries than W has filters");
  ORTB_ENFORCE_ARG(window <= WL, "WordConvEmbedding: Conv kernel width must not exceed word length");
  ORTB_ENFORCE_ARG(!n.has_attr("embedding_size") || n.attr_i("embedding_size", F) == F, "WordConvEmbedding: embedding_size does not match W");
  ORTB_ENFORCE_ARG(!n.has_attr("conv_window_size") || n.attr_i("conv_window_size", window) == window, "WordConvEmbedding: conv_window_size does not match W");
  ORTB_ENFORCE_ARG(!n.has_attr("char_embedding_size") || n.attr_i("char_embedding_size", E) == E, "WordConvEmbedding: char_embedding_size does not match C");
  at::Tensor ids = seq.reshape({-1, WL}).to(at::kLong);
  at::Tensor valid = ids.gt(0).logical_and(ids.lt(C.size(0)));
  at::Tensor emb = C.index_select(0, at::where(valid, ids, at::zeros_like(ids)).reshape({-1})).reshape({ids.size(0), WL, E}) * valid.unsqueeze(-1).to(C.scalar_type());
  at::Tensor windows = emb.unfold(1, window, 1).permute({0, 1, 3, 2}).reshape({ids.size(0), WL - window + 1, window * E});  // [words, positions, window * E]
  at::Tensor y = at::tanh(at::matmul(windows, W.reshape({F, window * E}).t()) + B.narrow(0, 0, F));                        // [words, positions, F]
  at::Tensor positions = at::clamp_min(valid.sum(1) - window + 1, 1);                                                         // inside the word
  at::Tensor outside = at::arange(WL - window + 1, ids.options()).unsqueeze(0).ge(positions.unsqueeze(1));
  y = y.masked_fill(outside.unsqueeze(-1), -std::numeric_limits<float>::infinity()).amax(1);
  std::vector<int64_t> shape = seq.sizes().vec();
  shape.back() = F;
  ctx.SetOutput(0, y.reshape(shape));
}

void RegisterContribKernels5(KernelRegistry& r) {
  r.RegisterFn(MS, "WordConvEmbedding", 1, kMax, WordConvEmbeddingImpl);
  r.RegisterFn(MS, "MatMulNBitsMlp", 1, kMax, NBitsMlpImpl);
  r.RegisterFn(MS, "MatMulNBitsQkv", 1, kMax, NBitsQkvImpl);
  r.RegisterFn(MS, "DecoderAttention", 1, kMax, DecoderAttentionImpl, {8, 9, 10, 11});
  r.RegisterFn(MS, "BifurcationDetector", 1, kMax, BifurcationDetectorImpl, {0, 1, 2, 3});
}

}  // namespace ortb
