// ONNX operators: TfIdfVectorizer (integer tokens), STFT, MelWeightMatrix, MaxRoiPool, Optional / OptionalGetElement /
// OptionalHasElement (tensor payloads); contrib GatherBlockQuantized (uint8 data, 2 / 4 / 8 bits).
// Reference kernels: onnxruntime/core/providers/cpu/nlp/tfidfvectorizer.cc, cpu/signal/dft.cc (STFT), cpu/signal/
// mel_weight_matrix.cc, cpu/object_detection/roialign.cc's neighbour cpu/nn/roi_pool.cc, cpu/optional/optional_ops.cc,
// contrib_ops/cpu/quantization/gather_block_quantized.cc.
#include <ATen/ATen.h>

#include <algorithm>
#include <cmath>
#include <map>

#include "kernel.h"
#include "string_table.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;

// ------------------------------------------------------------------------------------------------ TfIdfVectorizer
void TfIdfImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = x_in.to(at::kCPU, at::kLong).contiguous();
  ORTB_ENFORCE_ARG(x.dim() == 1 || x.dim() == 2, "TfIdfVectorizer: input must have rank 1 or 2");
  const int64_t rows = x.dim() == 2 ? x.size(0) : 1, C = x.dim() == 2 ? x.size(1) : x.size(0);
  const int64_t min_n = n.attr_i("min_gram_length", 1), max_n = n.attr_i("max_gram_length", 1), max_skip = n.attr_i("max_skip_count", 0);
  const std::string mode = n.attr_s("mode", "TF");
  const std::vector<int64_t> starts = n.attr_ints("ngram_counts"), out_index = n.attr_ints("ngram_indexes");
  std::vector<int64_t> pool = n.attr_ints("pool_int64s");
  if (ctx.InputIsString(0)) {  // string tokens are ids of the string table: the pool becomes ids as well
    pool.clear();
    for (auto& s : n.attr_strings("pool_strings")) pool.push_back(InternString(s));
  }
  const std::vector<float> weights = n.attr_floats("weights");
  ORTB_ENFORCE_ARG(min_n >= 1 && max_n >= min_n, "TfIdfVectorizer: bad gram lengths");
  // pool n-grams of each length -> id (position among all n-grams, the index into ngram_indexes / weights)
  std::vector<std::map<std::vector<int64_t>, int64_t>> by_len(static_cast<size_t>(max_n) + 1);
  int64_t id = 0;
  for (size_t len = 1; len <= starts.size(); ++len) {
    const int64_t begin = starts[len - 1], end = len < starts.size() ? starts[len] : static_cast<int64_t>(pool.size());
    ORTB_ENFORCE_ARG(begin <= end && end <= static_cast<int64_t>(pool.size()) && (end - begin) % static_cast<int64_t>(len) == 0,
                     "TfIdfVectorizer: ngram_counts do not match the pool");
    for (int64_t p = begin; p < end; p += static_cast<int64_t>(len), ++id)
      if (static_cast<int64_t>(len) <= max_n) by_len[len][std::vector<int64_t>(pool.begin() + p, pool.begin() + p + static_cast<int64_t>(len))] = id;
  }
  ORTB_ENFORCE_ARG(static_cast<int64_t>(out_index.size()) == id, "TfIdfVectorizer: ngram_indexes must have one entry per pool n-gram");
  int64_t width = 0;
  for (int64_t v : out_index) width = std::max(width, v + 1);
  at::Tensor y = at::zeros({rows, width}, at::kFloat);
  const int64_t* tok = x.data_ptr<int64_t>();
  std::vector<int64_t> gram;
  for (int64_t r = 0; r < rows; ++r) {
    float* out = y.data_ptr<float>() + r * width;
    for (int64_t len = min_n; len <= max_n; ++len) {
      const auto& table = by_len[static_cast<size_t>(len)];
      if (table.empty()) continue;
      const int64_t skips = len == 1 ? 0 : max_skip;
      for (int64_t skip = 0; skip <= skips; ++skip) {
        const int64_t stride = skip + 1, span = (len - 1) * stride;
        for (int64_t s = 0; s + span < C; ++s) {
          gram.clear();
          for (int64_t k = 0; k < len; ++k) gram.push_back(tok[r * C + s + k * stride]);
          auto it = table.find(gram);
          if (it != table.end()) out[out_index[static_cast<size_t>(it->second)]] += 1.f;
        }
      }
    }
    if (mode != "TF") {
      std::vector<float> w(static_cast<size_t>(width), 1.f);
      for (size_t i = 0; i < out_index.size() && i < weights.size(); ++i) w[static_cast<size_t>(out_index[i])] = weights[i];
      for (int64_t c = 0; c < width; ++c) out[c] = mode == "IDF" ? (out[c] > 0 ? w[static_cast<size_t>(c)] : 0.f) : out[c] * w[static_cast<size_t>(c)];
    }
  }
  ctx.SetOutput(0, (x.dim() == 1 ? y.reshape({width}) : y).to(x_in.device()));
}

// ------------------------------------------------------------------------------------------------ STFT / mel
int64_t ScalarInt(const at::Tensor& t) { return t.to(at::kCPU, at::kLong).reshape({-1})[0].item<int64_t>(); }
double ScalarDouble(const at::Tensor& t) { return t.to(at::kCPU, at::kDouble).reshape({-1})[0].item<double>(); }

void StftImpl(Ctx& ctx) {
  at::Tensor signal = ctx.RequiredInput(0);  // [B, L, 1] real or [B, L, 2] complex
  ORTB_ENFORCE_ARG(signal.dim() == 3 && (signal.size(2) == 1 || signal.size(2) == 2), "STFT: signal must be [batch, length, 1 or 2]");
  const int64_t step = ScalarInt(ctx.RequiredInput(1));
  const bool has_window = ctx.HasInput(2);
  int64_t frame_len = ctx.HasInput(3) ? ScalarInt(ctx.Input(3)) : (has_window ? ctx.Input(2).numel() : 0);
  ORTB_ENFORCE_ARG(frame_len > 0 && step > 0 && frame_len <= signal.size(1), "STFT: needs a window or a frame_length no longer than the signal");
  const bool complex_in = signal.size(2) == 2;
  const bool onesided = ctx.node().attr_i("onesided", 1) != 0 && !complex_in;
  at::Tensor s = complex_in ? at::view_as_complex(signal.to(at::kFloat).contiguous()) : signal.squeeze(2).to(at::kFloat);
  at::Tensor frames = s.unfold(1, frame_len, step);  // [B, frames, frame_len]
  if (has_window) {
    at::Tensor w = ctx.Input(2).to(signal.device(), at::kFloat);
    if (w.numel() < frame_len) w = at::constant_pad_nd(w, {0, frame_len - w.numel()});
    frames = frames * w;
  }
  at::Tensor spec = onesided ? at::fft_rfft(frames, c10::nullopt, -1) : at::fft_fft(frames, c10::nullopt, -1);
  ctx.SetOutput(0, at::view_as_real(spec).to(signal.scalar_type()));
}

void MelWeightMatrixImpl(Ctx& ctx) {
  const int64_t mels = ScalarInt(ctx.RequiredInput(0)), dft = ScalarInt(ctx.RequiredInput(1)), rate = ScalarInt(ctx.RequiredInput(2));
  const double lo = ScalarDouble(ctx.RequiredInput(3)), hi = ScalarDouble(ctx.RequiredInput(4));
  ORTB_ENFORCE_ARG(mels > 0 && dft > 0 && rate > 0, "MelWeightMatrix: sizes must be positive");
  const int64_t bins = dft / 2 + 1;
  auto to_mel = [](double hz) { return 2595.0 * std::log10(1.0 + hz / 700.0); };
  const double mel_lo = to_mel(lo), mel_step = (to_mel(hi) - mel_lo) / static_cast<double>(mels + 2);
  std::vector<int64_t> edge(static_cast<size_t>(mels) + 2);
  for (int64_t i = 0; i < mels + 2; ++i) {
    const double hz = 700.0 * (std::pow(10.0, (static_cast<double>(i) * mel_step + mel_lo) / 2595.0) - 1.0);
    edge[static_cast<size_t>(i)] = static_cast<int64_t>(std::floor(static_cast<double>(dft + 1) * hz / static_cast<double>(rate)));
  }
  at::Tensor out = at::zeros({bins, mels}, at::kDouble);
  auto o = out.accessor<double, 2>();
  auto put = [&](int64_t row, int64_t col, double v) {
    if (row >= 0 && row < bins) o[row][col] = v;
  };
  for (int64_t i = 0; i < mels; ++i) {
    const int64_t left = edge[static_cast<size_t>(i)], centre = edge[static_cast<size_t>(i) + 1], right = edge[static_cast<size_t>(i) + 2];
    if (centre == left) {
      put(centre, i, 1.0);
    } else {
      for (int64_t j = left; j <= centre; ++j) put(j, i, static_cast<double>(j - left) / static_cast<double>(centre - left));
    }
    for (int64_t j = centre; j < right; ++j) put(j, i, static_cast<double>(right - j) / static_cast<double>(right - centre));
  }
  static const std::map<int64_t, at::ScalarType> onnx_type = {{1, at::kFloat}, {10, at::kHalf}, {11, at::kDouble}, {16, at::kBFloat16},
                                                              {6, at::kInt}, {7, at::kLong}, {2, at::kByte}, {3, at::kChar}};
  auto t = onnx_type.find(ctx.node().attr_i("output_datatype", 1));
  ORTB_ENFORCE_ARG(t != onnx_type.end(), "MelWeightMatrix: unsupported output_datatype");
  ctx.SetOutput(0, out.to(t->second).to(ctx.device()));
}

// ------------------------------------------------------------------------------------------------ MaxRoiPool
void MaxRoiPoolImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& x_in = ctx.RequiredInput(0);
  at::Tensor x = x_in.to(at::kCPU, at::kFloat).contiguous();
  at::Tensor rois = ctx.RequiredInput(1).to(at::kCPU, at::kFloat).contiguous();
  const std::vector<int64_t> shape = n.attr_ints("pooled_shape");
  ORTB_ENFORCE_ARG(shape.size() == 2 && x.dim() == 4 && rois.dim() == 2 && rois.size(1) == 5, "MaxRoiPool: needs pooled_shape [h, w], X [N, C, H, W], rois [R, 5]");
  const float scale = n.attr_f("spatial_scale", 1.f);
  const int64_t PH = shape[0], PW = shape[1], C = x.size(1), H = x.size(2), W = x.size(3), R = rois.size(0);
  at::Tensor y = at::zeros({R, C, PH, PW}, at::kFloat);
  for (int64_t r = 0; r < R; ++r) {
    const float* roi = rois.data_ptr<float>() + r * 5;
    const int64_t b = static_cast<int64_t>(roi[0]);
    ORTB_ENFORCE_ARG(b >= 0 && b < x.size(0), "MaxRoiPool: roi batch index out of range");
    const int64_t x1 = std::llround(roi[1] * scale), y1 = std::llround(roi[2] * scale), x2 = std::llround(roi[3] * scale), y2 = std::llround(roi[4] * scale);
    const double bin_h = static_cast<double>(std::max<int64_t>(y2 - y1 + 1, 1)) / static_cast<double>(PH);
    const double bin_w = static_cast<double>(std::max<int64_t>(x2 - x1 + 1, 1)) / static_cast<double>(PW);
    for (int64_t c = 0; c < C; ++c) {
      const float* plane = x.data_ptr<float>() + (b * C + c) * H * W;
      for (int64_t ph = 0; ph < PH; ++ph) {
        const int64_t h0 = std::clamp<int64_t>(static_cast<int64_t>(std::floor(ph * bin_h)) + y1, 0, H);
        const int64_t h1 = std::clamp<int64_t>(static_cast<int64_t>(std::ceil((ph + 1) * bin_h)) + y1, 0, H);
        for (int64_t pw = 0; pw < PW; ++pw) {
          const int64_t w0 = std::clamp<int64_t>(static_cast<int64_t>(std::floor(pw * bin_w)) + x1, 0, W);
          const int64_t w1 = std::clamp<int64_t>(static_cast<int64_t>(std::ceil((pw + 1) * bin_w)) + x1, 0, W);
          if (h1 <= h0 || w1 <= w0) continue;  // empty bin stays 0
          float best = -std::numeric_limits<float>::infinity();
          for (int64_t h = h0; h < h1; ++h)
            for (int64_t w = w0; w < w1; ++w) best = std::max(best, plane[h * W + w]);
          y.data_ptr<float>()[((r * C + c) * PH + ph) * PW + pw] = best;
        }
      }
    }
  }
  ctx.SetOutput(0, y.to(x_in.device(), x_in.scalar_type()));
}

// ------------------------------------------------------------------------------------------------ GatherBlockQuantized
// uint8 storage holding `bits`-wide values, low-order bits first, along the last axis -> one value per element
at::Tensor UnpackBits(const at::Tensor& packed, int64_t bits) {
  if (bits == 8) return packed.to(at::kInt);
  const int64_t per = 8 / bits, mask = (1 << bits) - 1;
  std::vector<at::Tensor> parts;
  at::Tensor p = packed.to(at::kInt);
  for (int64_t k = 0; k < per; ++k) parts.push_back(at::bitwise_and(at::bitwise_right_shift(p, k * bits), mask));
  std::vector<int64_t> shape = packed.sizes().vec();
  shape.back() *= per;
  return at::stack(parts, -1).reshape(shape);
}

void GatherBlockQuantizedImpl(Ctx& ctx) {
  const Node& n = ctx.node();
  const at::Tensor& data = ctx.RequiredInput(0);
  const at::Tensor& scales = ctx.RequiredInput(2);
  ORTB_ENFORCE(data.scalar_type() == at::kByte, "GatherBlockQuantized: data must be uint8 (packed 2 / 4 bit or plain 8 bit)");
  const int64_t bits = n.attr_i("bits", 4), block = n.attr_i("block_size", 128), rank = data.dim();
  ORTB_ENFORCE_ARG(bits == 2 || bits == 4 || bits == 8, "GatherBlockQuantized: bits must be 2, 4 or 8");
  ORTB_ENFORCE_ARG(block >= 16 && (block & (block - 1)) == 0, "GatherBlockQuantized: block_size must be a power of two, at least 16");
  int64_t ga = n.attr_i("gather_axis", 0), qa = n.attr_i("quantize_axis", 1);
  if (ga < 0) ga += rank;
  if (qa < 0) qa += rank;
  ORTB_ENFORCE_ARG(ga == 0, "GatherBlockQuantized: uint8 data gathers along axis 0 only");
  ORTB_ENFORCE_ARG(qa == rank - 1 && rank >= 2, "GatherBlockQuantized: uint8 data is quantized along the last axis");
  const at::Tensor& indices = ctx.RequiredInput(1);
  at::Tensor idx = indices.to(data.device(), at::kLong).reshape({-1});
  idx = at::where(idx < 0, idx + data.size(0), idx);
  ORTB_ENFORCE_ARG(idx.numel() == 0 || (idx.min().item<int64_t>() >= 0 && idx.max().item<int64_t>() < data.size(0)), "GatherBlockQuantized: index out of range");
  at::Tensor q = UnpackBits(data.index_select(0, idx), bits);  // [n_idx, ..., K]
  const int64_t K = q.size(-1);
  at::Tensor s = scales.index_select(0, idx).repeat_interleave(block, -1).narrow(-1, 0, K);
  at::Tensor zp;
  if (ctx.HasInput(3)) {
    zp = UnpackBits(ctx.Input(3).index_select(0, idx), bits);
    zp = zp.narrow(-1, 0, scales.size(-1)).repeat_interleave(block, -1).narrow(-1, 0, K);
  } else {
    zp = at::full({}, static_cast<int64_t>(1) << (bits - 1), q.options());
  }
  at::Tensor y = ((q - zp).to(at::kFloat) * s.to(at::kFloat)).to(scales.scalar_type());
  std::vector<int64_t> shape = indices.sizes().vec();
  for (int64_t d = 1; d < rank; ++d) shape.push_back(q.size(d));
  ctx.SetOutput(0, y.reshape(shape));
}

}  // namespace

void RegisterOnnxExtraKernels3(KernelRegistry& r) {
  r.RegisterFn("", "TfIdfVectorizer", 9, kMax, TfIdfImpl);
  r.RegisterFn("", "STFT", 17, kMax, StftImpl, {1, 3});
  r.RegisterFn("", "MelWeightMatrix", 17, kMax, MelWeightMatrixImpl, {0, 1, 2, 3, 4});
  r.RegisterFn("", "MaxRoiPool", 1, kMax, MaxRoiPoolImpl);
  r.RegisterFn("com.microsoft", "GatherBlockQuantized", 1, kMax, GatherBlockQuantizedImpl);
  // com.microsoft Unique (contrib_ops/cpu/unique.cc): 1-D input -> distinct values in order of first appearance, for
  // every input element the position of its value among them, and the count of every distinct value
  r.RegisterFn("com.microsoft", "Unique", 1, kMax, [](Ctx& ctx) {
    const at::Tensor& x = ctx.RequiredInput(0);
    ORTB_ENFORCE_ARG(x.dim() == 1, "Unique: input must be 1-D");
    auto res = at::_unique2(x, /*sorted=*/true, /*return_inverse=*/true, /*return_counts=*/true);
    at::Tensor values = std::get<0>(res), inverse = std::get<1>(res), counts = std::get<2>(res);
    // re-order from sorted to first-appearance order
    at::Tensor first = at::full({values.numel()}, x.numel(), inverse.options());
    first.scatter_reduce_(0, inverse, at::arange(x.numel(), inverse.options()), "amin");
    at::Tensor order = at::argsort(first);             // sorted position -> appearance rank
    at::Tensor rank = at::empty_like(order);
    rank.scatter_(0, order, at::arange(order.numel(), order.options()));
    ctx.SetOutput(0, values.index_select(0, order));
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, rank.index_select(0, inverse));
    if (ctx.OutputCount() > 2) ctx.SetOutput(2, counts.index_select(0, order));
  });
  // SparseToDenseMatMul (contrib_ops/cpu/math/sparse_dense_matmul.cc): sparse tensors are expanded when they enter a
  // session, so this is alpha * op(A) @ op(B) on dense operands
  r.RegisterFn("com.microsoft", "SparseToDenseMatMul", 1, kMax, [](Ctx& ctx) {
    const Node& n = ctx.node();
    at::Tensor a = ctx.RequiredInput(0), b = ctx.RequiredInput(1);
    if (n.attr_i("transA", 0)) a = a.transpose(-1, -2);
    if (n.attr_i("transB", 0)) b = b.transpose(-1, -2);
    ctx.SetOutput(0, at::matmul(a, b) * n.attr_f("alpha", 1.f));
  });
  // optional values carry tensors here: an absent input is the empty optional
  r.RegisterFn("", "Optional", 15, kMax, [](Ctx& ctx) {
    if (ctx.HasInput(0)) ctx.SetOutput(0, ctx.Input(0));
  });
  r.RegisterFn("", "OptionalGetElement", 15, kMax, [](Ctx& ctx) { ctx.SetOutput(0, ctx.RequiredInput(0)); });
  r.RegisterFn("", "OptionalHasElement", 15, kMax, [](Ctx& ctx) {
    ctx.SetOutput(0, at::full({}, ctx.HasInput(0) ? 1 : 0, at::TensorOptions().dtype(at::kBool).device(ctx.device())));
  });
}

}  // namespace ortb
