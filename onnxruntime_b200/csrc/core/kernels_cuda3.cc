// GPU op wrappers, part 3: MatMulNBits, PagedAttention, BERT Attention / MultiHeadAttention.
//
// Reference counterparts: onnxruntime/contrib_ops/cuda/quantization/matmul_nbits.cc,
// contrib_ops/cuda/bert/paged_attention.cc, bert/attention.cc and bert/multihead_attention.cc.
#include <ATen/ATen.h>

#include <mutex>
#include <ATen/cuda/CUDAContext.h>

#include <algorithm>
#include <cmath>

#include "collective.h"
#include "contrib_math.h"
#include "cuda_ops.h"
#include "ortb200_kernels.h"
#include "session.h"

namespace ortb {
namespace {

using Ctx = OpKernelContext;
constexpr const char* MS = kMSDomain;

int DtypeCode(at::ScalarType t) {
  if (t == at::kHalf) return ORTB200_F16;
  if (t == at::kBFloat16) return ORTB200_BF16;
  return -1;
}
bool HalfType(at::ScalarType t) { return t == at::kHalf || t == at::kBFloat16; }

class WithFallback : public OpKernel {
 public:
  explicit WithFallback(const OpKernelInfo& info) : OpKernel(info) {
    const KernelDef* d = KernelRegistry::Generic().Find(info.node, info.graph);
    if (d) fallback_ = d->factory(info);
  }

 protected:
  void Fallback(Ctx& ctx) const {
    if (!fallback_) ORTB_THROW(NOT_IMPLEMENTED, "no fallback kernel for ", node_.op_type);
    fallback_->Compute(ctx);
  }
  std::unique_ptr<OpKernel> fallback_;
};

// ---------------------------------------------------------------------------------------------------------------
// MatMulNBits: the packed weights stay packed in device memory; each call expands them to [N, K] rows with the
// dequantisation kernel and runs the tcgen05 GEMM on the result (bias in the GEMM epilogue).
class MatMulNBitsKernel final : public WithFallback {
 public:
  explicit MatMulNBitsKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    K_ = n.attr_i("K", 0);
    N_ = n.attr_i("N", 0);
    bits_ = n.attr_i("bits", 4);
    block_ = n.attr_i("block_size", 32);
    all_reduce_ = n.attr_i("all_reduce", 0) != 0;
    // decode path: re-arrange the nibbles once for the in-kernel expansion (4-bit, block >= 32, K % 64 == 0,
    // constant weights, integer zero points)
    const at::Tensor* B = info.constant_input(1);
    const at::Tensor* sc = info.constant_input(2);
    const bool has_zp = n.inputs.size() > 3 && !n.inputs[3].empty();
    const at::Tensor* zp = has_zp ? info.constant_input(3) : nullptr;
    if (B && sc && B->is_cuda() && bits_ == 4 && block_ >= 32 && (block_ & (block_ - 1)) == 0 && K_ % 64 == 0 &&
        HalfType(sc->scalar_type()) && (!has_zp || (zp && zp->scalar_type() == at::kByte)) &&
        !(n.inputs.size() > 4 && !n.inputs[4].empty())) {
      at::Tensor zp_bytes;
      if (zp) {
        // packed nibbles [N, ceil(nb / 2)] -> one byte per block
        const int64_t nb = (K_ + block_ - 1) / block_;
        at::Tensor z = zp->reshape({N_, -1}).to(at::kInt);
        zp_bytes = at::stack({at::bitwise_and(z, 0xF), at::bitwise_and(at::bitwise_right_shift(z, 4), 0xF)}, -1)
                       .reshape({N_, -1}).narrow(1, 0, nb).to(at::kByte).contiguous();
      }
      packed_ = NbitsBuildBlobs(*B, *sc, zp_bytes, N_, K_, block_);
      scales_ = *sc;
    }
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& a = ctx.RequiredInput(0);
    const bool reduce = all_reduce_ && ctx.session()->world_size > 1;
    std::vector<int64_t> out_shape = a.sizes().vec();
    out_shape.back() = N_;
    at::Tensor res = ctx.HasInput(6) ? ctx.Input(6) : at::Tensor();
    if (res.defined() && (res.sizes().vec() != out_shape || res.scalar_type() != a.scalar_type())) {
      Fallback(ctx);  // a residual that needs broadcasting: the generic path adds it
      return;
    }
    if (packed_.defined() && a.scalar_type() == scales_.scalar_type() && a.numel() / K_ <= 64) {
      at::Tensor x2 = a.reshape({-1, K_}).contiguous();
      at::Tensor bias = ctx.HasInput(5) ? ctx.Input(5) : at::Tensor();
      at::Tensor res2 = res.defined() ? res.reshape({-1, N_}).contiguous() : at::Tensor();
      at::Tensor y;
      if (reduce && CanFuseAllReduce(ctx, x2.size(0), N_)) {
        y = LaunchGemmQ4(ctx, x2, packed_, N_, bias, res2, /*fused_allreduce=*/true);
      } else if (reduce) {
        y = GemmAllReduce(ctx, LaunchGemmQ4(ctx, x2, packed_, N_, bias, at::Tensor()), res2);
      } else {
        y = LaunchGemmQ4(ctx, x2, packed_, N_, bias, res2);
      }
      ctx.SetOutput(0, y.reshape(out_shape));
      return;
    }
    if (reduce || res.defined()) {
      Fallback(ctx);
      return;
    }
    const at::Tensor& B = ctx.RequiredInput(1);
    const at::Tensor& scales = ctx.RequiredInput(2);
    at::Tensor zp = ctx.HasInput(3) ? ctx.Input(3) : at::Tensor();
    const int dt = DtypeCode(a.scalar_type());
    const bool zp_packed = zp.defined() && zp.scalar_type() == at::kByte;
    if (dt < 0 || scales.scalar_type() != a.scalar_type() || (bits_ != 4 && bits_ != 8) || block_ < 16 ||
        (block_ & (block_ - 1)) != 0 || K_ % 8 != 0 || ctx.HasInput(4) || !B.is_cuda() ||
        (zp.defined() && !zp_packed && zp.scalar_type() != a.scalar_type())) {
      Fallback(ctx);
      return;
    }
    at::Tensor Bc = B.contiguous(), sc = scales.contiguous();
    if (zp.defined()) zp = zp.contiguous();
    at::Tensor w = at::empty({N_, K_}, a.options());
    CheckLaunch(ortb200_nbits_dequant(Bc.data_ptr(), sc.data_ptr(), zp.defined() ? zp.data_ptr() : nullptr, zp_packed ? 1 : 0,
                                      w.data_ptr(), N_, static_cast<int>(K_), static_cast<int>(bits_), static_cast<int>(block_), K_,
                                      dt, ctx.cuda_stream()),
                "ortb200_nbits_dequant");
    ctx.session()->AddLaunches(1);
    at::Tensor x2 = a.reshape({-1, K_}).contiguous();
    at::Tensor bias = ctx.HasInput(5) ? ctx.Input(5) : at::Tensor();
    at::Tensor y = LaunchGemm(ctx, x2, w, N_, 0, bias, at::Tensor(), ORTB200_ACT_NONE, 1.f);
    std::vector<int64_t> shape = a.sizes().vec();
    shape.back() = N_;
    ctx.SetOutput(0, y.reshape(shape));
  }

 private:
  int64_t K_ = 0, N_ = 0, bits_ = 4, block_ = 32;
  bool all_reduce_ = false;
  at::Tensor packed_, scales_;
};

// ---------------------------------------------------------------------------------------------------------------
// PagedAttention, decode form (one new token per sequence): rotary + cache write, then the split-KV kernel reading
// the cache through the block table.  Other forms (prompt chunks) take the generic path.
class PagedAttentionKernel final : public WithFallback {
 public:
  explicit PagedAttentionKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    N_ = n.attr_i("num_heads", 0);
    Nk_ = n.attr_i("kv_num_heads", 0);
    do_rotary_ = n.attr_i("do_rotary", 0) != 0;
    interleaved_ = n.attr_i("rotary_interleaved", 0) != 0;
    window_ = n.attr_i("local_window_size", -1);
    scale_ = n.attr_f("scale", 0.f);
    softcap_ = n.attr_f("softcap", 0.f);
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& query = ctx.RequiredInput(0);
    const at::Tensor& kc = ctx.RequiredInput(3);
    const at::Tensor& vc = ctx.RequiredInput(4);
    const at::Tensor& cum = ctx.RequiredInput(5);
    const at::Tensor& past = ctx.RequiredInput(6);
    const at::Tensor& table = ctx.RequiredInput(7);
    const int64_t T = query.size(0), B = past.numel();
    const int64_t H = kc.size(3), block_size = kc.size(1), num_blocks = kc.size(0);
    const bool packed = !ctx.HasInput(1);
    const int dt = DtypeCode(query.scalar_type());
    const bool decode = T == B;
    if (dt < 0 || !decode || (H != 64 && H != 128) || kc.scalar_type() != query.scalar_type() || !kc.is_contiguous() ||
        !vc.is_contiguous() || !cum.is_cuda() || !past.is_cuda() || !table.is_cuda() || cum.scalar_type() != at::kInt ||
        past.scalar_type() != at::kInt || table.scalar_type() != at::kInt ||
        (do_rotary_ && (!ctx.HasInput(8) || ctx.Input(8).scalar_type() != query.scalar_type()))) {
      Fallback(ctx);
      return;
    }
    at::Tensor qc = query.contiguous();
    at::Tensor q_rot = at::empty({T, N_, H}, query.options());
    at::Tensor tb = table.contiguous();
    // head size 128: the tcgen05 decode kernel rotates, appends and attends in one launch
    const bool fuse = packed && H == 128 && window_ <= 0 && (block_size & (block_size - 1)) == 0 && block_size >= 8 &&
                      (!do_rotary_ || ctx.Input(8).size(1) * 2 == H) && ctx.session()->config().Get("ortb200.fused_gqa_prep", "auto") != "0" &&
                      ctx.session()->config().Get("ortb200.decode_attention_algo", "0") != "1";
    ortb200_paged_prep_args pa{};
    pa.qkv = qc.data_ptr();
    at::Tensor kin, vin;
    if (!packed) {
      kin = ctx.Input(1).contiguous();
      vin = ctx.RequiredInput(2).contiguous();
      pa.k = kin.data_ptr();
      pa.v = vin.data_ptr();
    }
    pa.q_out = q_rot.data_ptr();
    pa.k_cache = kc.data_ptr();
    pa.v_cache = vc.data_ptr();
    pa.cu_seqlens = cum.data_ptr<int>();
    pa.past_seqlens = past.data_ptr<int>();
    pa.block_table = tb.data_ptr<int>();
    pa.cos_cache = do_rotary_ ? ctx.Input(8).data_ptr() : nullptr;
    pa.cos_rows = do_rotary_ ? static_cast<int>(ctx.Input(8).size(0)) : 0;
    pa.sin_cache = do_rotary_ ? ctx.RequiredInput(9).data_ptr() : nullptr;
    pa.T = static_cast<int>(T); pa.B = static_cast<int>(B); pa.N = static_cast<int>(N_); pa.Nk = static_cast<int>(Nk_);
    pa.H = static_cast<int>(H);
    pa.block_size = static_cast<int>(block_size); pa.max_blocks = static_cast<int>(tb.size(1)); pa.num_blocks = static_cast<int>(num_blocks);
    pa.rot_dim = do_rotary_ ? static_cast<int>(ctx.Input(8).size(1) * 2) : 0;
    pa.interleaved = interleaved_ ? 1 : 0;
    pa.do_rotary = do_rotary_ ? 1 : 0;
    pa.dtype = dt;
    pa.status = ctx.session()->StatusWord().data_ptr<int>();
    if (!fuse) CheckLaunch(ortb200_paged_prep(&pa, ctx.cuda_stream()), "ortb200_paged_prep");

    at::Tensor out = at::empty({T, N_ * H}, query.options());
    at::Tensor& ws = ctx.session()->AttnWorkspace(ortb200_gqa_decode_workspace_bytes(static_cast<int>(B), static_cast<int>(N_), static_cast<int>(H)));
    ortb200_gqa_decode_args da{};
    da.q = q_rot.data_ptr();
    da.k_cache = kc.data_ptr();
    da.v_cache = vc.data_ptr();
    da.seqlens_k = past.data_ptr<int>();  // total length - 1 == past length for a one-token step
    da.out = out.data_ptr();
    da.workspace = ws.data_ptr();
    da.workspace_bytes = ws.numel();
    da.B = static_cast<int>(B); da.N = static_cast<int>(N_); da.Nk = static_cast<int>(Nk_); da.H = static_cast<int>(H);
    da.Smax = static_cast<int>(tb.size(1) * block_size);
    da.window = static_cast<int>(window_);
    da.scale = scale_;
    da.softcap = softcap_;
    da.dtype = dt;
    da.use_pdl = 0;
    da.status = pa.status;
    da.block_table = tb.data_ptr<int>();
    da.block_size = static_cast<int>(block_size);
    da.max_blocks = static_cast<int>(tb.size(1));
    da.num_blocks = static_cast<int>(num_blocks);
    if (fuse) {
      da.qkv = qc.data_ptr();
      da.cos_cache = pa.cos_cache;
      da.cos_rows = pa.cos_rows;
      da.sin_cache = pa.sin_cache;
      da.do_rotary = pa.do_rotary;
      da.rotary_interleaved = pa.interleaved;
      da.algo = 2;
    }
    CheckLaunch(ortb200_gqa_decode(&da, ctx.cuda_stream()), "ortb200_gqa_decode(paged)");
    ctx.session()->AddLaunches(fuse ? 1 : 2);
    ctx.SetOutput(0, out);
    if (ctx.OutputCount() > 1) ctx.SetOutput(1, kc);
    if (ctx.OutputCount() > 2) ctx.SetOutput(2, vc);
  }

 private:
  int64_t N_ = 0, Nk_ = 0, window_ = -1;
  bool do_rotary_ = false, interleaved_ = false;
  float scale_ = 0.f, softcap_ = 0.f;
};

// ---------------------------------------------------------------------------------------------------------------
// Encoder attention on the tcgen05 flash kernel.  q / k / v are views described by strides, so neither the packed
// QKV projection output nor separate Q, K, V activations are transposed or copied.
struct EncoderAttnCall {
  at::Tensor q, k, v;          // any layout reachable as (batch, token, head, dim) with dim contiguous
  int64_t B, S, T, N, H;
  at::Tensor lengths;          // optional int32 [B]: keys [0, len) are valid
  at::Tensor key_mask;         // optional int32 [B, T]
  bool causal;
  float scale;
};

at::Tensor RunEncoderAttention(Ctx& ctx, const EncoderAttnCall& c, int dt) {
  at::Tensor out = at::empty({c.B, c.S, c.N, c.H}, c.q.options());
  ortb200_attn_prefill_args a{};
  a.q = c.q.data_ptr();
  a.k = c.k.data_ptr();
  a.v = c.v.data_ptr();
  at::Tensor lens_m1;
  if (c.lengths.defined()) {
    lens_m1 = (c.lengths.to(at::kInt) - 1).contiguous();
    a.seqlens_k = lens_m1.data_ptr<int>();
  }
  if (c.key_mask.defined()) a.key_mask = c.key_mask.data_ptr<int>();
  a.out = out.data_ptr();
  a.B = static_cast<int>(c.B); a.S = static_cast<int>(c.S); a.N = static_cast<int>(c.N); a.Nk = static_cast<int>(c.N);
  a.H = static_cast<int>(c.H);
  a.kv_len = static_cast<int>(c.T);
  a.q_strides[0] = c.q.stride(0); a.q_strides[1] = c.q.stride(1); a.q_strides[2] = c.q.stride(2);
  a.o_strides[0] = out.stride(0); a.o_strides[1] = out.stride(1); a.o_strides[2] = out.stride(2);
  // keys are addressed as (batch, head, position)
  a.kv_strides[0] = c.k.stride(0); a.kv_strides[1] = c.k.stride(2); a.kv_strides[2] = c.k.stride(1);
  a.first_prompt = 1;
  a.causal = c.causal ? 1 : 0;
  a.window = -1;
  a.scale = c.scale;
  a.dtype = dt;
  a.status = ctx.session()->StatusWord().data_ptr<int>();
  CheckLaunch(ortb200_attn_prefill(&a, ctx.cuda_stream()), "ortb200_attn_prefill(encoder)");
  ctx.session()->AddLaunches(1);
  return out;
}

// true when q, k, v (as [B, tokens, N, H] views) are usable by the kernel: dim contiguous, strides multiples of 8,
// k and v with identical strides (one stride triple describes both)
bool ViewsOk(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  auto ok = [](const at::Tensor& t) {
    if (t.stride(3) != 1) return false;
    for (int i = 0; i < 3; ++i)
      if (t.stride(i) % 8 != 0) return false;
    return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  return ok(q) && ok(k) && ok(v) && k.strides() == v.strides();
}

// mask_index -> (lengths | key mask).  Returns false for the forms the kernel does not take.
bool DecodeMask(const at::Tensor& m, int64_t B, int64_t T, at::Tensor* lengths, at::Tensor* key_mask) {
  if (m.dim() == 1 && m.size(0) == B) {
    *lengths = m;
    return true;
  }
  if (m.dim() == 2 && m.size(0) == B && m.size(1) == T) {
    *key_mask = m.ne(0).to(at::kInt).contiguous();
    return true;
  }
  return false;
}

class BertAttentionKernel final : public WithFallback {
 public:
  explicit BertAttentionKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    N_ = n.attr_i("num_heads", 1);
    causal_ = n.attr_i("unidirectional", 0) != 0;
    scale_ = n.attr_f("scale", 0.f);
    sizes_ = n.attr_ints("qkv_hidden_sizes");
    const at::Tensor* w = info.constant_input(1);
    if (w && w->dim() == 2 && HalfType(w->scalar_type()) && w->size(0) % 8 == 0) w_nk_ = w->t().contiguous();
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int dt = DtypeCode(x.scalar_type());
    const int64_t B = x.size(0), S = x.size(1);
    const int64_t W3 = w_nk_.defined() ? w_nk_.size(0) : 0;
    const bool equal_sizes = sizes_.empty() || (sizes_.size() == 3 && sizes_[0] == sizes_[1] && sizes_[1] == sizes_[2]);
    const int64_t H = W3 > 0 ? W3 / 3 / N_ : 0;
    at::Tensor lengths, key_mask;
    if (ctx.session()->config().Get("ortb200.math_attention", "0") == "1" ||
        dt < 0 || !w_nk_.defined() || w_nk_.scalar_type() != x.scalar_type() || !equal_sizes || (H != 64 && H != 128) ||
        ctx.HasInput(4) || ctx.HasInput(5) || (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) ||
        (ctx.HasInput(3) && !DecodeMask(ctx.Input(3), B, S, &lengths, &key_mask))) {
      Fallback(ctx);
      return;
    }
    at::Tensor bias = ctx.HasInput(2) ? ctx.Input(2) : at::Tensor();
    at::Tensor qkv = LaunchGemm(ctx, x.reshape({B * S, x.size(2)}).contiguous(), w_nk_, W3, 0, bias, at::Tensor(), ORTB200_ACT_NONE, 1.f);
    at::Tensor v5 = qkv.reshape({B, S, 3, N_, H});
    EncoderAttnCall c{v5.select(2, 0), v5.select(2, 1), v5.select(2, 2), B, S, S, N_, H, lengths, key_mask, causal_, scale_};
    ctx.SetOutput(0, RunEncoderAttention(ctx, c, dt).reshape({B, S, N_ * H}));
  }

 private:
  int64_t N_ = 1;
  bool causal_ = false;
  float scale_ = 0.f;
  std::vector<int64_t> sizes_;
  at::Tensor w_nk_;
};

class MultiHeadAttentionKernel final : public WithFallback {
 public:
  explicit MultiHeadAttentionKernel(const OpKernelInfo& info) : WithFallback(info) {
    N_ = info.node.attr_i("num_heads", 1);
    causal_ = info.node.attr_i("unidirectional", 0) != 0;
    scale_ = info.node.attr_f("scale", 0.f);
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& q_in = ctx.RequiredInput(0);
    const int dt = DtypeCode(q_in.scalar_type());
    const bool extra = ctx.HasInput(3) || ctx.HasInput(5) || ctx.HasInput(6) || ctx.HasInput(7) ||
                       (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) || (ctx.OutputCount() > 2 && ctx.OutputNeeded(2));
    if (dt < 0 || extra || ctx.session()->config().Get("ortb200.math_attention", "0") == "1") {
      Fallback(ctx);
      return;
    }
    const int64_t B = q_in.size(0), S = q_in.size(1);
    at::Tensor q, k, v;
    if (q_in.dim() == 5) {  // packed QKV [B, S, N, 3, H]
      q = q_in.select(3, 0);
      k = q_in.select(3, 1);
      v = q_in.select(3, 2);
    } else if (q_in.dim() == 3 && ctx.HasInput(1) && ctx.Input(1).dim() == 5) {  // packed KV [B, T, N, 2, H]
      const at::Tensor& kv = ctx.Input(1);
      q = q_in.reshape({B, S, N_, -1});
      k = kv.select(3, 0);
      v = kv.select(3, 1);
    } else if (q_in.dim() == 3 && ctx.HasInput(1) && ctx.Input(1).dim() == 3 && ctx.HasInput(2)) {
      q = q_in.reshape({B, S, N_, -1});
      k = ctx.Input(1).reshape({B, ctx.Input(1).size(1), N_, -1});
      v = ctx.Input(2).reshape({B, ctx.Input(2).size(1), N_, -1});
    } else {
      Fallback(ctx);
      return;
    }
    const int64_t T = k.size(1), H = q.size(3);
    at::Tensor lengths, key_mask;
    if ((H != 64 && H != 128) || v.size(3) != H || (causal_ && S != T) || !ViewsOk(q, k, v) ||
        (ctx.HasInput(4) && !DecodeMask(ctx.Input(4), B, T, &lengths, &key_mask))) {
      Fallback(ctx);
      return;
    }
    EncoderAttnCall c{q, k, v, B, S, T, N_, H, lengths, key_mask, causal_, scale_};
    ctx.SetOutput(0, RunEncoderAttention(ctx, c, dt).reshape({B, S, N_ * H}));
  }

 private:
  int64_t N_ = 1;
  bool causal_ = false;
  float scale_ = 0.f;
};

// ---------------------------------------------------------------------------------------------------------------
// MoE / ShardedMoE on the GPU: routing + permutation kernels, two grouped tcgen05 GEMMs driven by a device-side
// tile plan, weighted combine.  Seven launches, no host synchronisation.  With expert parallelism each rank serves its
// own experts and the partial outputs are summed across ranks.
class MoeKernel final : public WithFallback {
 public:
  explicit MoeKernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    sharded_ = n.op_type == "ShardedMoE";
    const bool quantised = n.op_type == "QMoE";
    attrs_ = contrib::ParseMoeAttrs(n);
    start_ = sharded_ ? n.attr_i("local_experts_start_index", 0) : 0;
    tensor_shards_ = sharded_ ? n.attr_i("tensor_shards", 1) : 1;
    // input slots: MoE (x, router, fc1, b1, fc2, b2, fc3, b3); QMoE adds a scales input behind every weight
    const int i1 = 2, i2 = quantised ? 5 : 4, i3 = quantised ? 8 : 6;
    b1_ = quantised ? 4 : 3;
    b2_ = quantised ? 7 : 5;
    b3_ = quantised ? 10 : 7;
    auto has = [&](int i) { return static_cast<int>(n.inputs.size()) > i && !n.inputs[i].empty(); };
    const at::Tensor* fc1 = info.constant_input(i1);
    const at::Tensor* fc2 = info.constant_input(i2);
    const bool has_fc3 = has(i3);
    const at::Tensor* fc3 = has_fc3 ? info.constant_input(i3) : nullptr;
    at::Tensor dq1, dq2, dq3;
    if (quantised) {
      // expert weights are expanded once, at session creation, to the scales' 16-bit type: the grouped GEMMs then run
      // as for MoE (memory for speed; the packed form stays the model's storage format)
      const at::Tensor* s1 = info.constant_input(3);
      const at::Tensor* s2 = info.constant_input(6);
      const at::Tensor* s3 = has_fc3 ? info.constant_input(9) : nullptr;
      if (!fc1 || !fc2 || !s1 || !s2 || (has_fc3 && (!fc3 || !s3)) || !HalfType(s1->scalar_type())) return;
      const int64_t bits = n.attr_i("expert_weight_bits", 4), block = n.attr_i("block_size", 0);
      dq1 = contrib::DequantizeQMoeWeights(*fc1, *s1, bits, block).to(s1->scalar_type());
      dq2 = contrib::DequantizeQMoeWeights(*fc2, *s2, bits, block).to(s1->scalar_type());
      if (has_fc3) dq3 = contrib::DequantizeQMoeWeights(*fc3, *s3, bits, block).to(s1->scalar_type());
      fc1 = &dq1;
      fc2 = &dq2;
      if (has_fc3) fc3 = &dq3;
    }
    if (!fc1 || !fc2 || (has_fc3 && !fc3) || !HalfType(fc1->scalar_type()) || fc1->dim() != 3 || fc2->dim() != 3) return;
    if (attrs_.activation == "swiglu" || tensor_shards_ > 1) return;
    if (has_fc3 && attrs_.activation != "silu") return;
    // to [E, out, in] with `in` contiguous; ShardedMoE stores [E, in, out]
    at::Tensor w1 = sharded_ ? fc1->transpose(1, 2) : *fc1;
    at::Tensor w2 = sharded_ ? fc2->transpose(1, 2) : *fc2;
    E_local_ = w1.size(0);
    I_ = w1.size(1);
    H_ = w1.size(2);
    if (w2.size(1) != H_ || w2.size(2) != I_ || H_ % 8 != 0 || I_ % 8 != 0) return;
    if (has_fc3) {
      at::Tensor w3 = sharded_ ? fc3->transpose(1, 2) : *fc3;
      if (w3.sizes() != w1.sizes()) return;
      w13_ = at::cat({w1, w3}, 1).contiguous();  // gate rows, then up rows
      dual_ = true;
    } else {
      w13_ = w1.contiguous();
    }
    w2_ = w2.contiguous();
    ok_ = true;
  }
  std::vector<int> PrepackedInputs() const override { return {}; }

  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    const at::Tensor& logits_in = ctx.RequiredInput(1);
    const int dt = DtypeCode(x.scalar_type());
    const bool fc3_bias = ctx.HasInput(b3_);
    // tokens_sharded: the dispatch / combine form lives in the generic kernel (process-group all-to-all around the experts)
    if (!ok_ || dt < 0 || x.scalar_type() != w13_.scalar_type() || x.size(-1) != H_ || fc3_bias ||
        attrs_.k > 8 || logits_in.size(-1) > 256 || node_.attr_i("tokens_sharded", 0) != 0) {
      Fallback(ctx);
      return;
    }
    at::Tensor x2 = x.reshape({-1, H_}).contiguous();
    const int64_t T = x2.size(0), E = logits_in.size(-1), k = attrs_.k;
    at::Tensor logits = logits_in.reshape({T, E}).contiguous();
    int ldt = DtypeCode(logits.scalar_type());
    if (logits.scalar_type() == at::kFloat) ldt = ORTB200_F32;
    if (ldt < 0) {
      Fallback(ctx);
      return;
    }
    const int64_t R = T * k;
    int tile_rows = ortb200_moe_tile_rows(R, static_cast<int>(E_local_));
    // the gated (two-accumulator) kernel stops at 128-token tiles; without a bias the 256-token path runs the gate
    // and up projections as one plain GEMM followed by a streaming SwiGLU
    if (dual_ && tile_rows == 256 && ctx.HasInput(b1_)) tile_rows = 128;
    const int max_tiles = ortb200_moe_max_tiles(R, static_cast<int>(E_local_), tile_rows);
    auto iopt = x.options().dtype(at::kInt);
    at::Tensor topk_idx = at::empty({T, k}, iopt), row_of = at::empty({T, k}, iopt);
    at::Tensor topk_w = at::empty({T, k}, x.options().dtype(at::kFloat));
    at::Tensor ints = at::empty({3 * E_local_ + 2 + 4}, iopt);  // counts | offsets | cursors | num_tiles
    at::Tensor tile_info = at::empty({max_tiles, 4}, iopt);
    at::Tensor xp = at::zeros({R, H_}, x.options());
    ortb200_moe_route_args ra{};
    ra.logits = logits.data_ptr();
    ra.x = x2.data_ptr();
    ra.tokens = static_cast<int>(T); ra.E = static_cast<int>(E); ra.k = static_cast<int>(k); ra.H = static_cast<int>(H_);
    ra.normalize = attrs_.normalize ? 1 : 0;
    ra.expert_begin = static_cast<int>(start_);
    ra.expert_end = static_cast<int>(start_ + E_local_);
    ra.tile_rows = tile_rows; ra.max_tiles = max_tiles;
    ra.dtype = ldt;
    ra.topk_idx = topk_idx.data_ptr<int>();
    ra.topk_w = topk_w.data_ptr<float>();
    int* ip = ints.data_ptr<int>();
    ra.counts = ip;
    ra.offsets = ip + E_local_;
    ra.cursors = ip + 2 * E_local_ + 1;
    ra.num_tiles = ip + 3 * E_local_ + 1;
    ra.tile_info = tile_info.data_ptr();
    ra.xp = xp.data_ptr();
    ra.row_of = row_of.data_ptr<int>();
    if (ra.expert_end > ra.E) {
      Fallback(ctx);
      return;
    }
    CheckLaunch(ortb200_moe_route(&ra, ctx.cuda_stream()), "ortb200_moe_route");

    at::Tensor fc1_bias = ctx.HasInput(b1_) ? ctx.Input(b1_).contiguous() : at::Tensor();
    at::Tensor fc2_bias = ctx.HasInput(b2_) ? ctx.Input(b2_).contiguous() : at::Tensor();
    if (fc2_bias.defined() && fc2_bias.size(0) != E_local_) fc2_bias = fc2_bias.narrow(0, start_, E_local_).contiguous();
    at::Tensor h = at::empty({R, I_}, x.options());
    ortb200_gemm_grouped_args g{};
    g.x = xp.data_ptr(); g.w = w13_.data_ptr(); g.out = h.data_ptr();
    g.bias = fc1_bias.defined() ? fc1_bias.data_ptr() : nullptr;
    g.tile_info = tile_info.data_ptr(); g.num_tiles = ra.num_tiles;
    g.rows = static_cast<int>(R); g.N = static_cast<int>(I_); g.K = static_cast<int>(H_);
    g.num_experts = static_cast<int>(E_local_);
    g.w_rows_per_expert = static_cast<int>(dual_ ? 2 * I_ : I_);
    g.dual_offset = dual_ ? static_cast<int>(I_) : 0;
    g.tile_rows = tile_rows; g.max_tiles = max_tiles;
    g.dtype = dt;
    g.act = dual_ ? ORTB200_ACT_SWIGLU : ActOf(attrs_.activation);
    g.status = ctx.session()->StatusWord().data_ptr<int>();
    if (dual_ && tile_rows == 256) {
      at::Tensor gu = at::empty({R, 2 * I_}, x.options());
      g.out = gu.data_ptr();
      g.N = static_cast<int>(2 * I_);
      g.dual_offset = 0;
      g.act = ORTB200_ACT_NONE;
      CheckLaunch(ortb200_gemm_grouped(&g, ctx.cuda_stream()), "ortb200_gemm_grouped(fc1|fc3)");
      CheckLaunch(ortb200_swiglu(gu.data_ptr(), h.data_ptr(), R, static_cast<int>(I_), dt, ctx.cuda_stream()), "ortb200_swiglu");
      ctx.session()->AddLaunches(1);
    } else {
      CheckLaunch(ortb200_gemm_grouped(&g, ctx.cuda_stream()), "ortb200_gemm_grouped(fc1)");
    }
    at::Tensor y = at::empty({R, H_}, x.options());
    g.x = h.data_ptr(); g.w = w2_.data_ptr(); g.out = y.data_ptr(); g.bias = nullptr;
    g.N = static_cast<int>(H_); g.K = static_cast<int>(I_);
    g.w_rows_per_expert = static_cast<int>(H_); g.dual_offset = 0; g.act = ORTB200_ACT_NONE;
    CheckLaunch(ortb200_gemm_grouped(&g, ctx.cuda_stream()), "ortb200_gemm_grouped(fc2)");
    at::Tensor out = at::empty({T, H_}, x.options());
    InferenceSession* sess = ctx.session();
    if (sharded_ && sess->world_size > 1 && static_cast<int>(sess->symm_peers.size()) == sess->world_size &&
        sess->config().Get("ortb200.fused_moe_combine", "1") == "1" && E == E_local_ * sess->world_size &&
        start_ == sess->rank * E_local_ &&
        T <= ortb200_moe_combine_symm_max_tokens(sess->world_size, static_cast<int>(k), static_cast<int>(H_), sess->symm_bytes)) {
      // expert parallelism: un-permute, scale, sum across ranks and replicate in one kernel over peer memory
      ortb200_moe_combine_symm_args ca{};
      ca.y = y.data_ptr();
      ca.bias = fc2_bias.defined() ? fc2_bias.data_ptr() : nullptr;
      ca.out = out.data_ptr();
      ca.topk_idx = topk_idx.data_ptr<int>(); ca.topk_w = topk_w.data_ptr<float>(); ca.row_of = row_of.data_ptr<int>();
      ca.T = static_cast<int>(T); ca.H = static_cast<int>(H_); ca.k = static_cast<int>(k);
      ca.E_local = static_cast<int>(E_local_); ca.expert_begin = static_cast<int>(start_);
      ca.dtype = dt;
      ca.world = sess->world_size; ca.rank = sess->rank;
      for (int i = 0; i < sess->world_size && i < 8; ++i) ca.peers[i] = sess->symm_peers[i];
      ca.symm_bytes = sess->symm_bytes;
      ca.status = sess->StatusWord().data_ptr<int>();
      CheckLaunch(ortb200_moe_combine_symm(&ca, ctx.cuda_stream()), "ortb200_moe_combine_symm");
      sess->AddLaunches(6);
      ctx.SetOutput(0, out.reshape(x.sizes()));
      return;
    }
    CheckLaunch(ortb200_moe_combine(y.data_ptr(), fc2_bias.defined() ? fc2_bias.data_ptr() : nullptr, out.data_ptr(), static_cast<int>(T),
                                    static_cast<int>(H_), static_cast<int>(k), static_cast<int>(start_), topk_idx.data_ptr<int>(),
                                    topk_w.data_ptr<float>(), row_of.data_ptr<int>(), dt, ctx.cuda_stream()),
                "ortb200_moe_combine");
    ctx.session()->AddLaunches(6);
    if (sharded_ && ctx.session()->world_size > 1) out = AllReduceSum(ctx.session(), out.to(at::kFloat)).to(x.scalar_type());
    ctx.SetOutput(0, out.reshape(x.sizes()));
  }

 private:
  static int ActOf(const std::string& a) {
    if (a == "relu") return ORTB200_ACT_RELU;
    if (a == "gelu") return ORTB200_ACT_GELU;
    if (a == "silu") return ORTB200_ACT_SILU;
    return ORTB200_ACT_NONE;
  }
  contrib::MoeAttrs attrs_;
  bool sharded_ = false, ok_ = false, dual_ = false;
  int b1_ = 3, b2_ = 5, b3_ = 7;
  int64_t start_ = 0, tensor_shards_ = 1, E_local_ = 0, I_ = 0, H_ = 0;
  at::Tensor w13_, w2_;
};

// ---------------------------------------------------------------------------------------------------------------
// AllReduce / AllGather / AllToAll as one kernel over the session's peer-mapped workspace; messages that do not fit
// (or sessions without a workspace) go through the process group instead.
class SymmCollectiveKernel final : public WithFallback {
 public:
  explicit SymmCollectiveKernel(const OpKernelInfo& info) : WithFallback(info) {
    const std::string& op = info.node.op_type;
    op_ = op == "AllReduce" ? ORTB200_COLL_ALLREDUCE : (op == "AllGather" ? ORTB200_COLL_ALLGATHER : ORTB200_COLL_ALLTOALL);
    axis_ = info.node.attr_i("axis", 0);
  }
  void Compute(Ctx& ctx) const override {
    InferenceSession* s = ctx.session();
    const int world = s->world_size;
    if (world <= 1 || world > 8 || static_cast<int>(s->symm_peers.size()) != world ||
        s->config().Get("ortb200.symm_collectives", "1") != "1") {
      Fallback(ctx);
      return;
    }
    const int n = op_ == ORTB200_COLL_ALLREDUCE ? std::min(ctx.InputCount(), ctx.OutputCount()) : 1;
    // decide for the whole node first: either every tensor takes the kernel or the node falls back
    for (int i = 0; i < n; ++i) {
      if (!ctx.HasInput(i)) continue;
      if (!Plan(ctx.Input(i), world, s->symm_bytes, nullptr)) {
        Fallback(ctx);
        return;
      }
    }
    for (int i = 0; i < n; ++i) {
      if (!ctx.HasInput(i)) continue;
      at::Tensor in = ctx.Input(i).contiguous();
      ortb200_symm_collective_args a{};
      Plan(in, world, s->symm_bytes, &a);
      std::vector<int64_t> shape = in.sizes().vec();
      if (op_ == ORTB200_COLL_ALLGATHER) {
        if (shape.empty()) shape = {1};
        shape[Axis(in)] *= world;
      }
      at::Tensor out = at::empty(shape, in.options());
      a.op = op_;
      a.in = in.data_ptr();
      a.out = out.data_ptr();
      a.world = world;
      a.rank = s->rank;
      for (int r = 0; r < world; ++r) a.peers[r] = s->symm_peers[r];
      a.symm_bytes = s->symm_bytes;
      a.mc_ptr = s->NvlsPointer();
      a.status = s->StatusWord().data_ptr<int>();
      a.use_pdl = s->config().Get("ortb200.pdl", "0") == "1" ? 1 : 0;
      CheckLaunch(ortb200_symm_collective(&a, ctx.cuda_stream()), "ortb200_symm_collective");
      s->AddLaunches(1);
      ctx.SetOutput(i, out);
    }
  }

 private:
  int64_t Axis(const at::Tensor& t) const {
    const int64_t d = std::max<int64_t>(t.dim(), 1);
    return axis_ < 0 ? axis_ + d : axis_;
  }
  // fills rows / row_bytes / dtype; false when the kernel cannot take this tensor
  bool Plan(const at::Tensor& t, int world, int64_t symm_bytes, ortb200_symm_collective_args* a) const {
    if (!t.defined() || !t.is_cuda() || t.numel() == 0) return false;
    const int64_t esz = t.element_size();
    const int64_t bytes = t.numel() * esz;
    const int64_t limit = ortb200_symm_collective_max_bytes(op_, world, symm_bytes);
    int64_t rows = 1, row_bytes = bytes;
    int dt = 0;
    if (op_ == ORTB200_COLL_ALLREDUCE) {
      if (t.scalar_type() == at::kBFloat16) dt = ORTB200_BF16;
      else if (t.scalar_type() == at::kHalf) dt = ORTB200_F16;
      else if (t.scalar_type() == at::kFloat) dt = ORTB200_F32;
      else return false;
      if (bytes % 16 != 0 || bytes > limit) return false;
    } else if (op_ == ORTB200_COLL_ALLGATHER) {
      const int64_t ax = Axis(t);
      if (ax < 0 || ax >= std::max<int64_t>(t.dim(), 1)) return false;
      for (int64_t d = 0; d < ax; ++d) rows *= t.size(d);
      row_bytes = bytes / rows;
      if (row_bytes % 16 != 0 || bytes > limit) return false;
    } else {
      if (bytes % (16 * world) != 0 || bytes > limit) return false;
      row_bytes = bytes / world;
    }
    if (a) {
      a->rows = rows;
      a->row_bytes = row_bytes;
      a->dtype = dt;
    }
    return true;
  }
  int op_ = 0;
  int64_t axis_ = 0;
};

// ---------------------------------------------------------------------------------------------------------------
// GemmFloat8 with e4m3 operands: Y = act(alpha * scaleA * scaleB * A @ B^T + C) / scaleY on the 8-bit tensor-core path.
class GemmFloat8Kernel final : public WithFallback {
 public:
  explicit GemmFloat8Kernel(const OpKernelInfo& info) : WithFallback(info) {
    const Node& n = info.node;
    trans_a_ = n.attr_i("transA", 0) != 0;
    trans_b_ = n.attr_i("transB", 0) != 0;
    alpha_ = n.attr_f("alpha", 1.f);
    beta_ = n.attr_f("beta", 0.f);
    act_name_ = n.attr_s("activation", "NONE");
    out_dtype_ = n.attr_i("dtype", 1);
    const at::Tensor* b = info.constant_input(1);
    if (b && b->dim() == 2 && b->scalar_type() == at::kFloat8_e4m3fn && !trans_b_)
      b_nk_ = b->view(at::kByte).t().contiguous().view(at::kFloat8_e4m3fn);  // pre-pack to [N, K]
    for (int i = 3; i <= 5; ++i) {
      const at::Tensor* sc = static_cast<int>(n.inputs.size()) > i && !n.inputs[i].empty() ? info.constant_input(i) : nullptr;
      if (sc) const_scale_[i - 3] = sc->to(at::kCPU, at::kFloat).reshape({-1})[0].item<float>();
    }
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& A = ctx.RequiredInput(0);
    at::ScalarType out_t = out_dtype_ == 10 ? at::kHalf : (out_dtype_ == 16 ? at::kBFloat16 : at::ScalarType::Undefined);
    const bool b_ok = b_nk_.defined() || (trans_b_ && ctx.RequiredInput(1).scalar_type() == at::kFloat8_e4m3fn);
    int act = ORTB200_ACT_NONE;
    bool act_ok = true;
    if (act_name_ == "RELU") act = ORTB200_ACT_RELU;
    else if (act_name_ == "GELU") act = ORTB200_ACT_GELU;
    else if (act_name_ != "NONE") act_ok = false;
    at::Tensor bias;
    bool c_ok = true;
    if (ctx.HasInput(2)) {
      bias = ctx.Input(2);
      c_ok = beta_ == 1.f && bias.dim() == 1 && bias.scalar_type() == out_t;
    }
    // scaleY divides after the activation; with an activation in between it cannot be folded into alpha
    const bool has_sy = ctx.HasInput(5);
    if (A.scalar_type() != at::kFloat8_e4m3fn || A.dim() != 2 || trans_a_ || !b_ok || out_t == at::ScalarType::Undefined || !act_ok ||
        !c_ok || (has_sy && (act != ORTB200_ACT_NONE || bias.defined())) || A.size(1) % 16 != 0) {
      Fallback(ctx);
      return;
    }
    // constant scales fold into alpha on the host; scales that are computed at run time stay on the device and the
    // kernel multiplies their product in (no host read, so the node can sit inside a captured graph)
    float alpha = alpha_;
    at::Tensor alpha_dev;
    auto fold = [&](int i, bool divide) {
      if (!ctx.HasInput(i)) return;
      if (!std::isnan(const_scale_[i - 3])) {
        alpha = divide ? alpha / const_scale_[i - 3] : alpha * const_scale_[i - 3];
        return;
      }
      at::Tensor s = ctx.Input(i).to(A.device(), at::kFloat).reshape({1});
      if (divide) s = s.reciprocal();
      alpha_dev = alpha_dev.defined() ? alpha_dev * s : s;
    };
    fold(3, false);
    fold(4, false);
    if (has_sy) fold(5, true);
    if (alpha_dev.defined()) alpha_dev = alpha_dev.contiguous();
    at::Tensor w = b_nk_.defined() ? b_nk_ : ctx.Input(1).contiguous();
    at::Tensor y = LaunchGemm(ctx, A.contiguous(), w, w.size(0), 0, bias, at::Tensor(), act, alpha, false, out_t, 0.f, alpha_dev);
    ctx.SetOutput(0, y);
  }

 private:
  bool trans_a_ = false, trans_b_ = false;
  float alpha_ = 1.f, beta_ = 0.f;
  std::string act_name_;
  int64_t out_dtype_ = 1;
  at::Tensor b_nk_;
  float const_scale_[3] = {NAN, NAN, NAN};
};

template <typename K>
void Reg(KernelRegistry& r, const std::string& domain, const std::string& op, std::vector<int> host = {},
         std::function<bool(const Node&, const Graph&)> supports = nullptr) {
  KernelDef d;
  d.domain = domain;
  d.op_type = op;
  d.host_inputs = std::move(host);
  d.supports = std::move(supports);
  d.factory = [](const OpKernelInfo& info) { return std::make_unique<K>(info); };
  r.Register(std::move(d));
}

}  // namespace

// EmbedLayerNormalization: gather of the three embedding rows + LayerNorm in one kernel.
class EmbedLayerNormKernel final : public WithFallback {
 public:
  explicit EmbedLayerNormKernel(const OpKernelInfo& info) : WithFallback(info) { eps_ = info.node.attr_f("epsilon", 1e-12f); }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& ids = ctx.RequiredInput(0);
    const at::Tensor& word = ctx.RequiredInput(2);
    const at::Tensor& pos = ctx.RequiredInput(3);
    const int dt = word.scalar_type() == at::kFloat ? static_cast<int>(ORTB200_F32) : DtypeCode(word.scalar_type());
    const bool has_seg = ctx.HasInput(1) && ctx.HasInput(4);
    auto id_ok = [&](const at::Tensor& t) {
      return t.is_cuda() && t.is_contiguous() && (t.scalar_type() == at::kInt || t.scalar_type() == at::kLong) &&
             t.scalar_type() == ids.scalar_type();
    };
    const int64_t H = word.size(1);
    bool ok = dt >= 0 && ids.dim() == 2 && id_ok(ids) && word.is_cuda() && word.is_contiguous() && pos.is_contiguous() &&
              pos.scalar_type() == word.scalar_type() && (H * word.element_size()) % 16 == 0 && H * word.element_size() <= 8192 &&
              ctx.RequiredInput(5).scalar_type() == word.scalar_type() && ctx.RequiredInput(6).scalar_type() == word.scalar_type();
    if (ok && has_seg) ok = id_ok(ctx.Input(1)) && ctx.Input(4).is_contiguous() && ctx.Input(4).scalar_type() == word.scalar_type();
    at::Tensor pos_ids;
    if (ok && ctx.HasInput(8)) {
      pos_ids = ctx.Input(8);
      ok = id_ok(pos_ids) && pos_ids.dim() == 2 && pos_ids.size(1) == ids.size(1) && (pos_ids.size(0) == ids.size(0) || pos_ids.size(0) == 1);
    }
    if (!ok) {
      Fallback(ctx);
      return;
    }
    const int64_t B = ids.size(0), S = ids.size(1);
    at::Tensor out = at::empty({B, S, H}, word.options());
    at::Tensor sum_out;
    const bool want_sum = ctx.OutputCount() > 2 && ctx.OutputNeeded(2);
    if (want_sum) sum_out = at::empty({B, S, H}, word.options());
    at::Tensor gamma = ctx.RequiredInput(5).contiguous(), beta = ctx.RequiredInput(6).contiguous();
    ortb200_embed_layernorm_args a{};
    a.input_ids = ids.data_ptr();
    a.segment_ids = has_seg ? ctx.Input(1).data_ptr() : nullptr;
    a.position_ids = pos_ids.defined() ? pos_ids.data_ptr() : nullptr;
    a.word_emb = word.data_ptr();
    a.pos_emb = pos.data_ptr();
    a.segment_emb = has_seg ? ctx.Input(4).data_ptr() : nullptr;
    a.gamma = gamma.data_ptr();
    a.beta = beta.data_ptr();
    a.out = out.data_ptr();
    a.sum_out = want_sum ? sum_out.data_ptr() : nullptr;
    a.B = static_cast<int>(B); a.S = static_cast<int>(S); a.hidden = static_cast<int>(H);
    a.word_rows = static_cast<int>(word.size(0)); a.pos_rows = static_cast<int>(pos.size(0));
    a.seg_rows = has_seg ? static_cast<int>(ctx.Input(4).size(0)) : 0;
    a.id_bytes = ids.scalar_type() == at::kLong ? 8 : 4;
    a.position_broadcast = pos_ids.defined() && pos_ids.size(0) == 1 && B > 1 ? 1 : 0;
    a.epsilon = eps_;
    a.dtype = dt;
    a.status = ctx.session()->StatusWord().data_ptr<int>();
    CheckLaunch(ortb200_embed_layernorm(&a, ctx.cuda_stream()), "ortb200_embed_layernorm");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, out);
    if (ctx.OutputCount() > 1 && ctx.OutputNeeded(1)) {
      if (ctx.HasInput(7)) ctx.SetOutput(1, ctx.Input(7).to(at::kInt).sum(-1).to(at::kInt));
      else ctx.SetOutput(1, at::zeros({B}, at::TensorOptions().dtype(at::kInt).device(word.device())));
    }
    if (want_sum) ctx.SetOutput(2, sum_out);
  }

 private:
  float eps_ = 1e-12f;
};

// MatMulBlockQuantizedFp8Weight: the fp8 weight with its per-block scales is expanded to the activation type once (at
// the first call; constant weights only) and the product runs on the tcgen05 GEMM.  Weight-only block scaling cannot
// ride the 8-bit tensor-core mode, whose accumulation would need one scale per output instead of one per K block.
class BlockFp8WeightMatMulKernel final : public WithFallback {
 public:
  explicit BlockFp8WeightMatMulKernel(const OpKernelInfo& info) : WithFallback(info) {
    block_ = info.node.attr_i("block_size", 128);
    const_weight_ = info.constant_input(1) != nullptr && info.constant_input(2) != nullptr;
  }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& a = ctx.RequiredInput(0);
    const at::Tensor& b = ctx.RequiredInput(1);
    const int dt = DtypeCode(a.scalar_type());
    if (!const_weight_ || ctx.HasInput(3) || dt < 0 || !a.is_cuda() || b.dim() != 2 || b.scalar_type() != at::kFloat8_e4m3fn ||
        b.size(1) % 8 != 0 || (ctx.HasInput(4) && ctx.Input(4).scalar_type() != a.scalar_type())) {
      Fallback(ctx);
      return;
    }
    const int64_t K = b.size(1), N = b.size(0);
    at::Tensor x2 = a.reshape({-1, K}).contiguous();
    at::Tensor bias = ctx.HasInput(4) ? ctx.Input(4) : at::Tensor();
    at::Tensor y;
    // decode-shaped calls keep the weights in fp8: the kernel expands them on their way to the tensor cores (half the
    // bytes of the 16-bit copy); larger ones use a 16-bit copy that is made when the first such call arrives
    const bool in_kernel = x2.size(0) <= 64 && K % 64 == 0 && block_ % 64 == 0 &&
                           ctx.session()->config().Get("ortb200.fp8_weight_in_kernel", "1") != "0";
    if (in_kernel) {
      {
        std::lock_guard<std::mutex> lock(mu_);
        if (!blobs_.defined()) blobs_ = Fp8WeightBuildBlobs(b, ctx.RequiredInput(2), block_);
      }
      y = LaunchGemmQ4(ctx, x2, blobs_, N, bias, at::Tensor(), false, ORTB200_F8W);
    } else {
      {
        std::lock_guard<std::mutex> lock(mu_);
        if (!w_.defined() || w_.scalar_type() != a.scalar_type()) {
          at::Tensor s = ctx.RequiredInput(2).to(at::kFloat).repeat_interleave(block_, 1).narrow(1, 0, b.size(1));
          w_ = (b.to(at::kFloat) * s).to(a.scalar_type()).contiguous();
        }
      }
      y = LaunchGemm(ctx, x2, w_, N, 0, bias, at::Tensor(), ORTB200_ACT_NONE, 1.f);
    }
    std::vector<int64_t> shape(a.sizes().begin(), a.sizes().end());
    shape.back() = N;
    ctx.SetOutput(0, y.reshape(shape));
  }

 private:
  int64_t block_ = 128;
  bool const_weight_ = false;
  mutable std::mutex mu_;
  mutable at::Tensor w_, blobs_;
};

// ---------------------------------------------------------------------------------------------------------------
// com.ortb200.AllGatherMatMul: Y = concat over ranks of X_local (axis 0) @ W (+ bias) as one kernel over the session's
// peer-mapped workspace.  Shapes the kernel does not take (or sessions without a workspace) run the generic form:
// the process group's all-gather, then a matmul.
class AllGatherMatMulKernel final : public WithFallback {
 public:
  explicit AllGatherMatMulKernel(const OpKernelInfo& info) : WithFallback(info) {
    const at::Tensor* w = info.constant_input(1);
    if (w && w->dim() == 2 && (w->scalar_type() == at::kHalf || w->scalar_type() == at::kBFloat16)) w_nk_ = w->t().contiguous();
  }
  void Compute(Ctx& ctx) const override {
    InferenceSession* s = ctx.session();
    const at::Tensor& x = ctx.RequiredInput(0);
    const int world = s->world_size;
    const bool ok = w_nk_.defined() && x.is_cuda() && x.dim() >= 2 && x.scalar_type() == w_nk_.scalar_type() && x.size(-1) == w_nk_.size(1) &&
                    world > 1 && world <= 8 && static_cast<int>(s->symm_peers.size()) == world && x.numel() > 0 && x.size(-1) % 8 == 0 &&
                    s->config().Get("ortb200.symm_collectives", "1") == "1" &&
                    x.numel() / x.size(-1) <= ortb200_allgather_gemm_max_rows(world, static_cast<int>(x.size(-1)), s->symm_bytes) &&
                    (!ctx.HasInput(2) || (ctx.Input(2).dim() == 1 && ctx.Input(2).scalar_type() == x.scalar_type()));
    if (!ok) {
      Fallback(ctx);
      return;
    }
    at::Tensor x2 = x.reshape({-1, x.size(-1)}).contiguous();
    std::vector<int64_t> shape = x.sizes().vec();
    shape[0] *= world;
    shape.back() = w_nk_.size(0);
    at::Tensor out = at::empty({x2.size(0) * world, w_nk_.size(0)}, x.options());
    at::Tensor bias = ctx.HasInput(2) ? ctx.Input(2).contiguous() : at::Tensor();
    ortb200_allgather_gemm_args a{};
    a.x_local = x2.data_ptr();
    a.w = w_nk_.data_ptr();
    a.bias = bias.defined() ? bias.data_ptr() : nullptr;
    a.out = out.data_ptr();
    a.rows_local = static_cast<int>(x2.size(0));
    a.N = static_cast<int>(w_nk_.size(0));
    a.K = static_cast<int>(x2.size(1));
    a.dtype = x.scalar_type() == at::kBFloat16 ? ORTB200_BF16 : ORTB200_F16;
    a.act = ORTB200_ACT_NONE;
    a.world = world;
    a.rank = s->rank;
    for (int r = 0; r < world; ++r) a.peers[r] = s->symm_peers[r];
    a.symm_bytes = s->symm_bytes;
    a.status = s->StatusWord().data_ptr<int>();
    a.use_pdl = s->config().Get("ortb200.pdl", "0") == "1" ? 1 : 0;
    CheckLaunch(ortb200_allgather_gemm(&a, ctx.cuda_stream()), "ortb200_allgather_gemm");
    s->AddLaunches(1);
    ctx.SetOutput(0, out.reshape(shape));
  }

 private:
  at::Tensor w_nk_;
};

void RegisterCudaKernels3(KernelRegistry& r) {
  Reg<MatMulNBitsKernel>(r, MS, "MatMulNBits");
  Reg<PagedAttentionKernel>(r, MS, "PagedAttention");
  Reg<BertAttentionKernel>(r, MS, "Attention");
  Reg<MultiHeadAttentionKernel>(r, MS, "MultiHeadAttention");
  Reg<MoeKernel>(r, MS, "MoE");
  Reg<MoeKernel>(r, MS, "ShardedMoE");
  Reg<MoeKernel>(r, MS, "QMoE");
  Reg<GemmFloat8Kernel>(r, MS, "GemmFloat8");
  Reg<BlockFp8WeightMatMulKernel>(r, MS, "MatMulBlockQuantizedFp8Weight");
  Reg<EmbedLayerNormKernel>(r, MS, "EmbedLayerNormalization");
  Reg<SymmCollectiveKernel>(r, MS, "AllReduce");
  Reg<SymmCollectiveKernel>(r, MS, "AllGather");
  Reg<SymmCollectiveKernel>(r, MS, "AllToAll");
  Reg<AllGatherMatMulKernel>(r, "com.ortb200", "AllGatherMatMul");
}

}  // namespace ortb
