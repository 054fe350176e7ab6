// GPU execution provider: op kernels that launch the hand-written sm_100a
// kernels of libortb200_kernels (csrc/cuda).  Each class parses its attributes
// and pre-packs constant weights once at session initialisation; Compute()
// only fills an argument struct and launches on the current torch stream, so a
// whole decode step is a flat, CUDA-graph-capturable launch sequence.
//
// Reference counterparts: onnxruntime/core/providers/cuda/math/matmul.cc,
// onnxruntime/contrib_ops/cuda/bert/{skip_layer_norm.cc,rotary_embedding.cc,
// group_query_attention.cc,fast_gelu.cc}, quantization/matmul_nbits.cc, moe/moe.cc.
#include <ATen/ATen.h>
#include <sstream>
#include <chrono>
#include <ATen/cuda/CUDAContext.h>

#include "cuda_ops.h"
#include "kernel.h"
#include "ortb200_kernels.h"
#include "session.h"

namespace ortb {

namespace {

using Ctx = OpKernelContext;
constexpr int kMax = 1 << 30;
constexpr const char* MS = kMSDomain;
constexpr const char* kFusedDomain = "com.ortb200";

int DtypeCode(at::ScalarType t) {
  if (t == at::kHalf) return ORTB200_F16;
  if (t == at::kBFloat16) return ORTB200_BF16;
  if (t == at::kFloat) return ORTB200_F32;
  ORTB_THROW(NOT_IMPLEMENTED, "dtype not supported by the GPU kernels");
}

int ActCode(const std::string& a) {
  if (a == "none" || a.empty()) return ORTB200_ACT_NONE;
  if (a == "gelu") return ORTB200_ACT_GELU;
  if (a == "fastgelu") return ORTB200_ACT_FASTGELU;
  if (a == "relu") return ORTB200_ACT_RELU;
  if (a == "silu") return ORTB200_ACT_SILU;
  if (a == "quickgelu") return ORTB200_ACT_QUICKGELU;
  if (a == "swiglu") return ORTB200_ACT_SWIGLU;
  ORTB_THROW(INVALID_ARGUMENT, "unknown activation ", a);
}

bool HalfType(at::ScalarType t) { return t == at::kHalf || t == at::kBFloat16; }

}  // namespace

void CheckLaunch(int rc, const char* what) {
  if (rc != 0) ORTB_THROW(EP_FAIL, what, " rejected its arguments (code ", rc, ")");
}

// TunableOp for the GEMM: the first time a signature is seen (and tuning is enabled, and the stream is not being
// captured) every candidate launch configuration runs a few times with the L2 flushed in between; the fastest one is
// remembered in the session.  Candidates are the forced forms of the kernels' own heuristics: token-tile width and
// split-K cluster size for decode-shaped problems, tile family for large ones.
void ApplyTunedConfig(Ctx& ctx, ortb200_gemm_args* a, at::ScalarType out_type) {
  InferenceSession* s = ctx.session();
  std::ostringstream key;
  key << "Gemm_" << c10::toString(out_type) << "_in" << a->in_dtype << "_" << a->M << "_" << a->N << "_" << a->K << "_act" << a->act
      << (a->rms_eps > 0.f ? "_rms" : "") << (a->bias ? "_b" : "") << (a->residual ? "_r" : "");
  auto it = s->tuning_results.find(key.str());
  cudaStream_t stream = static_cast<cudaStream_t>(ctx.cuda_stream());
  if (it == s->tuning_results.end()) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &cap);
    if (!s->tunable_op_tuning_enable || cap != cudaStreamCaptureStatusNone) return;
    struct Cand { int splits, bn, rows; };
    std::vector<Cand> cands = {{0, 0, 0}};
    if (a->M <= 64 && a->in_dtype != ORTB200_F8E4M3) {
      for (int bn : {16, 32, 64}) {
        if (bn < a->M && bn != 64) continue;  // one token tile per weight tile: the weights stream once
        for (int splits : {1, 2, 4, 8}) cands.push_back({splits, bn, 0});
      }
    } else if (a->M > 128 && a->in_dtype == 0 && a->act != ORTB200_ACT_SWIGLU) {
      cands.push_back({0, 0, 128});
      cands.push_back({0, 0, 512});
    }
    static at::Tensor flush;  // larger than the L2: every timed launch starts cold, as in a model step
    if (!flush.defined() || flush.device() != ctx.device()) flush = at::empty({256LL << 20}, at::TensorOptions().dtype(at::kByte).device(ctx.device()));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const auto t_begin = std::chrono::steady_clock::now();
    InferenceSession::TunedGemm best;
    float best_us = 0.f;
    for (const Cand& c : cands) {
      ortb200_gemm_args t = *a;
      t.force_splits = c.splits;
      t.force_bn = c.bn;
      t.force_tile_rows = c.rows;
      if (ortb200_gemm(&t, stream) != 0) continue;  // a configuration the kernels do not offer for this shape
      float sum = 0.f;
      const int iters = 3;
      for (int i = 0; i < iters; ++i) {
        flush.zero_();
        cudaEventRecord(e0, stream);
        ortb200_gemm(&t, stream);
        cudaEventRecord(e1, stream);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        sum += ms;
      }
      const float us = sum / iters * 1e3f;
      if (best_us == 0.f || us < best_us) {
        best_us = us;
        best.force_splits = c.splits;
        best.force_bn = c.bn;
        best.force_tile_rows = c.rows;
      }
      const auto elapsed = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t_begin).count();
      if (elapsed > s->tunable_op_max_tuning_duration_ms) break;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    best.microseconds = best_us;
    it = s->tuning_results.emplace(key.str(), best).first;
    ORTB_VLOG(s->logger(), 1) << "tuned " << key.str() << ": splits " << best.force_splits << ", bn " << best.force_bn << ", tile rows "
                              << best.force_tile_rows << " (" << best_us << " us)";
  }
  a->force_splits = it->second.force_splits;
  a->force_bn = it->second.force_bn;
  a->force_tile_rows = it->second.force_tile_rows;
}

// out[M,N] = act(x[M,K] @ w_nk[N,K]^T + bias) + residual on the tcgen05 GEMM.
at::Tensor LaunchGemm(Ctx& ctx, const at::Tensor& x2d, const at::Tensor& w_nk, int64_t n_out, int64_t dual_offset,
                      const at::Tensor& bias, const at::Tensor& residual2d, int act, float alpha, bool fused_allreduce,
                      at::ScalarType out_type, float rms_eps, const at::Tensor& alpha_dev) {
  InferenceSession* s = ctx.session();
  const int64_t M = x2d.size(0), K = x2d.size(1);
  const bool fp8 = x2d.scalar_type() == at::kFloat8_e4m3fn;
  if (out_type == at::ScalarType::Undefined) out_type = x2d.scalar_type();
  at::Tensor out = at::empty({M, n_out}, x2d.options().dtype(out_type));
  if (M == 0) return out;
  const int64_t ws_bytes = ortb200_gemm_workspace_bytes(static_cast<int>(M), static_cast<int>(n_out), static_cast<int>(K), act);
  at::Tensor& ws = s->GemmWorkspace(ws_bytes);
  ortb200_gemm_args a{};
  a.x = x2d.data_ptr();
  a.w = w_nk.data_ptr();
  a.out = out.data_ptr();
  a.bias = bias.defined() ? bias.data_ptr() : nullptr;
  a.residual = residual2d.defined() ? residual2d.data_ptr() : nullptr;
  a.ldo = n_out;
  a.ldr = residual2d.defined() ? residual2d.stride(0) : 0;
  a.M = static_cast<int>(M);
  a.N = static_cast<int>(n_out);
  a.K = static_cast<int>(K);
  a.w_rows = static_cast<int>(w_nk.size(0));
  a.dual_offset = static_cast<int>(dual_offset);
  a.dtype = DtypeCode(out_type);
  a.in_dtype = fp8 ? ORTB200_F8E4M3 : 0;
  a.rms_eps = rms_eps;
  a.act = act;
  a.alpha = alpha;
  a.alpha_dev = alpha_dev.defined() ? alpha_dev.data_ptr<float>() : nullptr;
  a.workspace = ws.data_ptr();
  a.workspace_bytes = ws.numel();
  a.status = s->StatusWord().data_ptr<int>();
  a.use_pdl = s->config().Get("ortb200.pdl", "0") == "1" ? 1 : 0;
  a.world = 1;
  if (fused_allreduce) {
    a.world = s->world_size;
    a.rank = s->rank;
    for (int i = 0; i < s->world_size && i < 8; ++i) a.peers[i] = s->symm_peers[i];
    a.symm_bytes = s->symm_bytes;
    a.mc_ptr = s->NvlsPointer();  // prompt-sized problems reduce through the switch when the workspace is multicast-mapped
  }
  if (s->tunable_op_enable && !fused_allreduce) ApplyTunedConfig(ctx, &a, out_type);
  CheckLaunch(ortb200_gemm(&a, ctx.cuda_stream()), "ortb200_gemm");
  s->AddLaunches(fused_allreduce && M > 64 ? 2 : 1);
  return out;
}

// x / rms(x) row-wise (no gamma): the explicit form of the normalisation that decode-shaped GEMMs do in their epilogue.
at::Tensor RmsNormalizeRows(Ctx& ctx, const at::Tensor& x2d, const at::Tensor& unit_gamma, float eps) {
  at::Tensor out = at::empty_like(x2d);
  ortb200_norm_args a{};
  a.x = x2d.data_ptr();
  a.gamma = unit_gamma.data_ptr();
  a.out = out.data_ptr();
  a.rows = x2d.size(0);
  a.hidden = static_cast<int>(x2d.size(1));
  a.epsilon = eps;
  a.simplified = 1;
  a.dtype = DtypeCode(x2d.scalar_type());
  const int rc = ortb200_norm(&a, ctx.cuda_stream());
  if (rc != 0) {
    // shapes the norm kernel does not take: plain tensor math
    at::Tensor xf = x2d.to(at::kFloat);
    return (xf * at::rsqrt(xf.pow(2).mean(-1, true) + eps)).to(x2d.scalar_type());
  }
  ctx.session()->AddLaunches(1);
  return out;
}

// Runs a GEMM whose weights carry the gamma of a preceding RMS normalisation (rms_eps > 0).
at::Tensor LaunchNormedGemm(Ctx& ctx, const at::Tensor& x2d, const at::Tensor& w_nk, int64_t n_out, int64_t dual_offset,
                            const at::Tensor& bias, const at::Tensor& residual2d, int act, float alpha, float rms_eps,
                            const at::Tensor& unit_gamma) {
  if (rms_eps > 0.f && x2d.size(0) > 64) {
    at::Tensor xn = RmsNormalizeRows(ctx, x2d, unit_gamma, rms_eps);
    return LaunchGemm(ctx, xn, w_nk, n_out, dual_offset, bias, residual2d, act, alpha);
  }
  return LaunchGemm(ctx, x2d, w_nk, n_out, dual_offset, bias, residual2d, act, alpha, false, at::ScalarType::Undefined, rms_eps);
}

// MatMulNBits weights -> the tile-blob array of the in-kernel expansion (layout: ortb200_gemm_args, in_dtype Q4).
// B uint8 [N, n_blocks, block / 2] (4-bit, low nibble = even k), scales [N, n_blocks], zp_bytes uint8 [N, n_blocks]
// (one byte per block) or undefined for the implicit 8.  All on the GPU.
at::Tensor NbitsBuildBlobs(const at::Tensor& B, const at::Tensor& scales, const at::Tensor& zp_bytes, int64_t N, int64_t K,
                           int64_t block) {
  ORTB_ENFORCE_ARG(B.is_cuda() && K % 64 == 0 && block >= 32 && (block & (block - 1)) == 0, "NbitsBuildBlobs: unsupported layout");
  const int64_t num_kb = K / 64, Np = (N + 127) / 128 * 128, nb = (K + block - 1) / block;
  at::Tensor src = B.contiguous().reshape({N, K / 2});
  at::Tensor nib = at::empty_like(src);
  CheckLaunch(ortb200_nbits_prepack(src.data_ptr(), nib.data_ptr(), N * (K / 2), at::cuda::getCurrentCUDAStream().stream()),
              "ortb200_nbits_prepack");
  auto pad_rows = [&](const at::Tensor& t) {
    if (Np == N) return t;
    std::vector<int64_t> shape = t.sizes().vec();
    shape[0] = Np - N;
    return at::cat({t, at::zeros(shape, t.options())}, 0);
  };
  // nibbles: [Np, num_kb, 32] -> [tiles, num_kb, 128, 32]
  at::Tensor w = pad_rows(nib).reshape({Np / 128, 128, num_kb, 32}).permute({0, 2, 1, 3}).reshape({Np / 128, num_kb, 4096});
  // scales and zero points at 32-element granularity (two per k-block), whatever the block size
  const int64_t rep = block / 32;
  at::Tensor s32 = scales.reshape({N, nb}).repeat_interleave(rep, 1).narrow(1, 0, K / 32).contiguous();
  at::Tensor sb = pad_rows(s32).reshape({Np / 128, 128, num_kb, 2}).permute({0, 2, 1, 3}).contiguous().view(at::kByte).reshape({Np / 128, num_kb, 512});
  at::Tensor z32 = zp_bytes.defined() ? zp_bytes.reshape({N, nb}).repeat_interleave(rep, 1).narrow(1, 0, K / 32).contiguous()
                                      : at::full({N, K / 32}, 8, B.options());
  at::Tensor zb = pad_rows(z32).reshape({Np / 128, 128, num_kb, 2}).permute({0, 2, 1, 3}).reshape({Np / 128, num_kb, 256});
  return at::cat({w, sb, zb}, 2).contiguous();
}

// out[M, N] = x[M, K] @ dequant(blobs)[N, K]^T + bias with the 4-bit weights expanded inside the kernel (M <= 64).
at::Tensor Fp8WeightBuildBlobs(const at::Tensor& B, const at::Tensor& scales, int64_t block) {
  const int64_t N = B.size(0), K = B.size(1);
  ORTB_ENFORCE_ARG(K % 64 == 0 && block % 64 == 0 && block > 0, "fp8 weight blobs need K and block_size to be multiples of 64");
  const int64_t tiles = (N + 127) / 128, kbs = K / 64, rows = tiles * 128;
  at::Tensor bytes = B.contiguous().view(at::kByte);
  at::Tensor sc = scales.to(at::kFloat).repeat_interleave(block / 64, 1).narrow(1, 0, kbs).contiguous();   // [N, K / 64]
  if (rows != N) {  // rows beyond N: zero weights, zero scales
    bytes = at::cat({bytes, at::zeros({rows - N, K}, bytes.options())}, 0);
    sc = at::cat({sc, at::zeros({rows - N, kbs}, sc.options())}, 0);
  }
  at::Tensor w = bytes.reshape({tiles, 128, kbs, 64}).permute({0, 2, 1, 3}).reshape({tiles, kbs, 128 * 64});
  at::Tensor s4 = sc.reshape({tiles, 128, kbs}).permute({0, 2, 1}).contiguous().view(at::kByte).reshape({tiles, kbs, 128 * 4});
  return at::cat({w, s4}, 2).contiguous();   // [tiles, K / 64, 8704]
}

at::Tensor LaunchGemmQ4(Ctx& ctx, const at::Tensor& x2d, const at::Tensor& blobs, int64_t n_out, const at::Tensor& bias,
                        const at::Tensor& residual2d, bool fused_allreduce, int in_dtype) {
  InferenceSession* s = ctx.session();
  const int64_t M = x2d.size(0), K = x2d.size(1);
  at::Tensor out = at::empty({M, n_out}, x2d.options());
  if (M == 0) return out;
  ortb200_gemm_args a{};
  a.x = x2d.data_ptr();
  a.w = blobs.data_ptr();
  a.out = out.data_ptr();
  a.bias = bias.defined() ? bias.data_ptr() : nullptr;
  a.residual = residual2d.defined() ? residual2d.data_ptr() : nullptr;
  a.ldo = n_out;
  a.ldr = residual2d.defined() ? residual2d.stride(0) : 0;
  a.M = static_cast<int>(M); a.N = static_cast<int>(n_out); a.K = static_cast<int>(K);
  a.w_rows = static_cast<int>(blobs.size(0) * 128);
  a.dtype = DtypeCode(x2d.scalar_type());
  a.in_dtype = in_dtype;
  a.act = ORTB200_ACT_NONE;
  a.alpha = 1.f;
  a.status = s->StatusWord().data_ptr<int>();
  a.use_pdl = s->config().Get("ortb200.pdl", "0") == "1" ? 1 : 0;
  a.world = 1;
  if (fused_allreduce) {
    a.world = s->world_size;
    a.rank = s->rank;
    for (int i = 0; i < s->world_size && i < 8; ++i) a.peers[i] = s->symm_peers[i];
    a.symm_bytes = s->symm_bytes;
  }
  CheckLaunch(ortb200_gemm(&a, ctx.cuda_stream()), "ortb200_gemm(q4)");
  s->AddLaunches(1);
  return out;
}

bool CanFuseAllReduce(OpKernelContext& ctx, int64_t M, int64_t N) {
  InferenceSession* s = ctx.session();
  if (!s || s->world_size <= 1 || s->world_size > 8) return false;
  if (static_cast<int>(s->symm_peers.size()) != s->world_size) return false;
  if (s->config().Get("ortb200.fused_allreduce", "1") != "1") return false;
  if (M > 64) {
    // prompt-sized: the CTA-pair GEMM pushes its product into the all-reduce scatter areas, a reduction kernel follows
    return N % 8 == 0 && M * N * 2 <= ortb200_symm_collective_max_bytes(ORTB200_COLL_ALLREDUCE, s->world_size, s->symm_bytes);
  }
  const int64_t slot = (s->symm_bytes / 2 - 262144) / (2LL * s->world_size * 8);
  return slot >= M * N && (N + 127) / 128 * 8 <= 4096;
}

namespace {

at::Tensor Flatten2D(const at::Tensor& x) { return x.reshape({-1, x.size(-1)}).contiguous(); }

std::vector<int64_t> OutShape(const at::Tensor& x, int64_t n) {
  std::vector<int64_t> s = x.sizes().vec();
  s.back() = n;
  return s;
}

// MatMul / FusedGemm / Gemm with a constant fp16/bf16 weight.
class GemmKernel final : public OpKernel {
 public:
  explicit GemmKernel(const OpKernelInfo& info) : OpKernel(info) {
    const Node& n = info.node;
    const at::Tensor* w = info.constant_input(1);
    ORTB_ENFORCE(w != nullptr, "GEMM kernel needs a constant weight");
    bool w_is_nk = false;
    if (n.op_type == "Gemm") {
      w_is_nk = n.attr_i("transB", 0) != 0;
      alpha_ = n.attr_f("alpha", 1.f);
      bias_idx_ = 2;
    } else if (n.op_type == "FusedMatMul") {
      w_is_nk = n.attr_i("transB", 0) != 0;
      alpha_ = n.attr_f("alpha", 1.f);
    } else if (n.op_type == "FusedGemm") {
      bias_idx_ = 2;
      residual_idx_ = 3;
      act_ = ActCode(n.attr_s("activation", "none"));
      all_reduce_ = n.attr_i("all_reduce", 0) != 0;
      rms_eps_ = n.attr_f("rms_eps", 0.f);
    }
    w_nk_ = w_is_nk ? w->contiguous() : w->t().contiguous();  // pre-pack: [N, K], K contiguous
    N_ = w_nk_.size(0);
    if (rms_eps_ > 0.f) {
      // the RMS norm in front of this GEMM was folded in: its gamma scales the K axis of the weights
      const at::Tensor* gamma = info.constant_input(4);
      ORTB_ENFORCE(gamma != nullptr && gamma->numel() == w_nk_.size(1), "FusedGemm with rms_eps needs a constant gamma of length K");
      w_nk_ = (w_nk_.to(at::kFloat) * gamma->to(at::kFloat).reshape({1, -1})).to(w_nk_.scalar_type()).contiguous();
      unit_gamma_ = at::ones({w_nk_.size(1)}, w_nk_.options());
    }
    if (info.session != nullptr && w_nk_.defined() && w_nk_.is_cuda())
      info.session->RegisterWeightHint(info.node.name, w_nk_.data_ptr(), static_cast<int64_t>(w_nk_.numel()) * w_nk_.element_size());
  }
  std::vector<int> PrepackedInputs() const override { return {1}; }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor x2 = Flatten2D(x);
    at::Tensor bias = bias_idx_ >= 0 && ctx.HasInput(bias_idx_) ? ctx.Input(bias_idx_) : at::Tensor();
    at::Tensor res = residual_idx_ >= 0 && ctx.HasInput(residual_idx_) ? ctx.Input(residual_idx_) : at::Tensor();
    at::Tensor late_res;  // a residual the kernels cannot index row by row: added afterwards with broadcasting
    if (res.defined()) {
      // The epilogues read residual[m * ld + n] for every m < M, so the operand must be exactly the output's shape
      // and type.  Anything else (a [B, 1, N] or [N] term that the original Add would have broadcast, or a larger
      // operand that broadcasts the product up) takes the plain Add after the GEMM.
      if (res.sizes().vec() == OutShape(x, N_) && res.scalar_type() == x.scalar_type()) {
        res = Flatten2D(res);
      } else {
        late_res = res;
        res = at::Tensor();
      }
    }
    if (late_res.defined()) {
      at::Tensor y;
      if (all_reduce_ && ctx.session()->world_size > 1) {
        y = LaunchGemm(ctx, x2, w_nk_, N_, 0, bias, at::Tensor(), act_, alpha_);
        y = GemmAllReduce(ctx, y, at::Tensor());
      } else {
        y = LaunchNormedGemm(ctx, x2, w_nk_, N_, 0, bias, at::Tensor(), act_, alpha_, rms_eps_, unit_gamma_);
      }
      ctx.SetOutput(0, at::add(y.reshape(OutShape(x, N_)), late_res));
      return;
    }
    if (all_reduce_ && ctx.session()->world_size > 1) {
      if (act_ == ORTB200_ACT_NONE && CanFuseAllReduce(ctx, x2.size(0), N_)) {
        // one kernel: tcgen05 GEMM, partial tiles pushed to every peer over NVLink, summed in rank order, + residual
        at::Tensor y = LaunchGemm(ctx, x2, w_nk_, N_, 0, bias, res, act_, alpha_, /*fused_allreduce=*/true);
        ctx.SetOutput(0, y.reshape(OutShape(x, N_)));
        return;
      }
      // baseline: partial product, library all-reduce over the process group, then the residual
      at::Tensor y = LaunchGemm(ctx, x2, w_nk_, N_, 0, bias, at::Tensor(), act_, alpha_);
      y = GemmAllReduce(ctx, y, res);
      ctx.SetOutput(0, y.reshape(OutShape(x, N_)));
      return;
    }
    at::Tensor y = LaunchNormedGemm(ctx, x2, w_nk_, N_, 0, bias, res, act_, alpha_, rms_eps_, unit_gamma_);
    ctx.SetOutput(0, y.reshape(OutShape(x, N_)));
  }

 private:
  at::Tensor w_nk_, unit_gamma_;
  float rms_eps_ = 0.f;
  int64_t N_ = 0;
  int bias_idx_ = -1, residual_idx_ = -1;
  int act_ = ORTB200_ACT_NONE;
  float alpha_ = 1.f;
  bool all_reduce_ = false;
};

bool GemmSupports(const Node& n, const Graph& g) {
  if (n.inputs.size() < 2) return false;
  const at::Tensor* w = g.GetConstant(n.inputs[1]);
  if (!w || w->dim() != 2 || !HalfType(w->scalar_type())) return false;
  if (g.GetConstant(n.inputs[0])) return false;
  const bool nk = (n.op_type == "Gemm" || n.op_type == "FusedMatMul") && n.attr_i("transB", 0) != 0;
  const int64_t K = nk ? w->size(1) : w->size(0);
  if (K % 8 != 0) return false;
  if (n.op_type == "Gemm" && (n.attr_i("transA", 0) != 0 || n.attr_f("beta", 1.f) != 1.f)) return false;
  if (n.op_type == "Gemm" && n.has_input(2)) {
    const at::Tensor* c = g.GetConstant(n.inputs[2]);
    if (!c || c->dim() != 1) return false;
  }
  if (n.op_type == "FusedMatMul" && (n.attr_i("transA", 0) || n.attr_i("transBatchA", 0) || n.attr_i("transBatchB", 0))) return false;
  return true;
}

class GemmSwiGLUKernel final : public OpKernel {
 public:
  explicit GemmSwiGLUKernel(const OpKernelInfo& info) : OpKernel(info) {
    const at::Tensor* wg = info.constant_input(1);
    const at::Tensor* wu = info.constant_input(2);
    ORTB_ENFORCE(wg && wu, "GemmSwiGLU needs constant weights");
    I_ = wg->size(1);
    w_ = at::cat({wg->t(), wu->t()}, 0).contiguous();  // [2I, K]: gate rows then up rows
    rms_eps_ = info.node.attr_f("rms_eps", 0.f);
    if (rms_eps_ > 0.f) {
      const at::Tensor* gamma = info.constant_input(3);
      ORTB_ENFORCE(gamma != nullptr && gamma->numel() == w_.size(1), "GemmSwiGLU with rms_eps needs a constant gamma of length K");
      w_ = (w_.to(at::kFloat) * gamma->to(at::kFloat).reshape({1, -1})).to(w_.scalar_type()).contiguous();
      unit_gamma_ = at::ones({w_.size(1)}, w_.options());
    }
  }
  std::vector<int> PrepackedInputs() const override { return {1, 2}; }
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    at::Tensor x2 = Flatten2D(x);
    if (x2.size(0) > 128 && I_ % 8 == 0) {
      // Large M: the two-accumulator kernel is limited to 128-token tiles (tensor memory), which costs more than it
      // saves; one plain GEMM over the stacked gate | up rows at 256-token tiles plus a streaming SwiGLU is faster.
      at::Tensor gu = LaunchNormedGemm(ctx, x2, w_, 2 * I_, 0, at::Tensor(), at::Tensor(), ORTB200_ACT_NONE, 1.f, rms_eps_, unit_gamma_);
      at::Tensor y = at::empty({x2.size(0), I_}, x2.options());
      CheckLaunch(ortb200_swiglu(gu.data_ptr(), y.data_ptr(), x2.size(0), static_cast<int>(I_), DtypeCode(x2.scalar_type()), ctx.cuda_stream()),
                  "ortb200_swiglu");
      ctx.session()->AddLaunches(1);
      ctx.SetOutput(0, y.reshape(OutShape(x, I_)));
      return;
    }
    at::Tensor y = LaunchNormedGemm(ctx, x2, w_, I_, I_, at::Tensor(), at::Tensor(), ORTB200_ACT_SWIGLU, 1.f, rms_eps_, unit_gamma_);
    ctx.SetOutput(0, y.reshape(OutShape(x, I_)));
  }

 private:
  at::Tensor w_, unit_gamma_;
  float rms_eps_ = 0.f;
  int64_t I_ = 0;
};

// com.ortb200.SwiGLU: [..., 2 I] -> silu(x[..., :I]) * x[..., I:], one streaming kernel (behind the stacked gate | up
// projection of 4-bit models).
class SwiGLUKernel final : public OpKernel {
 public:
  explicit SwiGLUKernel(const OpKernelInfo& info) : OpKernel(info) {}
  void Compute(Ctx& ctx) const override {
    const at::Tensor& x = ctx.RequiredInput(0);
    const int64_t I = x.size(-1) / 2;
    at::Tensor x2 = x.reshape({-1, 2 * I}).contiguous();
    std::vector<int64_t> shape = x.sizes().vec();
    shape.back() = I;
    if (!HalfType(x.scalar_type()) || I % 8 != 0 || x2.size(0) == 0) {
      ctx.SetOutput(0, (at::silu(x2.narrow(1, 0, I)) * x2.narrow(1, I, I)).reshape(shape));
      return;
    }
    at::Tensor y = at::empty({x2.size(0), I}, x.options());
    CheckLaunch(ortb200_swiglu(x2.data_ptr(), y.data_ptr(), x2.size(0), static_cast<int>(I), DtypeCode(x.scalar_type()), ctx.cuda_stream()),
                "ortb200_swiglu");
    ctx.session()->AddLaunches(1);
    ctx.SetOutput(0, y.reshape(shape));
  }
};

template <typename K>
void RegisterClass(KernelRegistry& r, const std::string& domain, const std::string& op,
                   std::function<bool(const Node&, const Graph&)> supports = nullptr, std::vector<int> host = {}) {
  KernelDef d;
  d.domain = domain;
  d.op_type = op;
  d.supports = std::move(supports);
  d.host_inputs = std::move(host);
  d.factory = [](const OpKernelInfo& info) { return std::make_unique<K>(info); };
  r.Register(std::move(d));
}

}  // namespace

void RegisterCudaKernels(KernelRegistry& r) {
  RegisterClass<GemmKernel>(r, "", "MatMul", GemmSupports);
  RegisterClass<GemmKernel>(r, "", "Gemm", GemmSupports);
  RegisterClass<GemmKernel>(r, MS, "FusedMatMul", GemmSupports);
  RegisterClass<GemmKernel>(r, kFusedDomain, "FusedGemm", GemmSupports);
  RegisterClass<GemmSwiGLUKernel>(r, kFusedDomain, "GemmSwiGLU");
  RegisterClass<SwiGLUKernel>(r, kFusedDomain, "SwiGLU");
  RegisterMoreCudaKernels(r);
  RegisterCudaKernels3(r);
}

}  // namespace ortb
