// Flash-attention forward for sm_100a on tcgen05: S = Q K^T and O_tile = P V run
// on the 5th-generation tensor cores with both accumulators in tensor memory.
//
// One CTA owns 128 query rows of one (batch, head).  Per 128-key tile:
//   MMA 1  S[128 q, 128 keys]   = Q[128, H] . K[128, H]^T      (both K-major)
//   softmax threads (one per query row) read their row of S from TMEM, apply the
//   mask and the online-softmax update, and write P as bf16/fp16 into shared
//   memory in the 128-byte-swizzled K-major layout the MMA expects
//   MMA 2  O_tile[128 q, H]     = P[128, 128 keys] . V[128 keys, H]   (V is MN-major)
//   the same threads fold O_tile into their fp32 register accumulator.
// K/V tiles are double-buffered by a TMA producer warp; MMA 1 of the next tile is
// issued as soon as P is published, so it overlaps the accumulator update.
//
// Replaces, for prompt processing and encoder self-attention, the FlashAttention-2
// (mma.sync) and CUTLASS FMHA kernels the reference dispatches to
// (onnxruntime/contrib_ops/cuda/bert/flash_attention/flash_fwd_kernel.h,
// bert/cutlass_fmha/kernel_forward.h) and its cuDNN SDPA path
// (bert/cudnn_fmha/cudnn_flash_attention.cc:105).
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"

namespace ortb200 {

constexpr int kQT = 128;   // query rows per CTA
constexpr int kKT = 128;   // keys per tile
constexpr int kAttnThreads = 192;

struct AttnParams {
  const int* seqlens_k;
  const int* key_mask;
  const void* head_sink;
  void* out;
  int B, S, N, Nk, kv_len;
  long long o_strides[3];
  int first_prompt, causal, window;
  float scale_log2, softcap, scale;
  int bf16;
  int* status;
};

template <int HD>
struct AttnSmem {
  static constexpr int kBoxBytes = 128 * 128;          // [128 rows][64 elems] of 16-bit data
  static constexpr int kBoxes = HD / 64;                // boxes per Q / K / V tile
  static constexpr int kQBytes = kBoxBytes * kBoxes;
  static constexpr int kKVBytes = kBoxBytes * kBoxes;   // each of K and V
  static constexpr int kPBytes = kBoxBytes * 2;         // P [128 q][128 keys]
  static constexpr int kStageBytes = 2 * kKVBytes;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kQBytes;
  static constexpr int kOffP = kOffKV + 2 * kStageBytes;
  static constexpr int kOffBar = kOffP + kPBytes;
  static constexpr int kTotal = kOffBar + 128 + 1024;
  static constexpr int kTmemCols = 512;                // two score buffers (2 x 128 columns) + O (HD columns)
};

// Bit j of the result = key (key0 + j) of batch b may be attended to.  Called by all 32 lanes of a warp.
__device__ __forceinline__ unsigned key_keep_bits(const int* key_mask, int b, int kv_len, int key0, int lane) {
  if (key_mask == nullptr) return 0xffffffffu;
  const int key = key0 + lane;
  const bool keep = key < kv_len && key_mask[static_cast<long long>(b) * kv_len + key] != 0;
  return __ballot_sync(0xffffffffu, keep);
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// barrier indices
enum { BAR_Q = 0, BAR_KV_FULL0, BAR_KV_FULL1, BAR_KV_EMPTY0, BAR_KV_EMPTY1, BAR_S_FULL0, BAR_S_FULL1, BAR_P_READY, BAR_O_FULL, BAR_COUNT };

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using L = AttnSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kQT;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.N / p.Nk);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int i = 0; i < BAR_COUNT; ++i) mbar_init(&bars[i], i == BAR_P_READY ? 128 : 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;          // S: two buffers, columns [0, 128) and [128, 256)
  const uint32_t tmem_o = tmem_base + 256;    // O: columns [256, 256 + HD), accumulated over all key tiles

  pdl_wait_prior_grids();
  const int total = p.seqlens_k ? p.seqlens_k[b] + 1 : p.kv_len;
  const int past = p.first_prompt ? 0 : total - p.S;
  // key range needed by this query tile
  int kv_end = total;
  if (p.causal) kv_end = min(kv_end, past + q0 + kQT);
  kv_end = min(kv_end, p.kv_len);
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, past + q0 - p.window + 1) / kKT * kKT;
  const int n_tiles = kv_end > kv_begin ? (kv_end - kv_begin + kKT - 1) / kKT : 0;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(&bars[BAR_Q], L::kQBytes);
      for (int bx = 0; bx < L::kBoxes; ++bx)
        tma_load_4d(smem + L::kOffQ + bx * L::kBoxBytes, &tm_q, &bars[BAR_Q], bx * 64, q0, head, b);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t & 1;
        if (t >= 2) {
          if (!mbar_wait(&bars[BAR_KV_EMPTY0 + s], ((t >> 1) - 1) & 1)) {
            if (p.status) atomicExch(p.status, kStatusTimeoutProducer);
            break;
          }
        }
        uint8_t* st = smem + L::kOffKV + s * L::kStageBytes;
        mbar_expect_tx(&bars[BAR_KV_FULL0 + s], L::kStageBytes);
        const int key0 = kv_begin + t * kKT;
        for (int bx = 0; bx < L::kBoxes; ++bx) {
          tma_load_4d(st + bx * L::kBoxBytes, &tm_k, &bars[BAR_KV_FULL0 + s], bx * 64, key0, kvh, b);
          tma_load_4d(st + L::kKVBytes + bx * L::kBoxBytes, &tm_v, &bars[BAR_KV_FULL0 + s], bx * 64, key0, kvh, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = umma_idesc_f16(p.bf16 != 0, kQT, kKT);
      const uint32_t idesc_o = umma_idesc_f16_bmn(p.bf16 != 0, kQT, HD);
      const uint32_t q_addr = smem_u32(smem + L::kOffQ);
      const uint32_t p_addr = smem_u32(smem + L::kOffP);
      bool ok = mbar_wait(&bars[BAR_Q], 0);
      auto issue_s = [&](int t) {
        const int s = t & 1;
        const uint32_t k_addr = smem_u32(smem + L::kOffKV + s * L::kStageBytes);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * L::kBoxBytes + (kk % 4) * 32;
          umma_f16(tmem_s + s * kKT, umma_desc_sw128(q_addr + off), umma_desc_sw128(k_addr + off), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars[BAR_S_FULL0 + s]);
      };
      if (ok && !mbar_wait(&bars[BAR_KV_FULL0], 0)) ok = false;
      if (ok) {
        tcgen05_fence_after();
        issue_s(0);
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int s = t & 1;
        if (t + 1 < n_tiles) {
          // S of the next tile goes to the other score buffer while the softmax threads work on this one; that
          // buffer was consumed before P of tile t - 1 was published, which this thread has waited for
          if (!mbar_wait(&bars[BAR_KV_FULL0 + (s ^ 1)], ((t + 1) >> 1) & 1)) { ok = false; break; }
          tcgen05_fence_after();
          issue_s(t + 1);
        }
        // P of tile t published (O rescaled if the row maxima moved)
        if (!mbar_wait(&bars[BAR_P_READY], t & 1)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t v_addr = smem_u32(smem + L::kOffKV + s * L::kStageBytes + L::kKVBytes);
#pragma unroll
        for (int kk = 0; kk < kKT / 16; ++kk) {
          const uint64_t pdesc = umma_desc_sw128(p_addr + (kk / 4) * L::kBoxBytes + (kk % 4) * 32);
          const uint64_t vdesc = umma_desc_mn_sw128(v_addr + kk * 2048, L::kBoxBytes, 1024);
          umma_f16(tmem_o, pdesc, vdesc, idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars[BAR_O_FULL]);
        umma_commit(&bars[BAR_KV_EMPTY0 + s]);
      }
      if (!ok && p.status) atomicExch(p.status, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------ softmax (one thread per query row); O accumulates in TMEM
    const int qw = warp & 3;
    const int r = qw * 32 + lane;
    const int s_idx = q0 + r;
    const int pos = past + s_idx;
    const uint32_t lane_addr = static_cast<uint32_t>(qw * 32) << 16;
    // The reference maximum of a row is raised only when a tile exceeds it by 2^8 (probabilities stay below 256),
    // so the accumulator in tensor memory is rescaled a few times per row instead of once per tile.
    constexpr float kRaise = 8.f;
    float m = -INFINITY, l = 0.f;
    uint8_t* p_smem = smem + L::kOffP;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      if (ok && !mbar_wait(&bars[BAR_S_FULL0 + (t & 1)], (t >> 1) & 1)) ok = false;
      tcgen05_fence_after();
      const int key0 = kv_begin + t * kKT;
      // Interior tiles (every key visible to every row of this query tile) skip the per-element mask logic.
      const bool need_mask = (key0 + kKT > total) || (key0 + kKT > p.kv_len) || (p.key_mask != nullptr) || (p.window > 0) ||
                             (p.causal && key0 + kKT - 1 > past + q0) || (p.softcap > 0.f);
      // The whole row of scores is fetched with back-to-back tensor-memory loads and one wait, then turned into
      // base-2 logits in place (-inf where masked).
      float sv[kKT];
      const uint32_t s_addr = tmem_s + (t & 1) * kKT + lane_addr;
#pragma unroll
      for (int g4 = 0; g4 < kKT / 32; ++g4) tmem_ld_x32(s_addr + g4 * 32, sv + g4 * 32);
      tmem_ld_wait();
      // Scores stay unscaled in registers: the scale is folded into the exponent's multiply-add.  Plain length /
      // causal masking is one compare and select per element against a per-row limit; key masks, sliding windows
      // and soft-capping take the general path, which leaves final base-2 logits (scale 1).
      float fs = p.scale_log2;
      if (need_mask) {
        if (p.softcap > 0.f) {   // soft-capped logits are final base-2 logits: the exponent then uses scale 1
          fs = 1.f;
#pragma unroll
          for (int j = 0; j < kKT; ++j) sv[j] = p.softcap * tanhf(sv[j] * p.scale / p.softcap) * 1.4426950408889634f;
        }
        // visible keys of this row within the tile: [lo, hi) and the tile's key-mask bits (one ballot per 32 keys)
        int hi = min(total, p.kv_len);
        if (p.causal) hi = min(hi, pos + 1);
        hi -= key0;
        const int lo = p.window > 0 ? pos - p.window + 1 - key0 : -kKT;
        if (p.key_mask == nullptr) {
#pragma unroll
          for (int j = 0; j < kKT; ++j) sv[j] = (j < hi && j >= lo) ? sv[j] : -INFINITY;
        } else {
#pragma unroll
          for (int g4 = 0; g4 < kKT / 32; ++g4) {
            const unsigned keep = key_keep_bits(p.key_mask, b, p.kv_len, key0 + g4 * 32, lane);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int jj = g4 * 32 + j;
              sv[jj] = (jj < hi && jj >= lo && ((keep >> j) & 1u)) ? sv[jj] : -INFINITY;
            }
          }
        }
      }
      float m_raw = -INFINITY;
#pragma unroll
      for (int j = 0; j < kKT; j += 2) m_raw = fmax3(m_raw, sv[j], sv[j + 1]);
      const float m_tile = m_raw * fs;   // fs > 0: -inf stays -inf
      // the previous PV product reads P and writes O: it must have finished before either is touched
      if (t > 0 && ok && !mbar_wait(&bars[BAR_O_FULL], (t - 1) & 1)) ok = false;
      tcgen05_fence_after();
      const bool raise = m_tile > m + kRaise;   // also the first finite maximum of a row (m = -inf)
      if (__any_sync(0xffffffffu, raise)) {
        // tensor-memory loads and stores are warp-wide: every lane takes part, rows that keep their maximum scale by 1
        const float corr = raise ? (m == -INFINITY ? 0.f : exp2f(m - m_tile)) : 1.f;
        if (t > 0) {
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            float v[32];
            tmem_ld_x32(tmem_o + lane_addr + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= corr;
            tmem_st_x32(tmem_o + lane_addr + c, v);
          }
          tmem_st_wait();
        }
        l *= corr;
        if (raise) m = m_tile;
      }
      // masked scores are -inf and give 0; a row with no visible key so far (m = -inf) uses 0 as its reference
      const float neg_m = m == -INFINITY ? 0.f : -m;
      float row_sum = 0.f, row_sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < kKT; c += 32) {
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = ex2_approx(fmaf(sv[c + j], fs, neg_m));
          const float p1 = ex2_approx(fmaf(sv[c + j + 1], fs, neg_m));
          row_sum += p0;
          row_sum1 += p1;
          if (p.bf16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            packed[j / 2] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __half2 h = __floats2half2_rn(p0, p1);
            packed[j / 2] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        // 32 keys = 4 chunks of 16 bytes; column c lives in box c / 64
        const int box = c / 64;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = ((c % 64) * 2) / 16 + ch;
          uint8_t* dst = p_smem + box * L::kBoxBytes + r * 128 + ((chunk ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
        }
      }
      l += row_sum + row_sum1;
      // make the generic-proxy writes of P visible to the tensor core, then publish
      fence_proxy_async();
      tcgen05_fence_before();
      mbar_arrive(&bars[BAR_P_READY]);
    }
    if (n_tiles > 0 && ok && !mbar_wait(&bars[BAR_O_FULL], (n_tiles - 1) & 1)) ok = false;
    tcgen05_fence_after();
    if (!ok && p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
    pdl_launch_dependents();
    float denom = l;
    float rescale = 1.f;
    if (p.head_sink) {
      const float sink = (p.bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.head_sink)[head])
                                 : __half2float(static_cast<const __half*>(p.head_sink)[head])) * 1.4426950408889634f;
      const float mm = fmaxf(m, sink);
      rescale = m == -INFINITY ? 0.f : exp2f(m - mm);
      denom = l * rescale + exp2f(sink - mm);
    }
    const float inv = (denom > 0.f && n_tiles > 0) ? rescale / denom : 0.f;
    uint8_t* orow = static_cast<uint8_t*>(p.out) + 2 * (b * p.o_strides[0] + s_idx * p.o_strides[1] + head * p.o_strides[2]);
#pragma unroll 1
    for (int c0 = 0; c0 < HD; c0 += 32) {
      float v[32];
      if (n_tiles > 0) {   // uniform over the CTA
        tmem_ld_x32(tmem_o + lane_addr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
      }
      if (ok && s_idx < p.S) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            if (p.bf16) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[c + j] * inv, v[c + j + 1] * inv);
              w[j / 2] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              __half2 h = __floats2half2_rn(v[c + j] * inv, v[c + j + 1] * inv);
              w[j / 2] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          *reinterpret_cast<uint4*>(orow + (c0 + c) * 2) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

template <int HD>
static int launch_attn(const ortb200_attn_prefill_args* a, cudaStream_t stream) {
  using L = AttnSmem<HD>;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tq, tk, tv;
  {
    const int64_t dims[4] = {HD, a->S, a->N, a->B};
    const int64_t strides[3] = {a->q_strides[1] * 2, a->q_strides[2] * 2, a->q_strides[0] * 2};
    if (make_tensor_map_4d(&tq, a->q, dt, 2, dims, strides, 64, kQT) != 0) return -6;
  }
  {
    const int64_t dims[4] = {HD, a->kv_len, a->Nk, a->B};
    const int64_t strides[3] = {a->kv_strides[2] * 2, a->kv_strides[1] * 2, a->kv_strides[0] * 2};
    if (make_tensor_map_4d(&tk, a->k, dt, 2, dims, strides, 64, kKT) != 0) return -6;
    if (make_tensor_map_4d(&tv, a->v, dt, 2, dims, strides, 64, kKT) != 0) return -6;
  }
  AttnParams p;
  p.seqlens_k = a->seqlens_k;
  p.key_mask = a->key_mask;
  p.head_sink = a->head_sink;
  p.out = a->out;
  p.B = a->B; p.S = a->S; p.N = a->N; p.Nk = a->Nk; p.kv_len = a->kv_len;
  for (int i = 0; i < 3; ++i) p.o_strides[i] = a->o_strides[i];
  p.first_prompt = a->first_prompt; p.causal = a->causal; p.window = a->window;
  p.scale = a->scale != 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(HD));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.softcap = a->softcap;
  p.bf16 = a->dtype == ORTB200_BF16 ? 1 : 0;
  p.status = a->status;
  auto kern = attn_prefill_kernel<HD>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return -10;
    attr_set = true;
  }
  dim3 grid((a->S + kQT - 1) / kQT, a->N, a->B);
  kern<<<grid, kAttnThreads, L::kTotal, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ortb200

using namespace ortb200;

extern "C" int ortb200_attn_prefill(const ortb200_attn_prefill_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->q || !a->k || !a->v || !a->out) return -1;
  if (a->B <= 0 || a->S <= 0 || a->N <= 0 || a->Nk <= 0 || a->N % a->Nk != 0 || a->kv_len <= 0) return -1;
  if (a->H != 64 && a->H != 128) return -2;
  if (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16) return -4;
  for (int i = 0; i < 3; ++i)
    if (a->q_strides[i] % 8 || a->o_strides[i] % 8 || a->kv_strides[i] % 8) return -3;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->out)) & 15)
    return -3;
  return a->H == 128 ? launch_attn<128>(a, stream) : launch_attn<64>(a, stream);
}
