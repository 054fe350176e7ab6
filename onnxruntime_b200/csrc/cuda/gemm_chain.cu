// A chain of decode-shaped GEMMs (M <= 16 tokens) as ONE persistent kernel for sm_100a.
//
//   stage s:  y_s[M, N_s] = act_s( (x_s[M, K_s] * W_s[N_s, K_s]^T) / rms(x_s) + bias_s ) + residual_s,   x_{s+1} = y_s
//
// A decoder layer between two attention steps is such a chain: output projection (+ residual), gate / up projection
// with SwiGLU (RMS norm folded in), down projection (+ residual), and the next layer's QKV projection (RMS norm folded
// in).  Run as four launches, every GEMM pays its own ramp-up and drain (the weight stream stops at each kernel
// boundary); here one grid of one CTA per SM walks all stages and the weight stream never stops:
//
//  * Work of a stage is the list of (128-row weight tile, 64-wide k-block) items, tile-major; CTA c owns the contiguous
//    slice [c T / G, (c + 1) T / G) of it ("stream-K"), so every CTA moves the same number of bytes in every stage.
//  * Warp 0 streams weight tiles through a ring of shared-memory slots with TMA.  Weights depend on nothing, so the
//    ring runs ahead across stage boundaries; beyond the ring it asks the L2 for the tiles it will need next.
//  * Warp 2 copies the activation k-blocks (a few KiB, written by other CTAs in the previous stage) into a second ring
//    once the previous stage has completed; warp 1 issues tcgen05.mma into one of two TMEM accumulators; warps 3-6
//    drain accumulators.
//  * A slice boundary inside a tile leaves a partial tile: it goes to a per-CTA slot of the workspace, a per-tile counter
//    tells who arrived last, and that CTA adds the partial tiles in CTA order (fixed order: bit-identical from run to
//    run), applies the epilogue, writes y_s, the per-tile sums of squares the next stage's RMS factor needs, and bumps
//    the stage's completion counter.
//  * Row-parallel stages (tensor parallelism) finish their tile across ranks in the same place: the partial sums are
//    pushed to every peer's staging area as (value, epoch) words and summed in rank order, exactly as
//    gemm_smallm_kernel does, while the weight stream of the following stage keeps running.
//
// Every wait is bounded; the first one that runs out sets the status word and an abort flag that makes all later waits
// of the CTA return at once, so a broken dependency costs about a second, never a hang.
//
// Reference counterpart: the per-operator dispatch of onnxruntime/core/framework/sequential_executor.cc:526-771 over
// MatMul (onnxruntime/core/providers/cuda/math/matmul.cc:180-419), SkipSimplifiedLayerNormalization and the
// AllReduce of onnxruntime/contrib_ops/cuda/collective/nccl_kernels.cc:413-427 - one launch each.
#include <cuda.h>
#include <cuda_runtime.h>
#include "gemm_internal.h"
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"

namespace ortb200 {

namespace {

constexpr int kBM = 128;        // weight rows per tile (the MMA's M)
constexpr int kBK = 64;         // k-block
constexpr int kBN = 16;         // token columns of the MMA (M <= 16)
constexpr int kNW = 10;         // weight ring slots (16 KiB each)
constexpr int kNX = 16;         // activation ring slots (2 KiB each)
constexpr int kWBytes = kBM * kBK * 2;
constexpr int kXBytes = kBN * kBK * 2;
constexpr int kThreads = 224;   // W producer, MMA issuer, X loader, four epilogue warps
constexpr int kMaxStages = ORTB200_CHAIN_MAX_STAGES;
constexpr int kMaxTiles = 4096;     // tiles per stage (N <= 524288)
constexpr int kMaxSsqTiles = 1024;  // tiles of a stage whose output is RMS-normalised by the next one
constexpr unsigned int kPollLimit = 1u << 22;

// workspace layout (bytes)
constexpr long long kWsDone = 0;                                         // unsigned done[4], exited, pad
constexpr long long kWsCnt = 256;                                        // unsigned cnt[4][kMaxTiles]
constexpr long long kWsSsq = kWsCnt + 4LL * kMaxStages * kMaxTiles;      // float ssq[4][kMaxSsqTiles][16]
constexpr long long kWsPart = kWsSsq + 4LL * kMaxStages * kMaxSsqTiles * 16;  // float part[G][2][32][128]
constexpr long long kPartBytesPerCta = 2LL * 32 * 128 * 4;

struct ChainStageDev {
  int N, K, Kb, tiles, wpk;   // wpk: weight tiles per item (2 = gate and up rows)
  int dual_offset, act, all_reduce, ar_index, residual_stage, next_rms;
  float rms_eps;
  long long T;                // items in the stage
  const void* bias;
  const void* residual;
  long long ldr;
  void* out;
};

struct ChainParams {
  ChainStageDev st[kMaxStages];
  const void* x;
  int M, num_stages, dtype, prefetch_dist;
  unsigned int* done;
  unsigned int* cnt;
  float* ssq;
  float* part;
  int* status;
  int world, rank, num_ar;
  void* peers[8];
  long long staging_offset, slot_elems;
  unsigned int* epoch;
  unsigned long long* trace;  // optional [G][32] device timestamps (ns) of one launch, for profiling
};

struct ChainMaps {
  CUtensorMap m[kMaxStages];
};

struct ChainSmem {
  static constexpr int kWOff = 0;
  static constexpr int kXOff = kNW * kWBytes;
  static constexpr int kBarOff = kXOff + kNX * kXBytes;
  static constexpr int kNumBars = 2 * kNW + 2 * kNX + 4 + 1;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;
  static constexpr int kTotal = kMiscOff + 1024 + 1024;  // misc + alignment slack
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned short ld_cg_u16(const void* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tma_prefetch_2d(const void* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void st_packed_sys(unsigned long long* p, float v, unsigned int epoch) {
  const unsigned long long w = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_packed_sys(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}

__device__ __forceinline__ void trace_mark(unsigned long long* trace, int cta, int idx) {
  if (trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    trace[cta * 32 + idx] = t;
  }
}

__device__ __forceinline__ float chain_act(int act, float v) {
  switch (act) {
    case ORTB200_ACT_GELU: return gelu_erf_fast(v);
    case ORTB200_ACT_FASTGELU: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
    case ORTB200_ACT_RELU: return fmaxf(v, 0.0f);
    case ORTB200_ACT_SILU: return v / (1.0f + __expf(-v));
    case ORTB200_ACT_QUICKGELU: return v / (1.0f + __expf(-1.702f * v));
    default: return v;
  }
}

// Bounded waits that give up at once after the first failure in this CTA.
struct Waiter {
  volatile int* abort_flag;
  int* status;
  __device__ __forceinline__ bool aborted() const { return *abort_flag != 0; }
  __device__ __forceinline__ void fail(int code) const {
    *abort_flag = 1;
    if (status) atomicExch(status, code);
  }
  __device__ __forceinline__ bool bar(uint64_t* b, uint32_t parity, int code) const {
    if (*abort_flag) return false;
    if (mbar_wait(b, parity)) return true;
    fail(code);
    return false;
  }
  // waits until *ctr >= target (another CTA's release-increments)
  __device__ __forceinline__ bool counter(const unsigned int* ctr, unsigned int target) const {
    if (*abort_flag) return false;
    for (unsigned int it = 0; it < kPollLimit; ++it) {
      if (ld_acquire_gpu(ctr) >= target) return true;
      if ((it & 255u) == 255u && *abort_flag) return false;
      __nanosleep(20);
    }
    fail(kStatusTimeoutSplitK);
    return false;
  }
};

__device__ __forceinline__ long long slice_lo(long long T, int c, int G) { return T * c / G; }

__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_cg_f4(float* p, float4 v) {
  asm volatile("st.global.cg.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// A parked partial tile is part[slot][row r][32]: columns [0, 16) hold the token sums of the first operand and
// [16, 32) those of the gate/up partner, so a thread moves its row with 16-byte accesses.
// Adds the partial tiles of `tile` in ascending CTA order (CH at a time so that their loads overlap) into acc[0..4 W4).
template <int W4, int CH>
__device__ __forceinline__ void sum_partials(const float* part, long long T, int Kb, int tile, int G, int r, int col_off, float* acc) {
  const long long t0 = static_cast<long long>(tile) * Kb, t1 = t0 + Kb;
  int c = static_cast<int>(t0 * G / T);
  while (c + 1 < G && slice_lo(T, c + 1, G) <= t0) ++c;
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  long long clo = slice_lo(T, c, G);
  while (c < G && clo < t1) {
    const float* src[CH];
    int nsrc = 0;
    for (; nsrc < CH && c < G && clo < t1; ++c) {
      const long long chi = slice_lo(T, c + 1, G);
      const long long start = clo > t0 ? clo : t0;
      if (chi > start) src[nsrc++] = part + ((static_cast<long long>(c) * 2 + (start == clo ? 0 : 1)) * 128 + r) * 32 + col_off;
      clo = chi;
    }
    float4 pv[CH][W4];
#pragma unroll
    for (int k = 0; k < CH; ++k) {
#pragma unroll
      for (int w = 0; w < W4; ++w) pv[k][w] = k < nsrc ? ld_cg_f4(src[k] + 4 * w) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < CH; ++k) {
#pragma unroll
      for (int w = 0; w < W4; ++w) {
        acc[4 * w] += pv[k][w].x;
        acc[4 * w + 1] += pv[k][w].y;
        acc[4 * w + 2] += pv[k][w].z;
        acc[4 * w + 3] += pv[k][w].w;
      }
    }
  }
}

// Activation loader (one warp).  A k-block of the activations is 16 token rows x 128 bytes; lane l moves the 16-byte
// chunk l & 7 of rows (l >> 3) + 4 j, j < RPL (RPL = 2 covers 8 token rows, RPL = 4 all 16; rows >= M are zero).  Sixteen
// 16-byte registers hold a batch of 16 / RPL k-blocks, and the next batch is requested before the current one is
// written to shared memory, so the L2 round trip of one batch hides behind the previous batch.
template <int RPL>
__device__ __forceinline__ void load_activations(const ChainParams& p, const Waiter& wt, uint8_t* x_ring, uint64_t* x_full,
                                                 uint64_t* x_empty, int cta, int G, int lane) {
  constexpr int NB = 16 / RPL;
  unsigned int xn = 0;
  const int c16 = lane & 7;
  const int r0 = lane >> 3;
  for (int s = 0; s < p.num_stages && !wt.aborted(); ++s) {
    const ChainStageDev& q = p.st[s];
    const long long lo = slice_lo(q.T, cta, G), hi = slice_lo(q.T, cta + 1, G);
    if (lo >= hi) continue;
    const uint8_t* src = static_cast<const uint8_t*>(s == 0 ? p.x : p.st[s - 1].out);
    if (s > 0 && !wt.counter(&p.done[s - 1], static_cast<unsigned int>(p.st[s - 1].tiles))) break;
    if (lane == 0) trace_mark(p.trace, cta, 1 + 6 * s);
    const long long row_bytes = static_cast<long long>(q.K) * 2;
    uint4 cur[NB][RPL], nxt[NB][RPL];
    auto fetch = [&](long long i0, uint4 (&buf)[NB][RPL]) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int kb = static_cast<int>((i0 + b) % q.Kb);
#pragma unroll
        for (int j = 0; j < RPL; ++j) {
          const int row = r0 + 4 * j;
          buf[b][j] = (i0 + b < hi && row < p.M) ? ld_cg_v4(src + row * row_bytes + kb * (kBK * 2) + c16 * 16) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    fetch(lo, cur);
    bool ok = true;
    for (long long i = lo; i < hi && ok; i += NB) {
      if (i + NB < hi) fetch(i + NB, nxt);
      const int nb = static_cast<int>(min(static_cast<long long>(NB), hi - i));
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if (b >= nb) break;
        const int xs = (xn + b) % kNX;
        const unsigned int use = (xn + b) / kNX;
        if (use > 0 && ok) ok = wt.bar(&x_empty[xs], (use - 1) & 1, kStatusTimeoutProducer);
        if (ok) {
          uint8_t* dst = x_ring + xs * kXBytes;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = r0 + 4 * j;
            *reinterpret_cast<uint4*>(dst + row * 128 + ((c16 ^ (row & 7)) << 4)) = j < RPL ? cur[b][j < RPL ? j : 0] : make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      // one cross-proxy fence for the whole batch (it is the expensive part), then publish the blocks
      fence_proxy_async();
      for (int b = 0; b < nb; ++b) mbar_arrive(&x_full[(xn + b) % kNX]);  // also on the failure path
      xn += nb;
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int j = 0; j < RPL; ++j) cur[b][j] = nxt[b][j];
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
  using S = ChainSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_ring = smem + S::kWOff;
  uint8_t* x_ring = smem + S::kXOff;
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
  uint64_t* w_empty = w_full + kNW;
  uint64_t* x_full = w_empty + kNW;
  uint64_t* x_empty = x_full + kNX;
  uint64_t* acc_full = x_empty + kNX;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* fin_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_flag = const_cast<int*>(abort_flag) + 1;
  float* s_rstd = reinterpret_cast<float*>(s_flag + 1);  // [16]
  float* s_red = s_rstd + 16;                            // [8][16]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const int cta = blockIdx.x;
  const bool bf16 = p.dtype == ORTB200_BF16;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxStages; ++i)
      if (i < p.num_stages) tma_prefetch_desc(&maps.m[i]);
    for (int i = 0; i < kNW; ++i) {
      mbar_init(&w_full[i], 1);
      mbar_init(&w_empty[i], 1);
    }
    for (int i = 0; i < kNX; ++i) {
      mbar_init(&x_full[i], 32);
      mbar_init(&x_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    mbar_init(fin_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const Waiter wt{abort_flag, p.status};
  if (threadIdx.x == 0) trace_mark(p.trace, cta, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ weight producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_first();
      unsigned int wn = 0;  // ring uses so far
      // the L2 prefetch cursor runs `prefetch_dist` items ahead of the ring, across stage boundaries
      int ps = 0;
      long long pi = slice_lo(p.st[0].T, cta, G), pend = slice_lo(p.st[0].T, cta + 1, G);
      long long ahead = 0;
      auto advance_prefetch = [&](long long want_ahead) {
        while (ahead < want_ahead && ps < p.num_stages) {
          if (pi >= pend) {
            ++ps;
            if (ps < p.num_stages) {
              pi = slice_lo(p.st[ps].T, cta, G);
              pend = slice_lo(p.st[ps].T, cta + 1, G);
            }
            continue;
          }
          const ChainStageDev& q = p.st[ps];
          const int tile = static_cast<int>(pi / q.Kb), kb = static_cast<int>(pi % q.Kb);
          for (int h = 0; h < q.wpk; ++h) tma_prefetch_2d(&maps.m[ps], kb * kBK, tile * kBM + h * q.dual_offset);
          ++pi;
          ++ahead;
        }
      };
      for (int s = 0; s < p.num_stages && !wt.aborted(); ++s) {
        const ChainStageDev& q = p.st[s];
        const long long lo = slice_lo(q.T, cta, G), hi = slice_lo(q.T, cta + 1, G);
        for (long long i = lo; i < hi; ++i) {
          const int tile = static_cast<int>(i / q.Kb), kb = static_cast<int>(i % q.Kb);
          bool ok = true;
          for (int h = 0; h < q.wpk && ok; ++h) {
            const int slot = wn % kNW;
            const unsigned int use = wn / kNW;
            if (use > 0) ok = wt.bar(&w_empty[slot], (use - 1) & 1, kStatusTimeoutProducer);
            if (!ok) break;
            mbar_expect_tx(&w_full[slot], kWBytes);
            tma_load_2d_hint(w_ring + slot * kWBytes, &maps.m[s], &w_full[slot], kb * kBK, tile * kBM + h * q.dual_offset, pol);
            ++wn;
          }
          if (!ok) break;
          if (p.prefetch_dist > 0) {
            --ahead;
            if (ahead < 0) {  // the cursor fell behind the ring (start of the kernel): skip what was just loaded
              ahead = 0;
              ps = s;
              pi = i + 1;
              pend = hi;
            }
            advance_prefetch(p.prefetch_dist);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(bf16, kBM, kBN);
      unsigned int wn = 0, xn = 0, seg = 0;
      for (int s = 0; s < p.num_stages && !wt.aborted(); ++s) {
        const ChainStageDev& q = p.st[s];
        const long long lo = slice_lo(q.T, cta, G), hi = slice_lo(q.T, cta + 1, G);
        long long i = lo;
        bool first_mma = true;
        while (i < hi && !wt.aborted()) {
          const int kb0 = static_cast<int>(i % q.Kb);
          const int n_items = static_cast<int>(min(static_cast<long long>(q.Kb - kb0), hi - i));
          const int a = seg & 1;
          if (seg >= 2 && !wt.bar(&acc_empty[a], ((seg >> 1) - 1) & 1, kStatusTimeoutMma)) break;
          tcgen05_fence_after();
          const uint32_t d0 = tmem_base + a * 32;
          bool ok = true;
          for (int j = 0; j < n_items; ++j) {
            const int xs = xn % kNX;
            ok = wt.bar(&x_full[xs], (xn / kNX) & 1, kStatusTimeoutMma);
            if (!ok) break;
            if (first_mma) {
              trace_mark(p.trace, cta, 2 + 6 * s);
              first_mma = false;
            }
            const uint64_t bdesc = umma_desc_sw128(smem_u32(x_ring + xs * kXBytes));
            for (int h = 0; h < q.wpk; ++h) {
              const int ws = wn % kNW;
              ok = wt.bar(&w_full[ws], (wn / kNW) & 1, kStatusTimeoutMma);
              if (!ok) break;
              tcgen05_fence_after();
              const uint64_t adesc = umma_desc_sw128(smem_u32(w_ring + ws * kWBytes));
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k) umma_f16(d0 + h * kBN, adesc + 2 * k, bdesc + 2 * k, idesc, (j > 0 || k > 0) ? 1u : 0u);
              umma_commit(&w_empty[ws]);
              ++wn;
            }
            if (!ok) break;
            umma_commit(&x_empty[xs]);
            ++xn;
          }
          umma_commit(&acc_full[a]);  // also on the failure path: the epilogue must not wait for nothing
          trace_mark(p.trace, cta, 3 + 6 * s);
          if (!ok) break;
          ++seg;
          i += n_items;
        }
      }
      umma_commit(fin_bar);
      mbar_wait(fin_bar, 0);  // every MMA has retired before tensor memory is released
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ activation loader
    pdl_wait_prior_grids();
    if (p.M <= 8) load_activations<2>(p, wt, x_ring, x_full, x_empty, cta, G, lane);
    else load_activations<4>(p, wt, x_ring, x_full, x_empty, cta, G, lane);
  } else {
    // ------------------------------------------------------------------ epilogue warps (3..6)
    pdl_wait_prior_grids();
    const int qd = warp & 3;
    const int r = qd * 32 + lane;               // weight row of the tile == output feature within the tile
    const int et = threadIdx.x - 96;            // 0..127
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const int M = p.M;
    unsigned int seg = 0;
    unsigned int epoch_base = 0, spin_limit = 1u << 22;
    if (p.world > 1) {
      epoch_base = *reinterpret_cast<volatile unsigned int*>(p.epoch);
      const unsigned int lim = reinterpret_cast<volatile unsigned int*>(p.epoch)[2];
      if (lim != 0) spin_limit = lim;
    }
    for (int s = 0; s < p.num_stages; ++s) {
      const ChainStageDev& q = p.st[s];
      const long long lo = slice_lo(q.T, cta, G), hi = slice_lo(q.T, cta + 1, G);
      if (lo >= hi) continue;
      const bool dual = q.wpk == 2;
      if (q.rms_eps > 0.f) {
        // 1 / rms of every token row of this stage's input, from the per-tile sums the previous stage left
        wt.counter(&p.done[s - 1], static_cast<unsigned int>(p.st[s - 1].tiles));
        const int tiles_prev = p.st[s - 1].tiles;
        const float* sq = p.ssq + static_cast<long long>(s - 1) * kMaxSsqTiles * 16;
        const int m = et & 15, g = et >> 4;
        float acc = 0.f;
        for (int t = g; t < tiles_prev; t += 8) acc += ld_cg_f32(sq + t * 16 + m);
        s_red[g * 16 + m] = acc;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et < 16) {
          float tot = 0.f;
#pragma unroll
          for (int gg = 0; gg < 8; ++gg) tot += s_red[gg * 16 + et];
          s_rstd[et] = rsqrtf(tot / static_cast<float>(q.K) + q.rms_eps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      long long i = lo;
      while (i < hi) {
        const int tile = static_cast<int>(i / q.Kb);
        const int kb0 = static_cast<int>(i % q.Kb);
        const int n_items = static_cast<int>(min(static_cast<long long>(q.Kb - kb0), hi - i));
        const int a = seg & 1;
        wt.bar(&acc_full[a], (seg >> 1) & 1, kStatusTimeoutEpilogue);
        if (et == 0 && i == lo) trace_mark(p.trace, cta, 6 + 6 * s);  // first accumulator of the stage arrived
        tcgen05_fence_after();
        float v[16], u[16];
        tmem_ld_x16(t_lane + a * 32, v);
        if (dual) tmem_ld_x16(t_lane + a * 32 + kBN, u);
        tmem_ld_wait();
        tcgen05_fence_before();
        mbar_arrive(&acc_empty[a]);
        ++seg;
        const int n = tile * kBM + r;
        const bool n_ok = n < q.N;
        bool finish = true;
        if (n_items != q.Kb) {
          // ---- partial tile: park it, count the k-blocks, and let the last arrival add everything up in CTA order
          float* mine = p.part + ((static_cast<long long>(cta) * 2 + (i == lo ? 0 : 1)) * 128 + r) * 32;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            if (4 * w < M) {
              st_cg_f4(mine + 4 * w, make_float4(v[4 * w], v[4 * w + 1], v[4 * w + 2], v[4 * w + 3]));
              if (dual) st_cg_f4(mine + 16 + 4 * w, make_float4(u[4 * w], u[4 * w + 1], u[4 * w + 2], u[4 * w + 3]));
            }
          }
          // bar.sync orders the 128 threads' stores before thread 0's release (cumulative at GPU scope); the acquire
          // half orders the last arrival's reads after every contributor's release
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) {
            unsigned int* ctr = p.cnt + s * kMaxTiles + tile;
            unsigned int old;
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(ctr), "r"(static_cast<unsigned int>(n_items)) : "memory");
            const int last = (old + n_items == static_cast<unsigned int>(q.Kb)) ? 1 : 0;
            if (last) *ctr = 0;  // left zero for the next launch
            *s_flag = last;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          finish = *s_flag != 0;
        }
        // the residual does not depend on this stage: fetch it while the partial tiles travel
        float resv[16];
        if (finish) {
          const uint8_t* res = static_cast<const uint8_t*>(q.residual_stage >= 0 ? p.st[q.residual_stage].out : q.residual);
          const long long ldr = q.residual_stage >= 0 ? p.st[q.residual_stage].N : q.ldr;
          unsigned short rb[16];
#pragma unroll
          for (int m = 0; m < 16; ++m) rb[m] = (res != nullptr && m < M && n_ok) ? ld_cg_u16(res + (static_cast<long long>(m) * ldr + n) * 2) : 0;
          if (n_items != q.Kb) {
            if (M <= 8) {
              sum_partials<2, 8>(p.part, q.T, q.Kb, tile, G, r, 0, v);
              if (dual) sum_partials<2, 8>(p.part, q.T, q.Kb, tile, G, r, 16, u);
            } else {
              sum_partials<4, 4>(p.part, q.T, q.Kb, tile, G, r, 0, v);
              if (dual) sum_partials<4, 4>(p.part, q.T, q.Kb, tile, G, r, 16, u);
            }
          }
#pragma unroll
          for (int m = 0; m < 16; ++m) resv[m] = bf16 ? __bfloat162float(__ushort_as_bfloat16(rb[m])) : __half2float(__ushort_as_half(rb[m]));
        }
        if (finish) {
          // ---- final epilogue of this tile
          if (q.all_reduce && p.world > 1) {
            // push the rank-local sums to every rank (value | epoch words), then gather all ranks' words in rank order
            const unsigned int epoch = epoch_base + 1 + static_cast<unsigned int>(q.ar_index);
            const long long stage_base = static_cast<long long>(epoch & 1) * p.world * p.slot_elems;
            if (n_ok) {
#pragma unroll
              for (int m = 0; m < 16; ++m) {
                if (m >= M) break;
                const long long off = stage_base + static_cast<long long>(p.rank) * p.slot_elems + static_cast<long long>(m) * q.N + n;
                for (int d = 0; d < p.world; ++d) {
                  const int dst = (p.rank + d) % p.world;
                  st_packed_sys(reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(p.peers[dst]) + p.staging_offset) + off, v[m], epoch);
                }
              }
              const unsigned long long* local =
                  reinterpret_cast<const unsigned long long*>(static_cast<const uint8_t*>(p.peers[p.rank]) + p.staging_offset) + stage_base;
              bool timed_out = wt.aborted();
#pragma unroll
              for (int m0 = 0; m0 < 16; m0 += 2) {
                if (m0 >= M) break;
                unsigned long long w[2][8];
                const unsigned long long* sp[2];
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                  const bool need = m0 + cb < M;
                  sp[cb] = local + static_cast<long long>(m0 + cb) * q.N + n;
#pragma unroll
                  for (int sr = 0; sr < 8; ++sr)
                    w[cb][sr] = (need && sr < p.world) ? ld_packed_sys(sp[cb] + static_cast<long long>(sr) * p.slot_elems)
                                                       : (static_cast<unsigned long long>(epoch) << 32);
                }
                unsigned int spins = 0;
                while (!timed_out) {
                  bool all = true;
#pragma unroll
                  for (int cb = 0; cb < 2; ++cb)
#pragma unroll
                    for (int sr = 0; sr < 8; ++sr) all = all && (static_cast<unsigned int>(w[cb][sr] >> 32) == epoch);
                  if (all) break;
                  if (++spins > spin_limit) {
                    timed_out = true;
                    break;
                  }
                  __nanosleep(32);
#pragma unroll
                  for (int cb = 0; cb < 2; ++cb)
#pragma unroll
                    for (int sr = 0; sr < 8; ++sr)
                      if (static_cast<unsigned int>(w[cb][sr] >> 32) != epoch)
                        w[cb][sr] = ld_packed_sys(sp[cb] + static_cast<long long>(sr) * p.slot_elems);
                }
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                  float y = 0.f;
#pragma unroll
                  for (int sr = 0; sr < 8; ++sr)  // fixed order: every rank adds in the same order and gets the same bits
                    if (sr < p.world) y += __uint_as_float(static_cast<unsigned int>(w[cb][sr]));
                  v[m0 + cb] = y;
                }
              }
              if (timed_out && !wt.aborted()) wt.fail(kStatusTimeoutPeer);
            }
          }
          const float bias_v = (q.bias != nullptr && n_ok)
                                   ? (bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(q.bias)[n]) : __half2float(static_cast<const __half*>(q.bias)[n]))
                                   : 0.f;
          float sq[16];
#pragma unroll
          for (int m = 0; m < 16; ++m) {
            sq[m] = 0.f;
            if (m < M && n_ok) {
              const float rs = q.rms_eps > 0.f ? s_rstd[m] : 1.0f;
              float y = v[m] * rs + bias_v;
              if (dual) {
                const float gte = y / (1.0f + __expf(-y));
                y = gte * (u[m] * rs);
              } else {
                y = chain_act(q.act, y);
              }
              y += resv[m];
              unsigned short bits;
              if (bf16) {
                const __nv_bfloat16 h = __float2bfloat16_rn(y);
                bits = __bfloat16_as_ushort(h);
                y = __bfloat162float(h);
              } else {
                const __half h = __float2half_rn(y);
                bits = __half_as_ushort(h);
                y = __half2float(h);
              }
              static_cast<unsigned short*>(q.out)[static_cast<long long>(m) * q.N + n] = bits;
              sq[m] = y * y;
            }
          }
          if (q.next_rms) {
            // sums of squares of this tile's 128 features per token, for the RMS factor of the next stage
#pragma unroll
            for (int m = 0; m < 16; ++m)
              if (m < M) sq[m] = warp_sum(sq[m]);
            // s_red is free here: the factors of this stage were computed before its first tile
            if (lane == 0) {
#pragma unroll
              for (int m = 0; m < 16; ++m) s_red[qd * 16 + m] = sq[m];
            }
          }
          // the barriers order every thread's stores before thread 0's release, which is cumulative at GPU scope
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (q.next_rms && et < 16) {
            const float tot = s_red[et] + s_red[16 + et] + s_red[32 + et] + s_red[48 + et];
            __stcg(p.ssq + (static_cast<long long>(s) * kMaxSsqTiles + tile) * 16 + et, tot);
          }
          if (q.next_rms) asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) {
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.done + s) : "memory");
          }
        }
        if (et == 0) trace_mark(p.trace, cta, (finish ? 5 : 4) + 6 * s);  // last partial parked / last tile finished
        i += n_items;
      }
    }
  }

  if (threadIdx.x == 0) trace_mark(p.trace, cta, 30);
  pdl_launch_dependents();
  if (*abort_flag) {
    // a wait ran out: loads issued before that may still be in flight; give them time to land before the shared
    // memory can be handed to another CTA
    for (int k = 0; k < 200; ++k) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
  if (threadIdx.x == 96) {
    // the CTA that leaves last clears the stage counters and advances the all-reduce epoch for the next launch
    unsigned int* exited = p.done + kMaxStages;
    __threadfence();
    if (atomicAdd(exited, 1u) == static_cast<unsigned int>(G) - 1) {
      for (int s = 0; s < kMaxStages; ++s) p.done[s] = 0;
      *exited = 0;
      if (p.world > 1 && p.num_ar > 0) {
        const unsigned int e = *reinterpret_cast<volatile unsigned int*>(p.epoch);
        __threadfence();
        *reinterpret_cast<volatile unsigned int*>(p.epoch) = e + static_cast<unsigned int>(p.num_ar);
      }
      __threadfence();
    }
  }
}

}  // namespace

}  // namespace ortb200

extern "C" int64_t ortb200_gemm_chain_workspace_bytes(void) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 256;
  return ortb200::kWsPart + ortb200::kPartBytesPerCta * sms;
}

extern "C" int ortb200_gemm_chain(const ortb200_gemm_chain_args* a, ortb200_stream_t stream_) {
  using namespace ortb200;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->x || !a->workspace) return -1;
  if (a->num_stages < 1 || a->num_stages > kMaxStages || a->M < 1) return -1;
  if (a->M > kBN) return -8;
  if (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16) return -4;
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->workspace)) & 15) return -3;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -10;
  }
  if (a->workspace_bytes < kWsPart + kPartBytesPerCta * sms) return -5;
  ChainParams p{};
  ChainMaps maps{};
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  int num_ar = 0;
  long long max_items = 0;
  int prev_n = 0;
  for (int s = 0; s < a->num_stages; ++s) {
    const ortb200_chain_stage& st = a->stage[s];
    ChainStageDev& q = p.st[s];
    if (!st.w || !st.out || st.N <= 0 || st.K <= 0 || st.K % kBK != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(st.w) | reinterpret_cast<uintptr_t>(st.out)) & 15) return -3;
    if (s > 0 && st.K != prev_n) return -2;  // the stage's input is the previous stage's output
    const bool dual = st.act == ORTB200_ACT_SWIGLU;
    if (dual && st.dual_offset <= 0) return -2;
    if (st.w_rows < (dual ? st.dual_offset + st.N : st.N)) return -2;
    if (st.rms_eps > 0.f && (s == 0 || (st.all_reduce && a->world > 1))) return -14;
    if (st.residual_stage >= s) return -2;
    if (st.residual_stage >= 0 && a->stage[st.residual_stage].N != st.N) return -2;
    if (st.residual_stage < 0 && st.residual && st.ldr < st.N) return -2;
    q.N = st.N; q.K = st.K; q.Kb = st.K / kBK; q.tiles = (st.N + kBM - 1) / kBM; q.wpk = dual ? 2 : 1;
    if (q.tiles > kMaxTiles) return -7;
    q.T = static_cast<long long>(q.tiles) * q.Kb;
    q.dual_offset = dual ? st.dual_offset : 0;
    q.act = dual ? ORTB200_ACT_NONE : st.act;
    q.all_reduce = (st.all_reduce && a->world > 1) ? 1 : 0;
    q.ar_index = num_ar;
    if (q.all_reduce) {
      if (dual) return -12;
      ++num_ar;
    }
    q.residual_stage = st.residual_stage;
    q.next_rms = (s + 1 < a->num_stages && a->stage[s + 1].rms_eps > 0.f) ? 1 : 0;
    if (q.next_rms && q.tiles > kMaxSsqTiles) return -7;
    q.rms_eps = st.rms_eps;
    q.bias = st.bias; q.residual = st.residual_stage >= 0 ? nullptr : st.residual; q.ldr = st.ldr; q.out = st.out;
    if (make_tensor_map_2d(&maps.m[s], st.w, dt, 2, st.K, st.w_rows, static_cast<int64_t>(st.K) * 2, kBK, kBM) != 0) return -6;
    max_items = q.T > max_items ? q.T : max_items;
    prev_n = st.N;
  }
  p.x = a->x; p.M = a->M; p.num_stages = a->num_stages; p.dtype = a->dtype;
  p.prefetch_dist = a->prefetch_items < 0 ? 0 : (a->prefetch_items > 64 ? 64 : a->prefetch_items);
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.done = reinterpret_cast<unsigned int*>(ws + kWsDone);
  p.cnt = reinterpret_cast<unsigned int*>(ws + kWsCnt);
  p.ssq = reinterpret_cast<float*>(ws + kWsSsq);
  p.part = reinterpret_cast<float*>(ws + kWsPart);
  p.status = a->status;
  p.trace = static_cast<unsigned long long*>(a->trace);
  p.world = 1; p.rank = 0; p.num_ar = 0;
  if (a->world > 1 && num_ar > 0) {
    if (a->world > 8 || a->rank < 0 || a->rank >= a->world) return -12;
    const long long staging_off = 262144;
    const long long slot = (a->symm_bytes / 2 - staging_off) / (2LL * a->world * 8);
    for (int s = 0; s < a->num_stages; ++s)
      if (p.st[s].all_reduce && slot < static_cast<long long>(a->M) * p.st[s].N) return -13;
    for (int i = 0; i < a->world; ++i) {
      if (!a->peers[i]) return -12;
      p.peers[i] = a->peers[i];
    }
    p.world = a->world; p.rank = a->rank; p.num_ar = num_ar; p.staging_offset = staging_off; p.slot_elems = slot;
    p.epoch = reinterpret_cast<unsigned int*>(a->peers[a->rank]);
  }
  int grid = sms;
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if (max_items < grid) grid = static_cast<int>(max_items);
  auto kern = gemm_chain_kernel;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ChainSmem::kTotal) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = ChainSmem::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int nattr = 0;
  if (a->use_pdl) {
    attrs[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = nattr;
  return cudaLaunchKernelEx(&cfg, kern, maps, p) == cudaSuccess ? 0 : -11;
}
