// Dense GEMM for sm_100a: TMA-fed tcgen05.mma with the accumulator in tensor
// memory.  out[M, N] = act(alpha * X[M,K] * W[N,K]^T + bias) + residual.
//
// Replaces the cuBLAS calls of the reference's MatMul/Gemm/FusedMatMul kernels
// (onnxruntime/core/providers/cuda/math/matmul.cc:180-419) and the QKV
// projection inside Attention (onnxruntime/contrib_ops/cuda/bert/attention.cc:251).
//
// Orientation: the WEIGHT tile is the MMA's A operand (128 rows = 128 TMEM
// lanes), the token tile is the B operand (BN = 16..256 columns).  A decode
// step with 8 tokens therefore wastes no tensor-core rows on padding: one CTA
// streams a 128 x K slab of W exactly once.  Split-K spreads narrow problems
// over all SMs; partial tiles go to an fp32 workspace and the CTA that arrives
// last on a per-tile counter reduces them in a fixed order (deterministic) and
// runs the epilogue.  No host round trip, no second launch.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer (one elected lane), warps 2..5 = epilogue (one TMEM lane quarter each).
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include <unordered_map>
#include <stdio.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"

namespace ortb200 {

constexpr int kBM = 128;      // weight rows per tile (TMEM lanes)
constexpr int kBK = 64;       // K elements per stage (128 bytes of 16-bit data)
constexpr int kThreads = 192;

struct GemmKernelParams {
  int M, N, K;
  int num_kb;         // ceil(K / 64)
  int kb_per_split;
  int splits;
  int dual_offset;
  int dtype;
  int act;
  float alpha;
  void* out;
  long long ldo;
  const void* bias;
  const void* residual;
  long long ldr;
  float* ws;
  unsigned int* counters;
  int* status;
};

__device__ __forceinline__ float apply_act(int act, float v) {
  switch (act) {
    case ORTB200_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    case ORTB200_ACT_FASTGELU: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
    case ORTB200_ACT_RELU: return fmaxf(v, 0.0f);
    case ORTB200_ACT_SILU: return v / (1.0f + __expf(-v));
    case ORTB200_ACT_QUICKGELU: return v / (1.0f + __expf(-1.702f * v));
    default: return v;
  }
}

template <int BN, int STAGES, bool DUAL>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes * (DUAL ? 2 : 1) + kBBytes;
  static constexpr int kBarOffset = kStageBytes * STAGES;
  static constexpr int kTotal = kBarOffset + 8 * (2 * STAGES + 1) + 16 + 1024;  // + alignment slack
  static constexpr int kTmemCols = (DUAL ? 2 : 1) * BN < 32 ? 32 : (DUAL ? 2 : 1) * BN;
};

template <int BN, int STAGES, bool DUAL>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const GemmKernelParams p) {
  using S = GemmSmem<BN, STAGES, DUAL>;
  static_assert((S::kTmemCols & (S::kTmemCols - 1)) == 0, "TMEM columns must be a power of two");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  uint32_t* last_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kBM;
  const int m0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int kb_begin = split * p.kb_per_split;
  int kb_end = kb_begin + p.kb_per_split;
  if (kb_end > p.num_kb) kb_end = p.num_kb;
  const int nkb = kb_end - kb_begin;  // >= 1 by construction on the host

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Let the next kernel in the stream start its own prologue.
  pdl_launch_dependents();

  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the previous kernel: fill the pipeline with W
      // tiles first, then wait for the producer of X, then add the X tiles.
      const uint64_t pol_w = policy_evict_first();
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * S::kStageBytes;
        mbar_expect_tx(&full_bar[i], S::kStageBytes);
        tma_load_2d_hint(st, &tmap_w, &full_bar[i], (kb_begin + i) * kBK, n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + S::kABytes, &tmap_w, &full_bar[i], (kb_begin + i) * kBK, n0 + p.dual_offset, pol_w);
      }
      pdl_wait_prior_grids();
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * S::kStageBytes;
        tma_load_2d(st + S::kABytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[i], (kb_begin + i) * kBK, m0);
      }
      for (int i = pre; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t parity = ((i / STAGES) - 1) & 1;
        if (!mbar_wait(&empty_bar[s], parity)) {
          failed = true;
          if (p.status) atomicExch(p.status, kStatusTimeoutProducer);
          break;
        }
        uint8_t* st = smem + s * S::kStageBytes;
        mbar_expect_tx(&full_bar[s], S::kStageBytes);
        tma_load_2d_hint(st, &tmap_w, &full_bar[s], (kb_begin + i) * kBK, n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + S::kABytes, &tmap_w, &full_bar[s], (kb_begin + i) * kBK, n0 + p.dual_offset, pol_w);
        tma_load_2d(st + S::kABytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[s], (kb_begin + i) * kBK, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(p.dtype == ORTB200_BF16, kBM, BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t parity = (i / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], parity)) {
          failed = true;
          if (p.status) atomicExch(p.status, kStatusTimeoutMma);
          break;
        }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * S::kStageBytes);
        const uint32_t b_addr = a_addr + S::kABytes * (DUAL ? 2 : 1);
        const uint64_t adesc = umma_desc_sw128(a_addr);
        const uint64_t bdesc = umma_desc_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          // 16 K-elements = 32 bytes: the start-address field advances by 2
          umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        if (DUAL) {
          const uint64_t a2desc = umma_desc_sw128(a_addr + S::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            umma_f16(tmem_base + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty_bar[s]);  // stage is reusable once these MMAs have read it
      }
      umma_commit(tmem_full_bar);    // accumulator complete (also signalled on the failure path)
    }
  } else {
    // ---------------------------------------------------------- epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;            // lane within the tile == weight row
    const int n = n0 + r;
    const bool n_ok = n < p.N;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;

    pdl_wait_prior_grids();                 // out / residual / workspace may belong to the previous kernel
    if (!mbar_wait(tmem_full_bar, 0)) {
      failed = true;
      if (p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
    }
    tcgen05_fence_after();

    bool do_output = !failed;
    if (!failed && p.splits > 1) {
      // 1) publish this split's partial tile
      constexpr int kCols = (DUAL ? 2 : 1) * BN;
      float* my_ws = p.ws + (static_cast<size_t>(tile_id) * p.splits + split) * (kCols * kBM);
#pragma unroll 1
      for (int c = 0; c < kCols; c += 16) {
        float v[16];
        tmem_ld_x16(t_lane + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) my_ws[(c + j) * kBM + r] = v[j];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const unsigned int old = atomicAdd(&p.counters[tile_id], 1u);
        const unsigned int last = (old == static_cast<unsigned int>(p.splits - 1)) ? 1u : 0u;
        if (last) p.counters[tile_id] = 0;  // re-arm for the next launch (graph replay safe)
        *last_flag = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      do_output = (*last_flag != 0);
      if (do_output) __threadfence();
    }

    if (do_output) {
      const float bias_v = (p.bias != nullptr && n_ok)
                               ? (p.dtype == ORTB200_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n])
                                                          : __half2float(reinterpret_cast<const __half*>(p.bias)[n]))
                               : 0.0f;
      constexpr int kCols = (DUAL ? 2 : 1) * BN;
      const float* tile_ws = p.splits > 1 ? p.ws + static_cast<size_t>(tile_id) * p.splits * (kCols * kBM) : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        float u[16];
        if (p.splits == 1) {
          tmem_ld_x16(t_lane + c, v);
          if (DUAL) tmem_ld_x16(t_lane + BN + c, u);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) { v[j] = 0.0f; u[j] = 0.0f; }
          for (int s = 0; s < p.splits; ++s) {
            const float* src = tile_ws + static_cast<size_t>(s) * (kCols * kBM);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] += __ldcg(&src[(c + j) * kBM + r]);
              if (DUAL) u[j] += __ldcg(&src[(BN + c + j) * kBM + r]);
            }
          }
        }
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c + j;
            if (m < p.M) {
              float y = v[j] * p.alpha + bias_v;
              if (DUAL) {
                const float g = y / (1.0f + __expf(-y));
                y = g * (u[j] * p.alpha);
              } else {
                y = apply_act(p.act, y);
              }
              if (p.dtype == ORTB200_BF16) {
                if (p.residual) y += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[m * p.ldr + n]);
                reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.ldo + n] = __float2bfloat16_rn(y);
              } else {
                if (p.residual) y += __half2float(reinterpret_cast<const __half*>(p.residual)[m * p.ldr + n]);
                reinterpret_cast<__half*>(p.out)[m * p.ldo + n] = __float2half_rn(y);
              }
            }
          }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
  (void)failed;
}

// ------------------------------------------------------------------ host side

struct GemmConfig {
  int bn, splits, stages;
};
static thread_local GemmConfig g_last_config = {0, 0, 0};

static int pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

static int pick_splits(int M, int N, int num_kb, int bn) {
  const int tiles = ((N + kBM - 1) / kBM) * ((M + bn - 1) / bn);
  const int kSMs = 148;
  if (tiles >= kSMs || num_kb < 8) return 1;
  int want = (2 * kSMs + tiles - 1) / tiles;
  int max_by_k = num_kb / 4;  // keep at least 4 k-blocks per split
  if (want > max_by_k) want = max_by_k;
  if (want > 16) want = 16;
  if (want < 1) want = 1;
  return want;
}

template <int BN, int STAGES, bool DUAL>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmKernelParams& p, dim3 grid,
                       cudaStream_t stream, bool use_pdl) {
  using S = GemmSmem<BN, STAGES, DUAL>;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, DUAL>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int nattr = 0;
  if (use_pdl) {
    attrs[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = nattr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  return e == cudaSuccess ? 0 : -11;
}

}  // namespace ortb200

using namespace ortb200;

extern "C" int64_t ortb200_gemm_workspace_bytes(int M, int N, int K, int act) {
  const int bn = pick_bn(M);
  const int num_kb = (K + kBK - 1) / kBK;
  const int splits_max = 16;
  const int64_t tiles = static_cast<int64_t>((N + kBM - 1) / kBM) * ((M + bn - 1) / bn);
  const int64_t cols = (act == ORTB200_ACT_SWIGLU ? 2 : 1) * bn;
  (void)num_kb;
  // counters live in the first 64 KiB
  return 65536 + tiles * splits_max * cols * kBM * 4;
}

extern "C" int ortb200_gemm_last_config(int* bn, int* splits, int* stages) {
  if (bn) *bn = g_last_config.bn;
  if (splits) *splits = g_last_config.splits;
  if (stages) *stages = g_last_config.stages;
  return 1;
}

extern "C" int ortb200_gemm(const ortb200_gemm_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->x || !a->w || !a->out) return -1;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return -1;
  if (a->K % 8 != 0) return -2;                                  // TMA row pitch must be a multiple of 16 bytes
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return -3;
  if (a->dtype != ORTB200_F16 && a->dtype != ORTB200_BF16) return -4;
  const bool dual = a->act == ORTB200_ACT_SWIGLU;
  if (dual && (a->dual_offset <= 0 || a->w_rows < a->dual_offset + a->N)) return -5;
  if (!dual && a->w_rows < a->N) return -5;

  int bn = a->force_bn ? a->force_bn : pick_bn(a->M);
  if (dual && bn > 128) bn = 128;     // two accumulators must fit 512 TMEM columns with room to spare
  const int num_kb = (a->K + kBK - 1) / kBK;
  int splits = a->force_splits ? a->force_splits : pick_splits(a->M, a->N, num_kb, bn);
  if (splits > num_kb) splits = num_kb;
  int kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per_split - 1) / kb_per_split;  // no empty splits

  const int tiles_n = (a->N + kBM - 1) / kBM;
  const int tiles_m = (a->M + bn - 1) / bn;
  const int64_t tiles = static_cast<int64_t>(tiles_n) * tiles_m;
  float* ws = nullptr;
  unsigned int* counters = nullptr;
  if (splits > 1) {
    const int64_t need = 65536 + tiles * splits * (dual ? 2 : 1) * bn * kBM * 4;
    if (!a->workspace || a->workspace_bytes < need || tiles > 16384) {
      splits = 1;
      kb_per_split = num_kb;
    } else {
      counters = reinterpret_cast<unsigned int*>(a->workspace);
      ws = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a->workspace) + 65536);
    }
  }

  CUtensorMap tw, tx;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, a->w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) return -6;
  if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->M, static_cast<int64_t>(a->K) * 2, kBK, bn) != 0) return -6;

  GemmKernelParams p;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.num_kb = num_kb; p.kb_per_split = kb_per_split; p.splits = splits;
  p.dual_offset = a->dual_offset; p.dtype = a->dtype; p.act = a->act; p.alpha = a->alpha;
  p.out = a->out; p.ldo = a->ldo; p.bias = a->bias; p.residual = a->residual; p.ldr = a->ldr;
  p.ws = ws; p.counters = counters; p.status = a->status;

  dim3 grid(tiles_n, tiles_m, splits);
  const bool pdl = a->use_pdl != 0;
  int stages = 0;
  int rc = -7;
#define ORTB200_LAUNCH(BN_, ST_)                                                        \
  do {                                                                                  \
    stages = ST_;                                                                       \
    rc = dual ? launch_gemm<BN_, (ST_ * (16384 * 2 + BN_ * 128) <= 200 * 1024 ? ST_ : ST_ / 2), true>(tw, tx, p, grid, stream, pdl) \
              : launch_gemm<BN_, ST_, false>(tw, tx, p, grid, stream, pdl);             \
  } while (0)
  switch (bn) {
    case 16: ORTB200_LAUNCH(16, 6); break;
    case 32: ORTB200_LAUNCH(32, 6); break;
    case 64: ORTB200_LAUNCH(64, 6); break;
    case 128: ORTB200_LAUNCH(128, 6); break;
    case 256:
      stages = 4;
      rc = launch_gemm<256, 4, false>(tw, tx, p, grid, stream, pdl);
      break;
    default: return -8;
  }
#undef ORTB200_LAUNCH
  g_last_config = {bn, splits, stages};
  return rc;
}
