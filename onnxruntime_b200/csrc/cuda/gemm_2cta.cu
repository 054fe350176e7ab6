// Large-M GEMM on pairs of SMs (tcgen05 cta_group::2) for sm_100a.
//
//   out[M, N] = act(alpha * X[M,K] * W[N,K]^T + bias) + residual        (bf16 / fp16, fp32 accumulation)
//
// A cluster of two CTAs computes one 256 (weight rows) x 256 (tokens) tile.  Each CTA stages its own 128 weight
// rows (A operand) and 128 of the 256 token rows (its half of the B operand) with TMA; ONE thread of the leader CTA
// issues tcgen05.mma.cta_group::2, which reads A and B from the shared memory of both CTAs and accumulates each
// CTA's 128 x 256 half of the tile in that CTA's tensor memory.  Per 128 x 256 x 64 unit of math a CTA therefore
// moves 32 KB through its shared memory (TMA in) + 32 KB (operand reads) instead of 48 + 48 KB for a lone CTA, which
// is what bounds the single-CTA kernel in gemm_tcgen05.cu.
//
// Synchronisation (all mbarriers live at the same shared-memory offset in both CTAs):
//   full[s]        leader only   both producers' TMA bytes land on the LEADER's barrier (.cta_group::2 loads)
//   empty[s]       per CTA       tcgen05.commit multicast to both CTAs once the MMAs reading stage s are done
//   tmem_full[b]   per CTA       multicast commit: accumulator buffer b complete
//   tmem_empty[b]  leader only   256 arrivals: the epilogue threads of both CTAs (the peer arrives remotely)
// Every wait is bounded; a timeout sets the status word and the kernel drains and returns.
//
// Reference counterpart: cublasGemmEx behind onnxruntime/core/providers/cuda/math/matmul.cc.
#include <cuda.h>
#include <cuda_runtime.h>
#include "gemm_internal.h"
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"

namespace ortb200 {
namespace {

constexpr int kBM = 128;        // weight rows per CTA (256 per pair)
constexpr int kBNHalf = 128;    // token rows each CTA stages (256 per pair)
constexpr int kBN = 256;        // tokens per tile = accumulator columns
constexpr int kBK = 64;
constexpr int kStages = 5;
constexpr int kThreads = 320;   // TMA warp, MMA warp, 4 epilogue warps, 4 store helpers
constexpr int kStoreThreads = 256;

struct Gemm2Params {
  int M, N, K, num_kb;
  int tiles_m, tiles;  // tiles of 256 x 256; tile = tile_n * tiles_m + tile_m
  int dtype, act;
  float alpha;
  const float* alpha_dev;  // optional device scalar multiplied into alpha (fp8 operands with run-time scales)
  int in_fp8;              // 1: x and w hold e4m3 bytes; a stage then carries 128 K-elements and the MMAs run as kind::f8f6f4
  int k_per_block;         // K elements per pipeline stage: 64 (16-bit operands) or 128 (fp8)
  void* out;
  long long ldo;
  const void* bias;
  const void* residual;
  long long ldr;
  int* status;
  // grouped mode (mixture of experts): token tiles of up to 256 rows from a device-side list
  const int4* tile_info;   // {expert, first row, end row, -}; null = ordinary GEMM
  const int* num_tiles;
  int tiles_n;             // 256-row weight tiles per expert
  int w_rows_per_expert;
  // tensor parallelism (world > 1): the epilogue pushes the product into the all-reduce scatter areas of the symmetric
  // workspace instead of `out` (see scatter_pass); the reduction kernel that follows finishes the sum
  int world, rank;
  void* peers[8];
  long long region_offset, half_bytes;
  unsigned int row_vecs;
};

struct Smem2 {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBNHalf * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStageBytes * kStages;
  static constexpr int kStagingOffset = kBarOffset + 256;
  static constexpr int kStagingBytes = 128 * kBM * 2;
  static constexpr int kTotal = kStagingOffset + kStagingBytes + 1024;
  static constexpr int kTmemCols = 512;  // two accumulator buffers of 256 columns
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load whose completion bytes are counted on a barrier given as a shared::cluster address (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once the MMAs issued so far are done) on the barrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 0x3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}


// Where this launch's products go when the GEMM feeds an all-reduce: the scatter area of the parity that the reduction
// kernel launched right after this one will use (it reads the same epoch word; the previous reduction has completed).
__device__ __forceinline__ ScatterArgs make_scatter_args(const Gemm2Params& p) {
  ScatterArgs sc{};
  if (p.world > 1) {
    const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(static_cast<uint8_t*>(p.peers[p.rank]) + 64) + 1;
    for (int i = 0; i < 8; ++i) sc.peers[i] = p.peers[i];
    sc.area_offset = p.region_offset + static_cast<long long>(epoch & 1) * p.half_bytes;
    sc.row_vecs = p.row_vecs;
    sc.rank = p.rank;
    sc.N = p.N;
  }
  return sc;
}

// FP8 is a compile-time switch: as a run-time branch inside the MMA loop it cost the 16-bit path a quarter of its
// speed (8192 x 6144 x 4096 bf16: 410 us against 312 us).
template <bool FP8>
__global__ void __launch_bounds__(kThreads, 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const Gemm2Params p) {
  constexpr int kKPerBlock = FP8 ? 2 * kBK : kBK;  // K elements per pipeline stage (a stage row is 128 bytes)
  using S = Smem2;
  extern __shared__ uint8_t smem_raw[];
  // the same rounding in both CTAs (the dynamic shared-memory window starts at the same offset in every CTA)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();         // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full_bar[i], 1);
      mbar_init(&tmem_empty_bar[i], 256);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, S::kTmemCols);
    tmem_relinquish2();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync();  // barriers of both CTAs initialised before anyone signals across
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait_prior_grids();

  // grouped mode: the number of token tiles is a device-side value written by the routing kernels
  const bool grouped = p.tile_info != nullptr;
  const int tiles_m = grouped ? *p.num_tiles : p.tiles_m;
  const int tiles = grouped ? p.tiles_n * tiles_m : p.tiles;

  if (warp == 0) {
    if (lane == 0) {
      // producer of this CTA: its 128 weight rows and its 128 token rows of every k-block; bytes are counted on the
      // leader's full barrier
      long long it = 0;
      bool ok = true;
      for (int t = pair; t < tiles && ok; t += num_pairs) {
        int n0 = (t / tiles_m) * (2 * kBM) + static_cast<int>(rank) * kBM;
        int m0 = (t % tiles_m) * kBN + static_cast<int>(rank) * kBNHalf;
        if (grouped) {
          const int4 ti = p.tile_info[t % tiles_m];
          n0 += ti.x * p.w_rows_per_expert;
          m0 = ti.y + static_cast<int>(rank) * kBNHalf;
        }
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = static_cast<int>(it % kStages);
          if (it >= kStages && !mbar_wait(&empty_bar[s], static_cast<uint32_t>((it / kStages) - 1) & 1)) {
            ok = false;
            break;
          }
          uint8_t* st = smem + s * S::kStageBytes;
          const uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);
          if (leader) mbar_expect_tx(&full_bar[s], 2 * S::kStageBytes);
          tma_load_2d_pair(st, &tmap_w, bar, kb * kKPerBlock, n0);
          tma_load_2d_pair(st + S::kABytes, &tmap_x, bar, kb * kKPerBlock, m0);
        }
      }
      if (!ok && p.status) atomicExch(p.status, kStatusTimeoutProducer);
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      const uint32_t idesc = FP8 ? umma_idesc_e4m3(2 * kBM, kBN) : umma_idesc_f16(p.dtype == ORTB200_BF16, 2 * kBM, kBN);
      long long it = 0;
      int seg = 0;
      bool ok = true;
      for (int t = pair; t < tiles && ok; t += num_pairs, ++seg) {
        const int buf = seg & 1;
        const uint32_t tmem_d = tmem_base + buf * kBN;
        if (seg >= 2 && !mbar_wait(&tmem_empty_bar[buf], ((seg >> 1) - 1) & 1)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = static_cast<int>(it % kStages);
          if (!mbar_wait(&full_bar[s], static_cast<uint32_t>(it / kStages) & 1)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * S::kStageBytes);
          const uint64_t adesc = umma_desc_sw128(a_addr);
          const uint64_t bdesc = umma_desc_sw128(a_addr + S::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {  // 32 bytes of K per instruction: 16 16-bit or 32 8-bit elements
            if (FP8) umma2_f8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma2_f16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty_bar[s]);
        }
        umma2_commit_both(&tmem_full_bar[buf]);  // also after a failed wait, so the epilogues do not wait for nothing
      }
      if (!ok && p.status) atomicExch(p.status, kStatusTimeoutMma);
    }
  } else if (warp >= 6) {
    // ---------------------------------------------------------------- store helpers: they take half of every store pass
    // (activation + residual + global stores of the staged tile), which the four epilogue warps alone could not
    // finish within one main loop when the epilogue carries a GELU
    const int et = static_cast<int>(threadIdx.x) - 64;   // 128 .. 255
    const uint16_t* stg = reinterpret_cast<const uint16_t*>(smem + S::kStagingOffset);
    const bool bf16 = p.dtype == ORTB200_BF16;
    const bool vec_ok = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (p.residual == nullptr || ((p.ldr % 8 == 0) && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
    const StoreArgs sa{p.out, p.residual, p.ldo, p.ldr, p.N};
    const ScatterArgs sc = make_scatter_args(p);
    for (int t = pair; t < tiles; t += num_pairs) {
      const int nrow0 = (t / tiles_m) * (2 * kBM) + static_cast<int>(rank) * kBM;
      int m0 = (t % tiles_m) * kBN, m_end = p.M;
      if (grouped) {
        const int4 ti = p.tile_info[t % tiles_m];
        m0 = ti.y;
        m_end = ti.z;
      }
#pragma unroll 1
      for (int pc = 0; pc < kBN; pc += 128) {
        asm volatile("bar.sync 1, 256;" ::: "memory");   // the pass is staged
        if (p.world > 1) {
          scatter_pass<kStoreThreads>(sc, stg, 128, et, m0 + pc, m_end, nrow0);
        } else if (p.act == ORTB200_ACT_NONE) {
          if (bf16) store_pass<true, ORTB200_ACT_NONE, kStoreThreads>(sa, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
          else store_pass<false, ORTB200_ACT_NONE, kStoreThreads>(sa, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
        } else if (bf16) {
          store_pass_act<true, kStoreThreads>(sa, p.act, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
        } else {
          store_pass_act<false, kStoreThreads>(sa, p.act, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");   // the staging tile may be overwritten
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: this CTA's 128 weight rows x 256 tokens
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int et = static_cast<int>(threadIdx.x) - 64;
    uint16_t* stg = reinterpret_cast<uint16_t*>(smem + S::kStagingOffset);
    const bool bf16 = p.dtype == ORTB200_BF16;
    const bool vec_ok = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (p.residual == nullptr || ((p.ldr % 8 == 0) && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
    const StoreArgs sa{p.out, p.residual, p.ldo, p.ldr, p.N};
    const ScatterArgs sc = make_scatter_args(p);
    const uint32_t empty_remote0 = map_to_rank(smem_u32(&tmem_empty_bar[0]), 0);
    const uint32_t empty_remote1 = map_to_rank(smem_u32(&tmem_empty_bar[1]), 0);
    int seg = 0;
    bool ok = true;
    const float alpha_v = p.alpha_dev ? p.alpha * __ldg(p.alpha_dev) : p.alpha;
    // a wait that gives up clears `ok`; the loop still runs to its end so that the store helpers, which count the same
    // barriers, never wait for nothing
    for (int t = pair; t < tiles; t += num_pairs, ++seg) {
      const int buf = seg & 1;
      const int nrow0 = (t / tiles_m) * (2 * kBM) + static_cast<int>(rank) * kBM;
      int m0 = (t % tiles_m) * kBN, m_end = p.M, bias0 = 0;
      if (grouped) {
        const int4 ti = p.tile_info[t % tiles_m];
        m0 = ti.y;
        m_end = ti.z;
        bias0 = ti.x * p.N;
      }
      const int n = nrow0 + r;
      const uint32_t t_lane = tmem_base + buf * kBN + (static_cast<uint32_t>(q * 32) << 16);
      if (ok && !mbar_wait(&tmem_full_bar[buf], (seg >> 1) & 1)) {
        ok = false;
        if (p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
      }
      tcgen05_fence_after();
      const float bias_v = (p.bias != nullptr && n < p.N)
                               ? (bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[bias0 + n])
                                       : __half2float(reinterpret_cast<const __half*>(p.bias)[bias0 + n]))
                               : 0.0f;
#pragma unroll 1
      for (int pc = 0; pc < kBN; pc += 128) {
        float v[128];
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) tmem_ld_x32(t_lane + pc + g4 * 32, v + g4 * 32);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 128; ++j) {
          const float y = v[j] * alpha_v + bias_v;
          uint16_t bits;
          if (bf16) {
            const __nv_bfloat16 h = __float2bfloat16_rn(y);
            bits = *reinterpret_cast<const uint16_t*>(&h);
          } else {
            const __half h = __float2half_rn(y);
            bits = *reinterpret_cast<const uint16_t*>(&h);
          }
          stg[j * kBM + r] = bits;
        }
        if (pc + 128 >= kBN) {
          // accumulator read completely: tell the leader's MMA warp (it counts the threads of both CTAs)
          tcgen05_fence_before();
          mbar_arrive_cluster(buf == 0 ? empty_remote0 : empty_remote1);
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // activation and type are compile-time constants inside the loop (a runtime switch per element tripled its
        // instruction count: 11 M -> 27 M warp instructions for a plain ReLU on 8192 x 4096 x 1024)
        // (the plain path stays inline: an out-of-line call cost it a quarter of its speed)
        if (p.world > 1) {
          scatter_pass<kStoreThreads>(sc, stg, 128, et, m0 + pc, m_end, nrow0);
        } else if (p.act == ORTB200_ACT_NONE) {
          if (bf16) store_pass<true, ORTB200_ACT_NONE, kStoreThreads>(sa, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
          else store_pass<false, ORTB200_ACT_NONE, kStoreThreads>(sa, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
        } else if (bf16) {
          store_pass_act<true, kStoreThreads>(sa, p.act, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
        } else {
          store_pass_act<false, kStoreThreads>(sa, p.act, stg, 128, et, m0 + pc, m_end, nrow0, vec_ok);
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
    }
  }

  // nobody leaves (or frees tensor memory) while the peer may still be reading this CTA's shared memory
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc2(tmem_base, S::kTmemCols);
  }
}

}  // namespace

int launch_gemm_2cta(const ortb200_gemm_args* a, cudaStream_t stream) {
  const bool fp8 = a->in_dtype == ORTB200_F8E4M3;
  if (a->act == ORTB200_ACT_SWIGLU || (a->in_dtype != 0 && !fp8) || a->rms_eps > 0.f) return -16;
  if (fp8 && (a->world > 1 || a->K % 16 != 0)) return -16;
  if (a->alpha_dev != nullptr && !fp8) return -16;
  if (a->world > 1 && (a->act != ORTB200_ACT_NONE || a->ldo != a->N || a->N % 8 != 0 || a->world > 8)) return -12;
  CUtensorMap tw, tx;
  const int k_per_block = fp8 ? 2 * kBK : kBK;   // a stage row is 128 bytes either way
  if (fp8) {
    if (make_tensor_map_2d(&tw, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->K, a->w_rows, a->K, k_per_block, kBM) != 0) return -6;
    if (make_tensor_map_2d(&tx, a->x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->K, a->M, a->K, k_per_block, kBNHalf) != 0) return -6;
  } else {
    const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, a->w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) return -6;
    if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->M, static_cast<int64_t>(a->K) * 2, kBK, kBNHalf) != 0) return -6;
  }
  Gemm2Params p;
  p.M = a->M; p.N = a->N; p.K = a->K; p.num_kb = (a->K + k_per_block - 1) / k_per_block;
  p.in_fp8 = fp8 ? 1 : 0; p.k_per_block = k_per_block; p.alpha_dev = a->alpha_dev;
  const int tiles_n = (a->N + 2 * kBM - 1) / (2 * kBM);
  p.tiles_m = (a->M + kBN - 1) / kBN;
  p.tiles = tiles_n * p.tiles_m;
  p.dtype = a->dtype; p.act = a->act; p.alpha = a->alpha; p.out = a->out; p.ldo = a->ldo; p.bias = a->bias;
  p.residual = a->residual; p.ldr = a->ldr; p.status = a->status;
  p.tile_info = nullptr; p.num_tiles = nullptr; p.tiles_n = 0; p.w_rows_per_expert = 0;
  p.world = 1; p.rank = 0; p.region_offset = 0; p.half_bytes = 0; p.row_vecs = 1;
  for (int i = 0; i < 8; ++i) p.peers[i] = nullptr;
  if (a->world > 1) {
    const long long total_vecs = static_cast<long long>(a->M) * a->N / 8;
    if (static_cast<long long>(a->M) * a->N * 2 > ortb200_symm_collective_max_bytes(ORTB200_COLL_ALLREDUCE, a->world, a->symm_bytes)) return -13;
    p.world = a->world; p.rank = a->rank;
    for (int i = 0; i < a->world; ++i) {
      if (!a->peers[i]) return -12;
      p.peers[i] = a->peers[i];
    }
    p.region_offset = a->symm_bytes / 2;
    p.half_bytes = a->symm_bytes / 4;
    p.row_vecs = static_cast<unsigned int>((total_vecs + a->world - 1) / a->world);
    p.out = nullptr; p.residual = nullptr;     // the reduction kernel applies the residual and writes `out`
    if (a->rank != 0) p.bias = nullptr;        // the bias enters the sum once
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int pairs = sms / 2;
  if (pairs > p.tiles) pairs = p.tiles;
  if (pairs < 1) return -1;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_2cta_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2::kTotal) != cudaSuccess) return -10;
    if (cudaFuncSetAttribute(gemm_2cta_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2::kTotal) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Smem2::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  int nattr = 1;
  if (a->use_pdl) {
    attrs[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = nattr;
  if (cudaLaunchKernelEx(&cfg, fp8 ? gemm_2cta_kernel<true> : gemm_2cta_kernel<false>, tw, tx, p) != cudaSuccess) return -11;
  return a->world > 1 ? launch_allreduce_prescattered(a, stream) : 0;
}

// Grouped GEMM (mixture of experts) on CTA pairs: 256-token tiles from the device-side tile list.
int launch_gemm_grouped_2cta(const ortb200_gemm_grouped_args* a, cudaStream_t stream) {
  if (a->act == ORTB200_ACT_SWIGLU || a->tile_rows != 256) return -16;
  CUtensorMap tw, tx;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int64_t w_rows = static_cast<int64_t>(a->num_experts) * a->w_rows_per_expert;
  if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) return -6;
  if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->rows, static_cast<int64_t>(a->K) * 2, kBK, kBNHalf) != 0) return -6;
  Gemm2Params p;
  p.M = a->rows; p.N = a->N; p.K = a->K; p.num_kb = (a->K + kBK - 1) / kBK;
  p.in_fp8 = 0; p.k_per_block = kBK; p.alpha_dev = nullptr;
  p.tiles_m = 0; p.tiles = 0;
  p.dtype = a->dtype; p.act = a->act; p.alpha = 1.0f; p.out = a->out; p.ldo = a->N; p.bias = a->bias;
  p.residual = nullptr; p.ldr = 0; p.status = a->status;
  p.tile_info = static_cast<const int4*>(a->tile_info);
  p.num_tiles = a->num_tiles;
  p.tiles_n = (a->N + 2 * kBM - 1) / (2 * kBM);
  p.w_rows_per_expert = a->w_rows_per_expert;
  p.world = 1; p.rank = 0; p.region_offset = 0; p.half_bytes = 0; p.row_vecs = 1;
  for (int i = 0; i < 8; ++i) p.peers[i] = nullptr;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int pairs = sms / 2;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_2cta_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2::kTotal) != cudaSuccess) return -10;
    if (cudaFuncSetAttribute(gemm_2cta_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2::kTotal) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Smem2::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_2cta_kernel<false>, tw, tx, p) == cudaSuccess ? 0 : -11;
}

}  // namespace ortb200
