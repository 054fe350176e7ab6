// Dense GEMM for sm_100a: TMA-fed tcgen05.mma with the accumulator in tensor
// memory.  out[M, N] = act(alpha * X[M,K] * W[N,K]^T + bias) + residual.
//
// Replaces the cuBLAS calls of the reference's MatMul/Gemm/FusedMatMul kernels
// (onnxruntime/core/providers/cuda/math/matmul.cc:180-419) and the QKV
// projection inside Attention (onnxruntime/contrib_ops/cuda/bert/attention.cc:251).
//
// Orientation: the WEIGHT tile is the MMA's A operand (128 rows = 128 TMEM
// lanes), the token tile is the B operand (BN = 16..256 columns).  A decode
// step with 8 tokens therefore wastes no tensor-core rows on padding and W is
// streamed exactly once.
//
// The kernel is persistent: one CTA per SM walks a contiguous range of
// (tile, k-block) work units, so the TMA pipeline never drains between tiles
// and two TMEM accumulator buffers let the epilogue of one tile overlap the
// main loop of the next.  With many tiles every CTA owns whole tiles; with few
// (decode) the units are dealt out evenly (stream-K): a tile shared by several
// CTAs is reduced through an fp32 workspace by the CTA that arrives last on a
// per-tile counter, in a fixed order (deterministic).  No host round trip, no
// second launch.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer (one elected lane), warps 2..5 = epilogue (one TMEM lane quarter each).
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include <unordered_map>
#include <stdio.h>
#include "gemm_internal.h"
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
  int tiles;          // tiles_n * tiles_m
  int tiles_m;        // tile index = tile_n * tiles_m + tile_m
  int tile_aligned;   // 1: every CTA owns whole tiles; 0: stream-K over (tile, k-block) units
  int max_contrib;    // workspace slots per tile in stream-K mode
  int dual_offset;
  int dtype;
  int in_fp8;         // 1: x and w are e4m3 bytes (a stage then holds 128 K-elements instead of 64)
  int k_per_block;    // K elements per pipeline stage: 64 (16-bit operands) or 128 (fp8)
  int act;
  float alpha;
  const float* alpha_dev;  // optional device scalar multiplied into alpha (runtime scales: no host read)
  void* out;
  long long ldo;
  const void* bias;
  const void* residual;
  long long ldr;
  float* ws;
  unsigned int* counters;
  int* status;
  // grouped mode (mixture of experts): the token tiles come from a device-side list built by the routing kernels
  const int4* tile_info;   // {expert, first row, end row, -}; null = ordinary GEMM
  const int* num_tiles;    // device scalar: token tiles in use
  int tiles_n;             // weight-row tiles per expert
  int w_rows_per_expert;
  // all-gather fused into the GEMM (gather kernels only; see ortb200_allgather_gemm): x is sharded by rows over the
  // ranks, every rank pushes its shard into the peers' gather areas while its own tiles already run
  int gather_world, gather_rank;
  int gather_rows;                 // rows of x per rank
  int gather_tiles_per_shard;      // token tiles per shard (ceil(gather_rows / BN))
  void* gather_peers[8];           // bases of the symmetric workspaces
  long long gather_area_offset;    // bytes from a workspace base to its gather area of parity 0
  long long gather_half_bytes;     // distance between the areas of the two parities
  const void* gather_x_local;      // this rank's shard [gather_rows, K]
};

constexpr long long kGatherFlagsOffset = 65536;   // flags[src rank < 8][4096] uint32 of the symmetric workspace header
constexpr int kGatherFlagSlot = 4095;             // the slot of a source rank that the gather kernels use
constexpr unsigned int kGatherSpinLimit = 1u << 19;
constexpr int kGatherThreads = 320;               // the six warps of the plain kernel + four that push the local shard

__device__ __forceinline__ float apply_act(int act, float v) {
  switch (act) {
    case ORTB200_ACT_GELU: return gelu_erf_fast(v);
    case ORTB200_ACT_FASTGELU: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
    case ORTB200_ACT_RELU: return fmaxf(v, 0.0f);
    case ORTB200_ACT_SILU: return v / (1.0f + __expf(-v));
    case ORTB200_ACT_QUICKGELU: return v / (1.0f + __expf(-1.702f * v));
    default: return v;
  }
}

// DUAL: two weight tiles (gate rows, up rows) share the activation tile and are combined by the SwiGLU epilogue.
// TWOM: two vertically adjacent weight tiles share the activation tile, i.e. the CTA tile is 256 weight rows x BN
// tokens.  Per k-block the CTA then loads 32 KiB of W and 2 * BN * 64 bytes of X for twice the math, which is what
// keeps a large GEMM from being bound by L2 -> SM bandwidth (131 instead of 85 FLOP per loaded byte at BN = 256).
template <int BN, int STAGES, bool DUAL, bool TWOM = false>
struct GemmSmem {
  static constexpr bool kTwoA = DUAL || TWOM;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes * (kTwoA ? 2 : 1) + kBBytes;
  static constexpr int kBarOffset = kStageBytes * STAGES;
  // epilogue staging: up to 128 token columns x 128 weight rows of 16-bit results, so that global memory is written
  // (and the residual read) with 16-byte accesses along the output rows
  static constexpr int kPassCols = BN < 128 ? BN : 128;
  static constexpr int kStagingOffset = kBarOffset + 256;
  static constexpr int kStagingBytes = kPassCols * kBM * 2;
  static constexpr int kTotal = kStagingOffset + kStagingBytes + 1024;          // + alignment slack
  static_assert(8 * (2 * STAGES + 4) + 16 <= 256, "barrier area");
  static constexpr int kCols = (kTwoA ? 2 : 1) * BN;                            // accumulator columns per buffer
  static constexpr int kBufCols = kCols < 32 ? 32 : kCols;
  static constexpr int kNumBufs = 2 * kBufCols <= 512 ? 2 : 1;                   // accumulator buffers that fit in TMEM
  static constexpr int kTmemCols = kNumBufs * kBufCols;
  static constexpr int kTileRows = TWOM ? 2 * kBM : kBM;                         // weight rows per CTA tile
};

// Work decomposition shared by the three warp roles.  Units are (tile, k-block) pairs numbered tile-major;
// CTA c owns units [c * U / G, (c + 1) * U / G), or whole tiles when `tile_aligned`.
struct WorkRange {
  long long begin, end;
};
__device__ __forceinline__ WorkRange cta_range(const GemmKernelParams& p, int c, long long tiles) {
  const long long G = gridDim.x;
  WorkRange r;
  if (p.tile_aligned) {
    r.begin = (static_cast<long long>(c) * tiles / G) * p.num_kb;
    r.end = (static_cast<long long>(c + 1) * tiles / G) * p.num_kb;
  } else {
    const long long U = static_cast<long long>(p.tiles) * p.num_kb;
    r.begin = static_cast<long long>(c) * U / G;
    r.end = static_cast<long long>(c + 1) * U / G;
  }
  return r;
}
// CTA that owns unit u in stream-K mode
__device__ __forceinline__ int owner_of(const GemmKernelParams& p, long long u) {
  const long long U = static_cast<long long>(p.tiles) * p.num_kb;
  return static_cast<int>(((u + 1) * gridDim.x - 1) / U);
}

// Gather kernels: the t-th tile of CTA c is physical tile c + t * gridDim.x, and the physical tiles are numbered
// token-tile-major starting with the rank's own shard, so every CTA begins with rows that are already here while
// the other shards are still crossing NVLink.
struct GatherTile {
  int n0, m0, m_end, src, local;
};
template <int BN, int TILE_ROWS>
__device__ __forceinline__ GatherTile gather_tile(const GemmKernelParams& p, long long vtile) {
  const long long phys = blockIdx.x + vtile * gridDim.x;
  const int tile_n = static_cast<int>(phys % p.tiles_n), j = static_cast<int>(phys / p.tiles_n);
  GatherTile t;
  t.src = (p.gather_rank + j / p.gather_tiles_per_shard) % p.gather_world;
  t.local = (j % p.gather_tiles_per_shard) * BN;
  t.n0 = tile_n * TILE_ROWS;
  t.m0 = t.src * p.gather_rows + t.local;
  t.m_end = (t.src + 1) * p.gather_rows;
  return t;
}
__device__ __forceinline__ unsigned int gather_ld_acquire_sys(const unsigned int* q) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(q) : "memory");
  return v;
}
__device__ __forceinline__ void gather_st_release_sys(unsigned int* q, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(q), "r"(v) : "memory");
}

template <int BN, int STAGES, bool DUAL, bool TWOM, bool GATHER>
__device__ __forceinline__ void gemm_tcgen05_body(const CUtensorMap* tmap_w, const CUtensorMap* tmap_x, const CUtensorMap* tmap_g,
                                                  const GemmKernelParams& p) {
  using S = GemmSmem<BN, STAGES, DUAL, TWOM>;
  constexpr bool TWO_A = S::kTwoA;
  constexpr int NBUF = S::kNumBufs;
  const int second_a_rows = DUAL ? p.dual_offset : kBM;  // row distance between the two weight tiles of a stage
  static_assert((S::kTmemCols & (S::kTmemCols - 1)) == 0 && S::kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  uint32_t* last_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // grouped mode: the number of token tiles is only known on the device (and only after the routing kernels ran)
  const bool grouped = p.tile_info != nullptr;
  int tiles_m = p.tiles_m;
  long long tiles_total = p.tiles;
  if (grouped) {
    pdl_wait_prior_grids();
    tiles_m = *p.num_tiles;
    tiles_total = static_cast<long long>(p.tiles_n) * tiles_m;
  }
  WorkRange range = cta_range(p, blockIdx.x, tiles_total);
  if (GATHER) {
    const long long mine = static_cast<long long>(blockIdx.x) < tiles_total ? (tiles_total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    range.begin = 0;
    range.end = mine * p.num_kb;
  }
  // gather kernels: header of the local symmetric workspace (word 16: epoch of the collectives, 17: CTAs done,
  // 18: polling limit override, 20 .. 26: CTAs done with the copy to the d-th destination)
  unsigned int* const ghdr = GATHER ? reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(p.gather_peers[p.gather_rank]) + 64) : nullptr;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(tmap_w);
    tma_prefetch_desc(tmap_x);
    if (GATHER) tma_prefetch_desc(tmap_g);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full_bar[i], 1);
      mbar_init(&tmem_empty_bar[i], 128);
    }
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

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the previous kernel: fill the pipeline with W tiles first, then wait for
      // the producer of X, then add the X tiles.  `it` counts k-blocks across all segments of this CTA.
      const uint64_t pol_w = policy_evict_first();
      const long long total = range.end - range.begin;
      const int pre = total < STAGES ? static_cast<int>(total) : STAGES;
      long long total_limit = total;  // 0 once a wait for another rank has run out
      // gather kernels: where the token rows of a tile come from (own shard: the input itself; others: the gather area)
      int x_src = 0, x_local = 0;
      unsigned int ready = GATHER ? (1u << p.gather_rank) : 0u, g_epoch = 0;
      auto coords = [&](long long u, int* kb, int* n0, int* m0) {
        if (GATHER) {
          const GatherTile t = gather_tile<BN, S::kTileRows>(p, u / p.num_kb);
          *kb = static_cast<int>(u % p.num_kb);
          *n0 = t.n0;
          *m0 = t.m0;
          x_src = t.src;
          x_local = t.local;
          return;
        }
        const int tile = static_cast<int>(u / p.num_kb);
        *kb = static_cast<int>(u % p.num_kb);
        *n0 = (tile / tiles_m) * S::kTileRows;
        *m0 = (tile % tiles_m) * BN;
        if (grouped) {
          const int4 ti = p.tile_info[tile % tiles_m];
          *n0 += ti.x * p.w_rows_per_expert;  // this expert's rows of the stacked weight matrix
          *m0 = ti.y;
        }
      };
      // X tile of the current coords() into `dst`.  Rows of another rank are first waited for (once per source: that
      // rank's push raises one flag here when all of its shard has arrived), with a bounded wait.
      auto load_x = [&](uint8_t* dst, uint64_t* bar, int kb, int m0) -> bool {
        if (!GATHER) {
          tma_load_2d(dst, tmap_x, bar, kb * p.k_per_block, m0);
          return true;
        }
        if (x_src == p.gather_rank) {
          tma_load_2d(dst, tmap_x, bar, kb * p.k_per_block, x_local);
          return true;
        }
        if (!((ready >> x_src) & 1u)) {
          const unsigned int* f = reinterpret_cast<const unsigned int*>(static_cast<const uint8_t*>(p.gather_peers[p.gather_rank]) + kGatherFlagsOffset) +
                                  x_src * 4096 + kGatherFlagSlot;
          const unsigned int lim_override = *reinterpret_cast<const volatile unsigned int*>(ghdr + 2);
          const unsigned int limit = lim_override != 0 ? lim_override : kGatherSpinLimit;
          const unsigned int want = 2 * g_epoch + 1;
          unsigned int spins = 0;
          while (static_cast<int>(gather_ld_acquire_sys(f) - want) < 0) {
            if (++spins > limit) {
              if (p.status) atomicExch(p.status, kStatusTimeoutPeer);
              return false;
            }
            __nanosleep(128);
          }
          fence_proxy_async();  // the rows were written with generic stores (by the peer); the copy engine reads them
          ready |= 1u << x_src;
        }
        tma_load_3d(dst, tmap_g, bar, kb * p.k_per_block, m0, static_cast<int>(g_epoch & 1u));
        return true;
      };
      for (int i = 0; i < pre; ++i) {
        int kb, n0, m0;
        coords(range.begin + i, &kb, &n0, &m0);
        uint8_t* st = smem + i * S::kStageBytes;
        mbar_expect_tx(&full_bar[i], S::kStageBytes);
        tma_load_2d_hint(st, tmap_w, &full_bar[i], kb * p.k_per_block, n0, pol_w);
        if (TWO_A) tma_load_2d_hint(st + S::kABytes, tmap_w, &full_bar[i], kb * p.k_per_block, n0 + second_a_rows, pol_w);
      }
      pdl_wait_prior_grids();
      if (GATHER) g_epoch = *reinterpret_cast<const volatile unsigned int*>(ghdr) + 1;
      bool x_ok = true;
      for (int i = 0; i < pre && x_ok; ++i) {
        int kb, n0, m0;
        coords(range.begin + i, &kb, &n0, &m0);
        uint8_t* st = smem + i * S::kStageBytes;
        x_ok = load_x(st + S::kABytes * (TWO_A ? 2 : 1), &full_bar[i], kb, m0);
      }
      if (!x_ok) total_limit = 0;
      for (long long i = pre; i < total_limit; ++i) {
        const int s = static_cast<int>(i % STAGES);
        const uint32_t parity = static_cast<uint32_t>((i / STAGES) - 1) & 1;
        if (!mbar_wait(&empty_bar[s], parity)) {
          if (p.status) atomicExch(p.status, kStatusTimeoutProducer);
          break;
        }
        int kb, n0, m0;
        coords(range.begin + i, &kb, &n0, &m0);
        uint8_t* st = smem + s * S::kStageBytes;
        mbar_expect_tx(&full_bar[s], S::kStageBytes);
        tma_load_2d_hint(st, tmap_w, &full_bar[s], kb * p.k_per_block, n0, pol_w);
        if (TWO_A) tma_load_2d_hint(st + S::kABytes, tmap_w, &full_bar[s], kb * p.k_per_block, n0 + second_a_rows, pol_w);
        if (!load_x(st + S::kABytes * (TWO_A ? 2 : 1), &full_bar[s], kb, m0)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // the gather kernels are 16-bit only: no run-time format branch in their MMA loop
      const uint32_t idesc = (!GATHER && p.in_fp8) ? umma_idesc_e4m3(kBM, BN) : umma_idesc_f16(p.dtype == ORTB200_BF16, kBM, BN);
      long long it = 0;
      int seg = 0;
      bool ok = true;
      pdl_wait_prior_grids();  // the bounded waits below must not span the previous grid's run time
      for (long long u = range.begin; u < range.end && ok; ++seg) {
        const long long tile_end = (u / p.num_kb + 1) * p.num_kb;
        const long long seg_end = tile_end < range.end ? tile_end : range.end;
        const int buf = seg % NBUF;
        const uint32_t tmem_d = tmem_base + buf * S::kBufCols;
        if (seg >= NBUF && !mbar_wait(&tmem_empty_bar[buf], ((seg / NBUF) - 1) & 1)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        bool first = true;
        for (; u < seg_end; ++u, ++it) {
          const int s = static_cast<int>(it % STAGES);
          if (!mbar_wait(&full_bar[s], static_cast<uint32_t>(it / STAGES) & 1)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * S::kStageBytes);
          const uint32_t b_addr = a_addr + S::kABytes * (TWO_A ? 2 : 1);
          const uint64_t adesc = umma_desc_sw128(a_addr);
          const uint64_t bdesc = umma_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // 16 K-elements = 32 bytes: the start-address field advances by 2
            // one instruction covers 32 bytes of K in either format: 16 half-precision or 32 fp8 elements
            if (!GATHER && p.in_fp8) umma_f8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
            else umma_f16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
          }
          if (TWO_A) {
            const uint64_t a2desc = umma_desc_sw128(a_addr + S::kABytes);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              if (!GATHER && p.in_fp8) umma_f8(tmem_d + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
              else umma_f16(tmem_d + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
            }
          }
          first = false;
          umma_commit(&empty_bar[s]);  // stage is reusable once these MMAs have read it
        }
        umma_commit(&tmem_full_bar[buf]);  // accumulator of this segment complete (also signalled on the failure path)
      }
      if (!ok && p.status) atomicExch(p.status, kStatusTimeoutMma);
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------- epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;            // lane within the tile == weight row
    pdl_wait_prior_grids();                 // out / residual / workspace may belong to the previous kernel
    int seg = 0;
    bool ok = true;
    for (long long u = range.begin; u < range.end && ok; ++seg) {
      const int tile = static_cast<int>(u / p.num_kb);
      const long long tile_begin = static_cast<long long>(tile) * p.num_kb;
      const long long tile_end = tile_begin + p.num_kb;
      const long long seg_end = tile_end < range.end ? tile_end : range.end;
      const bool whole = (u == tile_begin) && (seg_end == tile_end);
      const int buf = seg % NBUF;
      int n0 = (tile / tiles_m) * S::kTileRows, m0 = (tile % tiles_m) * BN;
      int m_end = p.M, bias0 = 0;
      if (grouped) {
        const int4 ti = p.tile_info[tile % tiles_m];
        m0 = ti.y;
        m_end = ti.z;
        bias0 = ti.x * p.N;
      }
      if (GATHER) {
        const GatherTile t = gather_tile<BN, S::kTileRows>(p, tile);
        n0 = t.n0;
        m0 = t.m0;
        m_end = t.m_end;
      }
      const uint32_t t_lane = tmem_base + buf * S::kBufCols + (static_cast<uint32_t>(q * 32) << 16);
      if (!mbar_wait(&tmem_full_bar[buf], (seg / NBUF) & 1)) {
        ok = false;
        if (p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
        break;
      }
      tcgen05_fence_after();

      bool do_output = true;
      int n_contrib = 1, first_owner = 0;
      if (!whole) {
        // 1) publish this CTA's partial tile; slot = position of this CTA among the tile's contributors
        first_owner = owner_of(p, tile_begin);
        n_contrib = owner_of(p, tile_end - 1) - first_owner + 1;
        const int slot = static_cast<int>(blockIdx.x) - first_owner;
        float* my_ws = p.ws + (static_cast<size_t>(tile) * p.max_contrib + slot) * (S::kCols * kBM);
#pragma unroll 1
        for (int c = 0; c < S::kCols; c += 16) {
          float v[16];
          tmem_ld_x16(t_lane + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) my_ws[(c + j) * kBM + r] = v[j];
        }
        tcgen05_fence_before();
        mbar_arrive(&tmem_empty_bar[buf]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const unsigned int old = atomicAdd(&p.counters[tile], 1u);
          const unsigned int last = (old == static_cast<unsigned int>(n_contrib - 1)) ? 1u : 0u;
          if (last) p.counters[tile] = 0;  // re-arm for the next launch (graph replay safe)
          *last_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        do_output = (*last_flag != 0);
        if (do_output) __threadfence();
      }

      if (whole) {
        // ---- whole tile: accumulator -> (bias, activation) -> 16-bit staging tile in shared memory -> coalesced
        // 16-byte global writes with the residual added on the way out
        constexpr int PASS = S::kPassCols;
        constexpr int LD = PASS >= 32 ? 32 : 16;
        uint16_t* stg = reinterpret_cast<uint16_t*>(smem + S::kStagingOffset);
        const int et = static_cast<int>(threadIdx.x) - 64;  // 0..127 among the epilogue threads
        const bool bf16 = p.dtype == ORTB200_BF16;
        const bool vec_ok = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                            (p.residual == nullptr || ((p.ldr % 8 == 0) && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
#pragma unroll 1
        for (int half = 0; half < (TWOM ? 2 : 1); ++half) {
          const int nrow0 = n0 + half * kBM;
          const int n = nrow0 + r;
          const float alpha_v = p.alpha_dev ? p.alpha * __ldg(p.alpha_dev) : p.alpha;
          const float bias_v = (p.bias != nullptr && n < p.N)
                                   ? (bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[bias0 + n])
                                           : __half2float(reinterpret_cast<const __half*>(p.bias)[bias0 + n]))
                                   : 0.0f;
#pragma unroll 1
          for (int pc = 0; pc < BN; pc += PASS) {
            // A tensor-memory load issued while the MMAs of the next tile run takes on the order of a microsecond, so
            // the loads of a whole group of columns go out back to back and are waited for once.
            constexpr int GC = (DUAL ? 64 : 128) < PASS ? (DUAL ? 64 : 128) : PASS;
#pragma unroll 1
            for (int c = 0; c < PASS; c += GC) {
              float v[GC];
              float uu[DUAL ? GC : 1];
#pragma unroll
              for (int g4 = 0; g4 < GC / LD; ++g4) {
                if (LD == 32) {
                  tmem_ld_x32(t_lane + half * BN + pc + c + g4 * LD, v + g4 * LD);
                  if (DUAL) tmem_ld_x32(t_lane + BN + pc + c + g4 * LD, uu + g4 * LD);
                } else {
                  tmem_ld_x16(t_lane + half * BN + pc + c + g4 * LD, v + g4 * LD);
                  if (DUAL) tmem_ld_x16(t_lane + BN + pc + c + g4 * LD, uu + g4 * LD);
                }
              }
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < GC; ++j) {
                // no activation switch in this fully unrolled loop (it would be copied GC times): activations other
                // than the gated one are applied on the way out, on the 16-bit value, as a separate op would
                float y = v[j] * alpha_v + bias_v;
                if (DUAL) {
                  const float g = y / (1.0f + __expf(-y));
                  y = g * (uu[j] * alpha_v);
                }
                uint16_t bits;
                if (bf16) {
                  const __nv_bfloat16 h = __float2bfloat16_rn(y);
                  bits = *reinterpret_cast<const uint16_t*>(&h);
                } else {
                  const __half h = __float2half_rn(y);
                  bits = *reinterpret_cast<const uint16_t*>(&h);
                }
                stg[(c + j) * kBM + r] = bits;
              }
            }
            if (half == (TWOM ? 1 : 0) && pc + PASS >= BN) {
              // the accumulator has been read completely: the MMA warp may reuse this buffer
              tcgen05_fence_before();
              mbar_arrive(&tmem_empty_bar[buf]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            {
              // activation and type are compile-time constants inside the store loop (shared with the CTA-pair kernel)
              const StoreArgs sa{p.out, p.residual, p.ldo, p.ldr, p.N};
              const int act = DUAL ? ORTB200_ACT_NONE : p.act;
              if (act == ORTB200_ACT_NONE) {
                if (bf16) store_pass<true, ORTB200_ACT_NONE, 128>(sa, stg, PASS, et, m0 + pc, m_end, nrow0, vec_ok);
                else store_pass<false, ORTB200_ACT_NONE, 128>(sa, stg, PASS, et, m0 + pc, m_end, nrow0, vec_ok);
              } else if (bf16) {
                store_pass_act<true, 128>(sa, act, stg, PASS, et, m0 + pc, m_end, nrow0, vec_ok);
              } else {
                store_pass_act<false, 128>(sa, act, stg, PASS, et, m0 + pc, m_end, nrow0, vec_ok);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // staging is free again
          }
        }
        u = seg_end;
        continue;
      }

      if (do_output) {
        const float* tile_ws = whole ? nullptr : p.ws + static_cast<size_t>(tile) * p.max_contrib * (S::kCols * kBM);
#pragma unroll 1
        for (int half = 0; half < (TWOM ? 2 : 1); ++half) {
          const int n = n0 + half * kBM + r;  // weight row == output column of this lane
          const bool n_ok = n < p.N;
          const int c_off = half * BN;        // accumulator columns of this half
          const float alpha_v = p.alpha_dev ? p.alpha * __ldg(p.alpha_dev) : p.alpha;
          const float bias_v = (p.bias != nullptr && n_ok)
                                   ? (p.dtype == ORTB200_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n])
                                                              : __half2float(reinterpret_cast<const __half*>(p.bias)[n]))
                                   : 0.0f;
#pragma unroll 1
          for (int c = 0; c < BN; c += 16) {
            // residual values first: 16 independent loads in flight while the accumulator is fetched (issued one by
            // one between the stores they would otherwise be serialised, since `out` may alias `residual`)
            float rv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) rv[j] = 0.0f;
            if (p.residual != nullptr && n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c + j;
                if (m < p.M) {
                  const long long idx = static_cast<long long>(m) * p.ldr + n;
                  rv[j] = p.dtype == ORTB200_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[idx])
                                                  : __half2float(reinterpret_cast<const __half*>(p.residual)[idx]);
                }
              }
            }
            float v[16];
            float uu[16];
            if (whole) {
              tmem_ld_x16(t_lane + c_off + c, v);
              if (DUAL) tmem_ld_x16(t_lane + BN + c, uu);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) { v[j] = 0.0f; uu[j] = 0.0f; }
              for (int s = 0; s < n_contrib; ++s) {
                const float* src = tile_ws + static_cast<size_t>(s) * (S::kCols * kBM);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  v[j] += __ldcg(&src[(c_off + c + j) * kBM + r]);
                  if (DUAL) uu[j] += __ldcg(&src[(BN + c + j) * kBM + r]);
                }
              }
            }
            if (n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c + j;
                if (m < p.M) {
                  float y = v[j] * alpha_v + bias_v;
                  if (DUAL) {
                    const float g = y / (1.0f + __expf(-y));
                    y = g * (uu[j] * alpha_v);
                  } else {
                    y = apply_act(p.act, y);
                  }
                  y += rv[j];
                  const long long o = static_cast<long long>(m) * p.ldo + n;
                  if (p.dtype == ORTB200_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(y);
                  else reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(y);
                }
              }
            }
          }
        }
      }
      u = seg_end;
    }
  } else if (GATHER) {
    // ---------------------------------------------------------- push (gather kernels: warps 6..9)
    // This rank's shard goes into every other rank's gather area with 16-byte peer stores, one grid-strided share per
    // CTA, while the other warps already work on the shard.  Rank r reaches the shard of rank r + d as its d-th, so
    // the copies go out nearest consumer first (to rank - 1, then rank - 2, ...) and each destination gets its flag
    // as soon as its copy is complete: stores, system-wide fence, a local counter per destination; the CTA that
    // completes a copy fences again and releases this rank's flag on that destination.
    pdl_wait_prior_grids();
    const unsigned int epoch = *reinterpret_cast<const volatile unsigned int*>(ghdr) + 1;
    const int pt = static_cast<int>(threadIdx.x) - 192;
    const long long shard_bytes = static_cast<long long>(p.gather_rows) * p.K * 2;
    const long long vecs = shard_bytes / 16;
    const long long area = p.gather_area_offset + static_cast<long long>(epoch & 1u) * p.gather_half_bytes + p.gather_rank * shard_bytes;
    const uint4* src = static_cast<const uint4*>(p.gather_x_local);
    for (int d = 1; d < p.gather_world; ++d) {
      const int dst = (p.gather_rank - d + p.gather_world) % p.gather_world;
      uint4* to = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.gather_peers[dst]) + area);
      // four loads in flight per thread: with one, the copy runs at a fraction of the link's rate
      const long long step = static_cast<long long>(gridDim.x) * 128;
      for (long long i = static_cast<long long>(blockIdx.x) * 128 + pt; i < vecs; i += 4 * step) {
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (i + k * step < vecs) v[k] = __ldg(src + i + k * step);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (i + k * step < vecs) to[i + k * step] = v[k];
      }
      __threadfence_system();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (pt == 0) {
        unsigned int* counter = ghdr + 3 + d;   // words 20 .. 26 of the workspace header: CTAs done with copy d
        if (atomicAdd(counter, 1u) == gridDim.x - 1) {
          *counter = 0;
          __threadfence_system();
          unsigned int* f = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(p.gather_peers[dst]) + kGatherFlagsOffset) +
                            p.gather_rank * 4096 + kGatherFlagSlot;
          gather_st_release_sys(f, 2 * epoch + 1);
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
  if (GATHER && threadIdx.x == 0) {
    // the CTA that finishes last closes the epoch (every CTA has read it by then)
    const unsigned int epoch = *reinterpret_cast<const volatile unsigned int*>(ghdr) + 1;
    if (atomicAdd(ghdr + 1, 1u) == gridDim.x - 1) {
      ghdr[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(ghdr) = epoch;
    }
  }
}

template <int BN, int STAGES, bool DUAL, bool TWOM = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const GemmKernelParams p) {
  gemm_tcgen05_body<BN, STAGES, DUAL, TWOM, false>(&tmap_w, &tmap_x, nullptr, p);
}

// All-gather fused into the GEMM: tmap_x covers this rank's shard of x, tmap_g the gather areas of the local symmetric
// workspace ([K, world * rows, 2 parities]) that the other ranks' push warps fill.
template <int BN, int STAGES, bool TWOM>
__global__ void __launch_bounds__(kGatherThreads, 1)
gemm_allgather_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_g, const GemmKernelParams p) {
  gemm_tcgen05_body<BN, STAGES, false, TWOM, true>(&tmap_w, &tmap_x, &tmap_g, p);
}

// ------------------------------------------------------------------ host side

struct GemmConfig {
  int bn, splits, stages;
};
static thread_local GemmConfig g_last_config = {0, 0, 0};

static int num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

static int pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

template <int BN, int STAGES, bool DUAL, bool TWOM = false>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmKernelParams& p, int grid,
                       cudaStream_t stream, bool use_pdl) {
  using S = GemmSmem<BN, STAGES, DUAL, TWOM>;
  static_assert(S::kTotal <= 227 * 1024, "shared memory limit exceeded");
  auto kern = gemm_tcgen05_kernel<BN, STAGES, DUAL, TWOM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
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

template <int BN, int STAGES, bool TWOM>
static int launch_gemm_allgather(const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tg, const GemmKernelParams& p, int grid,
                                 cudaStream_t stream, bool use_pdl) {
  using S = GemmSmem<BN, STAGES, false, TWOM>;
  static_assert(S::kTotal <= 227 * 1024, "shared memory limit exceeded");
  auto kern = gemm_allgather_kernel<BN, STAGES, TWOM>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kGatherThreads, 1, 1);
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
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, tg, p) == cudaSuccess ? 0 : -11;
}

}  // namespace ortb200

using namespace ortb200;

namespace {
struct GemmPlan {
  int bn, num_kb, tiles_n, tiles_m, grid, max_contrib;
  int64_t tiles, ws_need;
  bool tile_aligned;
  bool twom;  // CTA tiles of 256 weight rows (two stacked 128-row MMA tiles)
};

// Persistent grid: one CTA per SM.  With many tiles each CTA takes whole tiles; with few, the (tile, k-block)
// units are dealt out evenly (stream-K) and tiles shared by several CTAs are reduced through the workspace.
// ws_available < 0 means "unlimited" (used to size the workspace).
int plan_gemm(int M, int N, int K, bool dual, int force_bn, int force_splits, int64_t ws_available, GemmPlan* pl,
              int force_tile_rows = 0) {
  int bn = force_bn ? force_bn : pick_bn(M);
  if (dual && bn > 128) bn = 128;     // two accumulators, double-buffered, must fit 512 TMEM columns
  pl->bn = bn;
  pl->num_kb = (K + kBK - 1) / kBK;
  // 256 x 256 CTA tiles (two stacked weight tiles sharing the activation tile) halve the X traffic from L2, but the
  // second MMA re-reads the X tile from shared memory and the 512-column accumulator cannot be double-buffered;
  // measured slower than 128 x 256 tiles on B200 (8192 x 6144 x 4096: 575 vs 429 us), so only on request
  pl->twom = !dual && bn == 256 && N >= 256 && force_tile_rows == 256;
  const int tile_rows = pl->twom ? 2 * kBM : kBM;
  pl->tiles_n = (N + tile_rows - 1) / tile_rows;
  pl->tiles_m = (M + bn - 1) / bn;
  pl->tiles = static_cast<int64_t>(pl->tiles_n) * pl->tiles_m;
  if (pl->tiles > 0x7fffffff / pl->num_kb) return -9;
  const int sms = num_sms();
  int grid = sms;
  bool tile_aligned = pl->tiles >= 4LL * sms || force_splits == 1;
  const int64_t units = pl->tiles * pl->num_kb;
  int max_contrib = 1;
  int64_t need = 0;
  if (!tile_aligned) {
    if (units < 2LL * grid) grid = static_cast<int>((units + 1) / 2);
    if (force_splits > 1) {
      int64_t g = pl->tiles * force_splits;
      if (g > sms) g = sms;
      if (g > units) g = units;
      grid = static_cast<int>(g);
    }
    if (grid < 1) grid = 1;
    const int64_t per_cta = units / grid;  // >= 1
    max_contrib = static_cast<int>(pl->num_kb / (per_cta > 0 ? per_cta : 1)) + 2;
    if (max_contrib > grid) max_contrib = grid;
    need = 65536 + pl->tiles * max_contrib * ((dual || pl->twom) ? 2 : 1) * bn * kBM * 4;
    if (pl->tiles > 16384 || (ws_available >= 0 && ws_available < need)) tile_aligned = true;
  }
  if (tile_aligned) {
    max_contrib = 1;
    need = 0;
    if (grid > pl->tiles) grid = static_cast<int>(pl->tiles);
    if (grid > sms) grid = sms;
  }
  pl->grid = grid;
  pl->max_contrib = max_contrib;
  pl->tile_aligned = tile_aligned;
  pl->ws_need = need;
  return 0;
}
}  // namespace

extern "C" int64_t ortb200_allgather_gemm_area_offset(int64_t symm_bytes, int parity) {
  return symm_bytes / 2 + (parity & 1) * (symm_bytes / 4) + symm_bytes / 8;
}
extern "C" int64_t ortb200_allgather_gemm_flag_offset(int src) {
  return kGatherFlagsOffset + (static_cast<int64_t>(src) * 4096 + kGatherFlagSlot) * 4;
}
extern "C" int64_t ortb200_allgather_gemm_max_rows(int world, int K, int64_t symm_bytes) {
  if (world < 1 || K <= 0) return 0;
  return (symm_bytes / 8) / (static_cast<int64_t>(world) * K * 2);
}

extern "C" int ortb200_allgather_gemm(const ortb200_allgather_gemm_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->x_local || !a->w || !a->out) return -1;
  if (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16) return -2;
  if (a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world) return -12;
  if (a->rows_local <= 0 || a->N <= 0 || a->K <= 0 || a->K % 8 != 0) return -3;
  if (a->act == ORTB200_ACT_SWIGLU) return -8;
  if ((reinterpret_cast<uintptr_t>(a->x_local) | reinterpret_cast<uintptr_t>(a->w)) & 15) return -3;
  if (a->rows_local > ortb200_allgather_gemm_max_rows(a->world, a->K, a->symm_bytes)) return -13;
  for (int i = 0; i < a->world; ++i)
    if (!a->peers[i]) return -12;
  const int bn = a->rows_local >= 256 ? 256 : 128;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int64_t pitch = static_cast<int64_t>(a->K) * 2;
  CUtensorMap tw, tx, tg;
  if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, a->N, pitch, kBK, kBM) != 0) return -6;
  if (make_tensor_map_2d(&tx, a->x_local, dt, 2, a->K, a->rows_local, pitch, kBK, bn) != 0) return -6;
  const uint8_t* area0 = static_cast<const uint8_t*>(a->peers[a->rank]) + ortb200_allgather_gemm_area_offset(a->symm_bytes, 0);
  if (make_tensor_map_3d(&tg, area0, dt, 2, a->K, static_cast<int64_t>(a->world) * a->rows_local, 2, pitch, a->symm_bytes / 4, kBK, bn) != 0)
    return -6;
  GemmKernelParams p = {};
  p.M = a->world * a->rows_local; p.N = a->N; p.K = a->K;
  p.num_kb = (a->K + kBK - 1) / kBK;
  const bool twom = bn == 256 && a->N >= 2 * kBM;   // 256 weight rows x 256 tokens per CTA tile
  p.tiles_n = twom ? (a->N + 2 * kBM - 1) / (2 * kBM) : (a->N + kBM - 1) / kBM;
  p.gather_tiles_per_shard = (a->rows_local + bn - 1) / bn;
  p.tiles_m = a->world * p.gather_tiles_per_shard;
  p.tiles = p.tiles_n * p.tiles_m;
  p.tile_aligned = 1; p.max_contrib = 1;
  p.dtype = a->dtype; p.in_fp8 = 0; p.k_per_block = kBK; p.act = a->act; p.alpha = 1.0f; p.alpha_dev = nullptr;
  p.out = a->out; p.ldo = a->N; p.bias = a->bias; p.residual = nullptr; p.ldr = 0;
  p.status = a->status;
  p.gather_world = a->world; p.gather_rank = a->rank; p.gather_rows = a->rows_local;
  for (int i = 0; i < 8; ++i) p.gather_peers[i] = i < a->world ? a->peers[i] : nullptr;
  p.gather_area_offset = ortb200_allgather_gemm_area_offset(a->symm_bytes, 0);
  p.gather_half_bytes = a->symm_bytes / 4;
  p.gather_x_local = a->x_local;
  if (twom) return launch_gemm_allgather<256, 3, true>(tw, tx, tg, p, num_sms(), stream, a->use_pdl != 0);
  return bn == 256 ? launch_gemm_allgather<256, 4, false>(tw, tx, tg, p, num_sms(), stream, a->use_pdl != 0)
                   : launch_gemm_allgather<128, 6, false>(tw, tx, tg, p, num_sms(), stream, a->use_pdl != 0);
}

extern "C" int64_t ortb200_gemm_workspace_bytes(int M, int N, int K, int act) {
  GemmPlan pl, pl128;
  if (M <= 0 || N <= 0 || K <= 0 || plan_gemm(M, N, K, act == ORTB200_ACT_SWIGLU, 0, 0, -1, &pl) != 0) return 65536;
  int64_t need = pl.ws_need;
  if (plan_gemm(M, N, K, act == ORTB200_ACT_SWIGLU, 0, 0, -1, &pl128, 128) == 0 && pl128.ws_need > need) need = pl128.ws_need;
  return need > 65536 ? need : 65536;
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
  const bool fp8 = a->in_dtype == ORTB200_F8E4M3;
  const bool q4 = a->in_dtype == ORTB200_Q4 || a->in_dtype == ORTB200_F8W;  // tile-blob weights expanded inside the decode kernel
  if (a->in_dtype != 0 && !fp8 && !q4 && a->in_dtype != a->dtype) return -4;
  if (a->K % (fp8 ? 16 : 8) != 0) return -2;                     // TMA row pitch must be a multiple of 16 bytes
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return -3;
  if (a->dtype != ORTB200_F16 && a->dtype != ORTB200_BF16) return -4;
  const bool dual = a->act == ORTB200_ACT_SWIGLU;
  if (dual && (a->dual_offset <= 0 || a->w_rows < a->dual_offset + a->N)) return -5;
  if (!dual && a->w_rows < a->N) return -5;
  if (q4 && (a->force_bn ? a->force_bn : pick_bn(a->M)) > 64) return -15;  // packed weights: decode-shaped problems only

  {
    // decode-shaped problems: non-persistent kernel with the split-K reduction inside a cluster
    const int bn_small = a->force_bn ? a->force_bn : pick_bn(a->M);
    if (bn_small <= 64 && !fp8) {
      int cluster = 1, st = 0;
      const int rc_small = launch_gemm_smallm(a, bn_small, stream, &cluster, &st);
      g_last_config = {bn_small, cluster, st};
      return rc_small;
    }
  }
  // Large problems run on CTA pairs (256 x 256 tiles, cta_group::2): measured 1.3 PFLOP/s against 0.98 for the
  // single-CTA kernel on 8192 x 6144 x 4096.  Needs at least most of a wave of 74 pairs to pay off.
  const long long tiles256 = static_cast<long long>((a->M + 255) / 256) * ((a->N + 255) / 256);
  if (a->alpha_dev != nullptr && !fp8) return -16;  // the device-side alpha factor exists in the fp8 kernel only
  const bool pair_ok = !dual && !q4 && a->rms_eps <= 0.f && !(fp8 && a->world > 1);  // fp8 operands run on the pair kernel too
  // world > 1 (row-parallel linear at prompt size): only the CTA-pair kernel has the epilogue that pushes the product
  // into the all-reduce scatter areas; the reduction kernel is launched right behind it
  if (a->force_tile_rows == 512 || (a->world > 1 && pair_ok) ||
      (a->force_tile_rows == 0 && a->force_bn == 0 && a->force_splits == 0 && pair_ok && a->M >= 512 && tiles256 >= 60)) {
    const int rc2 = launch_gemm_2cta(a, stream);
    g_last_config = {256, 2, 5};
    return rc2;
  }
  if (a->world > 1) return -12;  // no fused all-reduce for this combination
  if (a->rms_eps > 0.f) return -14;  // so does the fused RMS normalisation
  GemmPlan pl;
  // fp8 operands: the planner counts 64-element k-blocks, and a stage holds 128 fp8 elements
  const int k_planned = fp8 ? (a->K + 1) / 2 : a->K;
  const int force_bn = fp8 && (a->force_bn == 0 || a->force_bn < 128) ? (a->M > 128 ? 256 : 128) : a->force_bn;
  const int prc = plan_gemm(a->M, a->N, k_planned, dual, force_bn, a->force_splits, a->workspace ? a->workspace_bytes : 0, &pl,
                            a->force_tile_rows);
  if (prc != 0) return prc;
  const int bn = pl.bn, num_kb = pl.num_kb, tiles_m = pl.tiles_m, grid = pl.grid, max_contrib = pl.max_contrib;
  const int64_t tiles = pl.tiles;
  const bool tile_aligned = pl.tile_aligned;

  CUtensorMap tw, tx;
  if (fp8) {
    if (make_tensor_map_2d(&tw, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->K, a->w_rows, a->K, 2 * kBK, kBM) != 0) return -6;
    if (make_tensor_map_2d(&tx, a->x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->K, a->M, a->K, 2 * kBK, bn) != 0) return -6;
  } else {
    const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, a->w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) return -6;
    if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->M, static_cast<int64_t>(a->K) * 2, kBK, bn) != 0) return -6;
  }

  GemmKernelParams p;
  p.in_fp8 = fp8 ? 1 : 0;
  p.k_per_block = fp8 ? 2 * kBK : kBK;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.num_kb = num_kb; p.tiles = static_cast<int>(tiles); p.tiles_m = tiles_m;
  p.tile_info = nullptr; p.num_tiles = nullptr; p.tiles_n = 0; p.w_rows_per_expert = 0;
  p.tile_aligned = tile_aligned ? 1 : 0; p.max_contrib = max_contrib;
  p.dual_offset = a->dual_offset; p.dtype = a->dtype; p.act = a->act; p.alpha = a->alpha; p.alpha_dev = a->alpha_dev;
  p.out = a->out; p.ldo = a->ldo; p.bias = a->bias; p.residual = a->residual; p.ldr = a->ldr;
  p.counters = reinterpret_cast<unsigned int*>(a->workspace);
  p.ws = a->workspace ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a->workspace) + 65536) : nullptr;
  p.status = a->status;

  const bool pdl = a->use_pdl != 0;
  int stages = 0;
  int rc = -7;
  switch (bn) {
    case 16:
      if (dual) { stages = 6; rc = launch_gemm<16, 6, true>(tw, tx, p, grid, stream, pdl); }
      else { stages = 10; rc = launch_gemm<16, 10, false>(tw, tx, p, grid, stream, pdl); }
      break;
    case 32:
      if (dual) { stages = 5; rc = launch_gemm<32, 5, true>(tw, tx, p, grid, stream, pdl); }
      else { stages = 9; rc = launch_gemm<32, 9, false>(tw, tx, p, grid, stream, pdl); }
      break;
    case 64:
      if (dual) { stages = 5; rc = launch_gemm<64, 5, true>(tw, tx, p, grid, stream, pdl); }
      else { stages = 8; rc = launch_gemm<64, 8, false>(tw, tx, p, grid, stream, pdl); }
      break;
    case 128:
      if (dual) { stages = 4; rc = launch_gemm<128, 4, true>(tw, tx, p, grid, stream, pdl); }
      else { stages = 6; rc = launch_gemm<128, 6, false>(tw, tx, p, grid, stream, pdl); }
      break;
    case 256:
      if (pl.twom) { stages = 3; rc = launch_gemm<256, 3, false, true>(tw, tx, p, grid, stream, pdl); }
      else { stages = 4; rc = launch_gemm<256, 4, false>(tw, tx, p, grid, stream, pdl); }
      break;
    default: return -8;
  }
  g_last_config = {bn, tile_aligned ? 1 : max_contrib, stages};
  return rc;
}

// Grouped GEMM on the persistent kernel: token tiles of 128 or 256 rows taken from the device-side tile list.
namespace ortb200 {
int launch_gemm_grouped_large(const ortb200_gemm_grouped_args* a, cudaStream_t stream) {
  const bool dual = a->act == ORTB200_ACT_SWIGLU;
  const int bn = a->tile_rows;
  if ((bn != 128 && bn != 256) || (dual && bn != 128)) return -8;
  const int num_kb = (a->K + kBK - 1) / kBK;
  const int tiles_n = (a->N + kBM - 1) / kBM;
  CUtensorMap tw, tx;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int64_t w_rows = static_cast<int64_t>(a->num_experts) * a->w_rows_per_expert;
  if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) return -6;
  if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->rows, static_cast<int64_t>(a->K) * 2, kBK, bn) != 0) return -6;
  GemmKernelParams p;
  p.M = a->rows; p.N = a->N; p.K = a->K;
  p.num_kb = num_kb; p.tiles = 0; p.tiles_m = 0;
  p.tile_aligned = 1; p.max_contrib = 1;
  p.dual_offset = a->dual_offset; p.dtype = a->dtype; p.in_fp8 = 0; p.k_per_block = kBK; p.act = a->act; p.alpha = 1.0f; p.alpha_dev = nullptr;
  p.out = a->out; p.ldo = a->N; p.bias = a->bias; p.residual = nullptr; p.ldr = 0;
  p.counters = nullptr; p.ws = nullptr; p.status = a->status;
  p.tile_info = static_cast<const int4*>(a->tile_info);
  p.num_tiles = a->num_tiles;
  p.tiles_n = tiles_n;
  p.w_rows_per_expert = a->w_rows_per_expert;
  const int grid = num_sms();
  const bool pdl = a->use_pdl != 0;
  if (dual) return launch_gemm<128, 4, true>(tw, tx, p, grid, stream, pdl);
  if (bn == 128) return launch_gemm<128, 6, false>(tw, tx, p, grid, stream, pdl);
  return launch_gemm<256, 4, false>(tw, tx, p, grid, stream, pdl);
}
}  // namespace ortb200

