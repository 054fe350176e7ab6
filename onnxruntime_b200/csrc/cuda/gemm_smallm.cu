// Decode-shaped GEMM (M <= 64 tokens) for sm_100a: the weight matrix is streamed
// once at HBM speed through TMA into tcgen05.mma, and split-K partial tiles are
// combined inside a thread-block cluster through distributed shared memory.
//
//   out[M, N] = act(alpha * X[M,K] * W[N,K]^T + bias) + residual
//
// A cluster of C CTAs (C = 1, 2, 4 or 8) owns one 128-row weight tile; CTA r
// multiplies k-blocks [r * KB / C, (r + 1) * KB / C) into its own TMEM
// accumulator, drops the fp32 partial tile into its shared memory, and after one
// cluster barrier CTA r sums token columns [r * BN / C, (r + 1) * BN / C) of all
// C partial tiles with ld.shared::cluster (fixed order, so the result does not
// depend on timing) and runs the epilogue for them.  Nothing but the final
// output touches global memory: no workspace, no atomics, no second launch.
//
// This is the path a decode step takes for every projection; it replaces the
// skinny-GEMM special cases of the reference (SmallNGemvSplitKKernel,
// onnxruntime/core/providers/cuda/math/matmul_small_n_gemv.cu:16-60, which keeps
// an fp32 workspace plus an atomic tile counter) and cuBLAS for M <= 64.
#include <cuda.h>
#include <cuda_runtime.h>
#include "gemm_internal.h"
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"

namespace ortb200 {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 192;
// Packed 4-bit weights: four more warps share the expansion (they take the odd k-blocks), and two CTAs per SM keep
// four expansion warps on every SM sub-partition, so one warp's barrier waits and stores hide behind another's ALU work.
constexpr int kThreadsNBits = 320;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// address of the same shared-memory location in CTA `cta` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ float ld_dsmem(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// One 64-bit word carries a partial sum (low half) and the epoch of the launch that wrote it (high half).  A
// naturally aligned 64-bit scalar access is single-copy atomic, so a reader that sees the expected epoch also sees
// the value: no fence, no separate flag and no second NVLink round trip.
__device__ __forceinline__ void st_packed_sys(unsigned long long* p, float v, unsigned int epoch) {
  const unsigned long long w = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_packed_sys(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
// about a second of polling at most; then the launch reports kStatusTimeoutPeer and finishes with what it has
constexpr unsigned int kPeerSpinLimit = 1u << 22;

__device__ __forceinline__ float act_apply(int act, float v) {
  switch (act) {
    case ORTB200_ACT_GELU: return gelu_erf_fast(v);
    case ORTB200_ACT_FASTGELU: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
    case ORTB200_ACT_RELU: return fmaxf(v, 0.0f);
    case ORTB200_ACT_SILU: return v / (1.0f + __expf(-v));
    case ORTB200_ACT_QUICKGELU: return v / (1.0f + __expf(-1.702f * v));
    default: return v;
  }
}

// NBITS: the weight tile arrives as packed 4-bit values (32 bytes per row and k-block, nibbles pre-arranged by
// ortb200_nbits_prepack).  Eight warps expand it to 16-bit values and store them straight into tensor memory
// (thread r = weight row r = TMEM lane r, 32 columns of packed pairs per k-block); the MMA takes its A operand from
// there.  Shared memory only carries the packed bytes and the token tile: an expanded copy in shared memory would be
// written once and read once per k-block (32 KiB against 7 KiB of input), and that traffic, not the ALU work, was
// the bound of the first version of this kernel.
template <int BN, int STAGES, bool DUAL, int NBITS = 0>
struct SmallSmem {
  // NBITS: one tile blob per k-block = 4096 bytes of nibbles + 128 x 2 scales + 128 x 2 zero points (4864 bytes,
  // laid out contiguously in global memory by the prepack step), padded to 5 KiB so the X tile stays 1 KiB aligned
  // NBITS == 2 (fp8 weights, weight-only): 128 rows x 64 e4m3 bytes + 128 fp32 scales = 8704 bytes, padded to 9 KiB
  static constexpr int kBlobBytes = NBITS == 2 ? 8192 + 512 : 4096 + 512 + 256;
  static constexpr int kABytes = NBITS == 2 ? 9216 : (NBITS ? 5120 : kBM * kBK * 2);
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes * (DUAL ? 2 : 1) + kBBytes;
  static constexpr int kCols = (DUAL ? 2 : 1) * BN;
  static constexpr int kPartOffset = 0;  // float part[kCols][128] re-uses the pipeline stages once the main loop is done
  static constexpr int kPartBytes = kCols * kBM * 4;
  static constexpr int kDqOffset = kStageBytes * STAGES;
  static constexpr int kNumDq = 2;    // expansion buffers in tensor memory, one per set of expansion warps (four measured the same)
  static constexpr int kDqCol0 = 64;  // first TMEM column of the buffers (the accumulator uses at most 64 columns)
  static constexpr int kDqCols = kBK / 2;
  static constexpr int kDqBytes = 0;
  static constexpr int kBarOffset = kDqOffset + kDqBytes;
  static_assert(kPartBytes <= kStageBytes * STAGES, "partial tile must fit in the drained pipeline stages");
  static_assert(!NBITS || kStageBytes % 1024 == 0, "swizzled tiles need 1 KiB alignment");
  static_assert(!NBITS || kCols <= kDqCol0, "accumulator and expansion buffers overlap in tensor memory");
  static_assert(!(NBITS && DUAL), "the gated epilogue is not combined with packed weights");
  static constexpr int kRstdOffset = kBarOffset + 8 * (2 * STAGES + 1 + 8) + 16;  // float rstd[64] (fused RMS norm)
  static constexpr int kTotal = kRstdOffset + 64 * 4 + 1024;
  static constexpr int kTmemCols = NBITS ? 128 : (kCols < 32 ? 32 : kCols);
};

// ---- 4-bit expansion helpers.  A prepacked 32-bit word holds 8 weights: bits [4i, 4i+4) = weight 2i, bits
// [16+4i, 16+4i+4) = weight 2i+1, so (w >> 4i) & 0x000F000F is the pair (2i, 2i+1) in the two halves of a register.
// OR-ing the exponent pattern of 128 (bf16) / 1024 (fp16) turns the pair into exact small numbers without a convert.
template <typename T2>
struct Nib {};
template <>
struct Nib<__nv_bfloat162> {
  static constexpr uint32_t kMagic = 0x43004300u;  // 128.0 | 128.0
  static constexpr float kBase = 128.0f;
  __device__ static __nv_bfloat162 bcast(float v) { return __float2bfloat162_rn(v); }
};
template <>
struct Nib<__half2> {
  static constexpr uint32_t kMagic = 0x64006400u;  // 1024.0 | 1024.0
  static constexpr float kBase = 1024.0f;
  __device__ static __half2 bcast(float v) { return __float2half2_rn(v); }
};

// 32 packed weights (four prepacked words) of one quantisation block -> four 16-byte chunks of 8 values each.
// Per pair of weights: one shift, one three-input logic op ((w >> 4i) & 0x000F000F | magic), an exact subtraction of
// (base + zero point) and the multiplication by the scale.  (Folding the last two into one fused multiply-add would
// round -(base + zero point) * scale to the 16-bit type first: an error of up to half a quantisation step.)
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int shift, uint32_t magic) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x000F000F, %2, 0xEA;" : "=r"(r) : "r"(w >> shift), "r"(magic));  // (a & b) | c
  return r;
}
template <typename T2>
__device__ __forceinline__ void expand_words(const uint32_t w[4], T2 zero, T2 scale, uint32_t out[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t bits = nib_pair(w[j], 4 * i, Nib<T2>::kMagic);
      T2 v = *reinterpret_cast<const T2*>(&bits);
      v = __hmul2(__hsub2(v, zero), scale);
      out[4 * j + i] = *reinterpret_cast<const uint32_t*>(&v);
    }
  }
}

// ---- fp8 (e4m3) weight expansion.  An e4m3 byte moved to bits [4, 12) of a bf16 (sign to bit 15) is the same number
// scaled by 2^-120 (exponent bias 7 against 127; subnormals line up as well), so one multiplication by
// 2^120 * block scale yields the dequantised weight.  For fp16 the hardware conversion is used.
__device__ __forceinline__ uint32_t e4m3_pair_to_bf16_bits(uint32_t w, uint32_t selector) {
  uint32_t t;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(w), "r"(0u), "r"(selector));   // bytes -> high halves of the two lanes
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x80008000, %2, 0xEA;" : "=r"(r) : "r"(t), "r"((t >> 4) & 0x07F007F0u));  // (t & sign) | magnitude
  return r;
}
__device__ __forceinline__ void expand_fp8_row(const uint4 (&src)[4], float scale, bool bf16, uint32_t out[32]) {
  const uint32_t w[16] = {src[0].x, src[0].y, src[0].z, src[0].w, src[1].x, src[1].y, src[1].z, src[1].w,
                          src[2].x, src[2].y, src[2].z, src[2].w, src[3].x, src[3].y, src[3].z, src[3].w};
  if (bf16) {
    const __nv_bfloat162 m = __float2bfloat162_rn(scale * 1.329227995784916e36f);   // 2^120 * scale
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t lo = e4m3_pair_to_bf16_bits(w[i], 0x1404u), hi = e4m3_pair_to_bf16_bits(w[i], 0x3424u);
      __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&lo), b = *reinterpret_cast<const __nv_bfloat162*>(&hi);
      a = __hmul2(a, m);
      b = __hmul2(b, m);
      out[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
      out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
    }
  } else {
    const __half2 m = __float2half2_rn(scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      uint32_t lo, hi;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"(static_cast<unsigned short>(w[i] & 0xffffu)));
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"(static_cast<unsigned short>(w[i] >> 16)));
      __half2 a = *reinterpret_cast<const __half2*>(&lo), b = *reinterpret_cast<const __half2*>(&hi);
      a = __hmul2(a, m);
      b = __hmul2(b, m);
      out[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
      out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
    }
  }
}

#ifdef ORTB200_NBITS_TRACE
__device__ unsigned long long g_nbits_trace[16];
#define NB_T(i) do { if (tr) { long long c_ = clock64(); tacc[i] += c_ - tlast; tlast = c_; } } while (0)
#define NB_DECL(cond) const bool tr = (cond); long long tacc[6] = {0, 0, 0, 0, 0, 0}; long long tlast = clock64()
#define NB_DUMP(base, n) do { if (tr) for (int t_ = 0; t_ < (n); ++t_) g_nbits_trace[(base) + t_] = tacc[t_]; } while (0)
#else
#define NB_T(i) do {} while (0)
#define NB_DECL(cond) do {} while (0)
#define NB_DUMP(base, n) do {} while (0)
#endif

template <int BN, int STAGES, bool DUAL, int NBITS = 0>
__global__ void __launch_bounds__(NBITS ? kThreadsNBits : kThreads, NBITS ? 2 : 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const SmallGemmParams p) {
  using S = SmallSmem<BN, STAGES, DUAL, NBITS>;
  static_assert((S::kTmemCols & (S::kTmemCols - 1)) == 0, "TMEM columns must be a power of two");
  extern __shared__ uint8_t smem_raw[];
  // every CTA of the cluster applies the same rounding, so shared-memory offsets agree across the cluster
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem + S::kPartOffset);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  constexpr int NDQ = S::kNumDq;
  uint64_t* dq_full_bar = tmem_full_bar + 1;     // [NDQ] dequantised tile ready (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_full_bar + NDQ);
  float* s_rstd = reinterpret_cast<float*>(smem + S::kRstdOffset);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int C = p.cluster;
  const int rank = C > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int n0 = (blockIdx.x / C) * kBM;
  int m0 = blockIdx.y * BN;
  int m_end = p.M;
  int w_row0 = 0;       // first W row of this tile's expert
  int bias0 = 0;
  if (p.tile_info != nullptr) {
    // grouped mode: the tile list comes from the kernel before this one
    pdl_wait_prior_grids();
    if (static_cast<int>(blockIdx.y) >= *p.num_tiles) return;  // nothing allocated yet; the whole CTA leaves
    const int4 ti = p.tile_info[blockIdx.y];
    m0 = ti.y;
    m_end = ti.z;
    w_row0 = ti.x * p.w_rows_per_expert;
    bias0 = ti.x * p.N;
  }
  const int kb_begin = static_cast<int>(static_cast<long long>(rank) * p.num_kb / C);
  const int kb_end = static_cast<int>(static_cast<long long>(rank + 1) * p.num_kb / C);
  const int nkb = kb_end - kb_begin;  // >= 1 (the host keeps C <= num_kb)

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    for (int d = 0; d < NDQ; ++d) {
      mbar_init(&dq_full_bar[d], 128);
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

  pdl_launch_dependents();  // the next kernel may begin its prologue

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the previous kernel: start streaming them before waiting for X's producer.
      const uint64_t pol_w = policy_evict_first();
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * S::kStageBytes;
        mbar_expect_tx(&full_bar[i], NBITS ? S::kBlobBytes + S::kBBytes : S::kStageBytes);
        if (NBITS) bulk_load(st, static_cast<const uint8_t*>(p.nbits_blob) + (static_cast<long long>(blockIdx.x / C) * p.num_kb + kb_begin + i) * S::kBlobBytes, S::kBlobBytes, &full_bar[i]);
        else tma_load_2d_hint(st, &tmap_w, &full_bar[i], (kb_begin + i) * kBK, w_row0 + n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + S::kABytes, &tmap_w, &full_bar[i], (kb_begin + i) * kBK, w_row0 + n0 + p.dual_offset, pol_w);
      }
      pdl_wait_prior_grids();
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * S::kStageBytes;
        tma_load_2d(st + S::kABytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[i], (kb_begin + i) * kBK, m0);
      }
      NB_DECL(NBITS && blockIdx.x == 5);
      for (int i = pre; i < nkb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) {
          if (p.status) atomicExch(p.status, kStatusTimeoutProducer);
          break;
        }
        NB_T(0);
        uint8_t* st = smem + s * S::kStageBytes;
        mbar_expect_tx(&full_bar[s], NBITS ? S::kBlobBytes + S::kBBytes : S::kStageBytes);
        if (NBITS) bulk_load(st, static_cast<const uint8_t*>(p.nbits_blob) + (static_cast<long long>(blockIdx.x / C) * p.num_kb + kb_begin + i) * S::kBlobBytes, S::kBlobBytes, &full_bar[s]);
        else tma_load_2d_hint(st, &tmap_w, &full_bar[s], (kb_begin + i) * kBK, w_row0 + n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + S::kABytes, &tmap_w, &full_bar[s], (kb_begin + i) * kBK, w_row0 + n0 + p.dual_offset, pol_w);
        tma_load_2d(st + S::kABytes * (DUAL ? 2 : 1), &tmap_x, &full_bar[s], (kb_begin + i) * kBK, m0);
        NB_T(1);
      }
      NB_DUMP(11, 2);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(p.dtype == ORTB200_BF16, kBM, BN);
      // Every bounded wait below depends on the activations, which the producer only requests once the previous grid
      // has finished.  Waiting for that grid here (an unbounded hardware wait that costs nothing once it is satisfied)
      // keeps a slow predecessor - a fused all-reduce waiting for a late rank - from running out this kernel's limits.
      pdl_wait_prior_grids();
      NB_DECL(NBITS && blockIdx.x == 5);
      if (NBITS) {
        // Every k-block of the CTA passes through this one thread, which shares its scheduler with expansion warps:
        // the loop keeps running counters instead of divisions and builds the descriptor once.  The expansion warps
        // waited for the stage before they published the expanded tile, so the token tile that arrived on the same
        // barrier is complete as well and is not waited for again.
        const uint64_t bdesc0 = umma_desc_sw128(smem_u32(smem) + S::kABytes);
        int s = 0, d = 0;
        uint32_t dq_parity = 0, acc = 0;
        for (int i = 0; i < nkb; ++i) {
          if (!mbar_wait(&dq_full_bar[d], dq_parity)) {
            if (p.status) atomicExch(p.status, kStatusTimeoutMma);
            break;
          }
          NB_T(1);
          tcgen05_fence_after();
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(s * (S::kStageBytes >> 4));
          const uint32_t a_tmem = tmem_base + S::kDqCol0 + d * S::kDqCols;
          umma_f16_ts(tmem_base, a_tmem, bdesc, idesc, acc);
          acc = 1u;
#pragma unroll
          for (int k = 1; k < kBK / 16; ++k) umma_f16_ts(tmem_base, a_tmem + 8 * k, bdesc + 2 * k, idesc, 1u);
          umma_commit(&empty_bar[s]);  // frees the stage and tells the expansion warps that the TMEM buffer is free
          NB_T(2);
          if (++s == STAGES) s = 0;
          if (++d == NDQ) { d = 0; dq_parity ^= 1u; }
        }
      } else
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) {
          if (p.status) atomicExch(p.status, kStatusTimeoutMma);
          break;
        }
        tcgen05_fence_after();
        const uint32_t stage_addr = smem_u32(smem + s * S::kStageBytes);
        const uint32_t a_addr = stage_addr;
        const uint32_t b_addr = stage_addr + S::kABytes * (DUAL ? 2 : 1);
        const uint64_t adesc = umma_desc_sw128(a_addr);
        const uint64_t bdesc = umma_desc_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        if (DUAL) {
          const uint64_t a2desc = umma_desc_sw128(a_addr + S::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) umma_f16(tmem_base + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      NB_DUMP(8, 3);
      umma_commit(tmem_full_bar);  // also on the failure path, so the epilogue never waits for nothing
    }
  } else {
    // epilogue warps: TMEM -> registers -> this CTA's partial tile in shared memory
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const bool extra = warp >= 6;  // NBITS only: the second set of expansion warps, no part in the epilogue
    pdl_wait_prior_grids();  // same reason as in the MMA warp: no bounded wait may span the previous grid's run time
    if (NBITS) {
      // ---- weight expansion: thread r owns weight row r of the tile.  Per k-block it reads 32 packed bytes, two
      // scales and two zero points, and writes one 128-byte row of the swizzled MMA operand.
      bool dq_ok = true;
      NB_DECL(blockIdx.x == 5 && r == 0 && !extra);
      // one k-block: wait for the packed tile, expand row r in registers, wait for the buffer, store, publish
      auto expand_kblock = [&](int i) {
        const int s = i % STAGES, d = i % NDQ;
        if (dq_ok && !mbar_wait(&full_bar[s], (i / STAGES) & 1)) dq_ok = false;
        dq_ok = __all_sync(0xffffffffu, dq_ok);
        NB_T(0);
        uint32_t o[32];
        if (dq_ok && NBITS == 2) {
          // fp8 weights: the 64 bytes of row r
          const uint8_t* blob = smem + s * S::kStageBytes;
          const uint4* src = reinterpret_cast<const uint4*>(blob + r * 64);
          const uint4 chunk[4] = {src[0], src[1], src[2], src[3]};
          const float sc = *reinterpret_cast<const float*>(blob + 8192 + r * 4);
          expand_fp8_row(chunk, sc, p.dtype == ORTB200_BF16, o);
        } else if (dq_ok) {
          const uint8_t* blob = smem + s * S::kStageBytes;
          const uint4* src = reinterpret_cast<const uint4*>(blob + r * 32);
          const uint4 p0 = src[0], p1 = src[1];
          // the row's two scales and two zero points travel in the same blob as its nibbles
          const uint32_t sw = *reinterpret_cast<const uint32_t*>(blob + 4096 + r * 4);
          const uint32_t zw = *reinterpret_cast<const uint16_t*>(blob + 4608 + r * 2);
          float s0, s1;
          if (p.dtype == ORTB200_BF16) {
            s0 = __uint_as_float(sw << 16);
            s1 = __uint_as_float(sw & 0xffff0000u);
          } else {
            s0 = __half2float(__ushort_as_half(static_cast<unsigned short>(sw & 0xffffu)));
            s1 = __half2float(__ushort_as_half(static_cast<unsigned short>(sw >> 16)));
          }
          const float z0 = static_cast<float>(zw & 0xffu), z1 = static_cast<float>(zw >> 8);
          const uint32_t w0[4] = {p0.x, p0.y, p0.z, p0.w};
          const uint32_t w1[4] = {p1.x, p1.y, p1.z, p1.w};
          if (p.dtype == ORTB200_BF16) {
            using T2 = __nv_bfloat162;
            expand_words<T2>(w0, Nib<T2>::bcast(Nib<T2>::kBase + z0), Nib<T2>::bcast(s0), o);
            expand_words<T2>(w1, Nib<T2>::bcast(Nib<T2>::kBase + z1), Nib<T2>::bcast(s1), o + 16);
          } else {
            using T2 = __half2;
            expand_words<T2>(w0, Nib<T2>::bcast(Nib<T2>::kBase + z0), Nib<T2>::bcast(s0), o);
            expand_words<T2>(w1, Nib<T2>::bcast(Nib<T2>::kBase + z1), Nib<T2>::bcast(s1), o + 16);
          }
        }
        NB_T(2);
        // The MMAs that read this buffer two k-blocks ago must have finished: their commit completed a phase of that
        // k-block's stage barrier, and the phase after it cannot complete before this k-block has been expanded.
        if (dq_ok && i >= NDQ && !mbar_wait(&empty_bar[(i - NDQ) % STAGES], ((i - NDQ) / STAGES) & 1)) dq_ok = false;
        dq_ok = __all_sync(0xffffffffu, dq_ok);
        NB_T(1);
        if (dq_ok) {
          tcgen05_fence_after();
          const uint32_t t_a = t_lane + S::kDqCol0 + d * S::kDqCols;
          tmem_st_x16_u32(t_a, o);
          tmem_st_x16_u32(t_a + 16, o + 16);
          tmem_st_wait();
          tcgen05_fence_before();  // orders the stores before the arrival the MMA thread waits for
          NB_T(3);
        }
        mbar_arrive(&dq_full_bar[d]);  // also on the failure path: the MMA warp must not wait for nothing
        NB_T(5);
      };
#pragma unroll 1
      for (int i = extra ? 1 : 0; i < nkb; i += 2) expand_kblock(i);
      if (!dq_ok && p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
      NB_DUMP(0, 6);
#ifdef ORTB200_NBITS_TRACE
      if (tr) { g_nbits_trace[6] = (nkb + 1) / 2; g_nbits_trace[7] = nkb; }
#endif
    }
    if (!extra && p.rms_eps > 0.f) {
      // Fused RMS normalisation: the weights carry gamma, so only 1 / rms(x[m, :]) is missing, and it is a per-token
      // factor that commutes with the GEMM.  These warps are idle while the weights stream, so they read the token
      // rows (a few KiB, L2 resident) and leave the factors in shared memory for the epilogue.
      pdl_wait_prior_grids();
      const int vecs = p.K / 8;
      for (int j = q; j < BN; j += 4) {
        const int m = m0 + j;
        float ss = 0.f;
        if (m < m_end) {
          const uint4* row = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x_rows) + static_cast<long long>(m) * p.K * 2);
          for (int v = lane; v < vecs; v += 32) {
            const uint4 u4 = __ldg(row + v);
            const uint32_t w4[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              if (p.dtype == ORTB200_BF16) {
                lo = __uint_as_float(w4[e] << 16);
                hi = __uint_as_float(w4[e] & 0xffff0000u);
              } else {
                const __half2 h2 = *reinterpret_cast<const __half2*>(&w4[e]);
                lo = __low2float(h2);
                hi = __high2float(h2);
              }
              ss += lo * lo + hi * hi;
            }
          }
        }
        ss = warp_sum(ss);
        if (lane == 0) s_rstd[j] = rsqrtf(ss / static_cast<float>(p.K) + p.rms_eps);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");  // the four epilogue warps only
    }
    if (!extra && !mbar_wait(tmem_full_bar, 0)) {
      if (p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
    }
    tcgen05_fence_after();
    if (!extra && C > 1) {
#pragma unroll 1
      for (int c = 0; c < S::kCols; c += 16) {
        float v[16];
        tmem_ld_x16(t_lane + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) part[(c + j) * kBM + r] = v[j];
      }
    }
  }

  // every thread of every CTA in the cluster meets here: partial tiles are complete and visible
  if (C > 1) cluster_sync_all();

  if (warp >= 2 && warp < 6) {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int n = n0 + r;
    const bool n_ok = n < p.N;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    pdl_wait_prior_grids();  // out / residual may still be in use by the previous kernel
    const float bias_v = (p.bias != nullptr && n_ok)
                             ? (p.dtype == ORTB200_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[bias0 + n])
                                                        : __half2float(reinterpret_cast<const __half*>(p.bias)[bias0 + n]))
                             : 0.0f;
    // token columns this CTA finishes
    const int cols_per = BN / C;
    const int j_begin = rank * cols_per;
    const uint32_t part_addr = smem_u32(part);
    const bool fused_ar = p.world > 1;
    unsigned int epoch = 0;
    unsigned int spin_limit = kPeerSpinLimit;
    long long stage_base = 0;  // element offset of staging[epoch & 1][0][0]
    if (fused_ar) {
      epoch = *reinterpret_cast<volatile unsigned int*>(p.epoch) + 1;  // stable: the previous fused launch has completed
      // word 2 of the workspace header overrides the polling limit (0 = default); failure-detection tests set a small
      // one so that a peer that never answers costs milliseconds
      const unsigned int lim = reinterpret_cast<volatile unsigned int*>(p.epoch)[2];
      if (lim != 0) spin_limit = lim;
      stage_base = static_cast<long long>(epoch & 1) * p.world * p.slot_elems;
    }
#pragma unroll 1
    for (int jj = 0; jj < cols_per; ++jj) {
      const int j = j_begin + jj;
      float v = 0.f, u = 0.f;
      if (C > 1) {
        for (int c = 0; c < C; ++c) {
          const uint32_t base = map_to_cta(part_addr, static_cast<uint32_t>(c));
          v += ld_dsmem(base + static_cast<uint32_t>((j * kBM + r) * 4));
          if (DUAL) u += ld_dsmem(base + static_cast<uint32_t>(((BN + j) * kBM + r) * 4));
        }
      } else {
        float t1[8];
        tmem_ld_x8(t_lane + (j & ~7), t1);
        tmem_ld_wait();
        v = t1[j & 7];
        if (DUAL) {
          tmem_ld_x8(t_lane + BN + (j & ~7), t1);
          tmem_ld_wait();
          u = t1[j & 7];
        }
      }
      const int m = m0 + j;
      if (fused_ar) {
        // push this rank's partial sum to every rank (its own copy included); 128 lanes write 1 KiB contiguous
        if (n_ok && m < m_end) {
          const long long off = stage_base + static_cast<long long>(p.rank) * p.slot_elems + static_cast<long long>(m) * p.ldo + n;
          for (int d = 0; d < p.world; ++d) {
            const int dst_rank = (p.rank + d) % p.world;  // spread the first stores over the peers
            st_packed_sys(reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(p.peers[dst_rank]) + p.staging_offset) + off,
                          v * p.alpha, epoch);
          }
        }
        continue;
      }
      if (n_ok && m < m_end) {
        const float row_scale = p.rms_eps > 0.f ? s_rstd[j] * p.alpha : p.alpha;
        float y = v * row_scale + bias_v;
        if (DUAL) {
          const float g = y / (1.0f + __expf(-y));
          y = g * (u * row_scale);
        } else {
          y = act_apply(p.act, y);
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
    if (fused_ar) {
      // gather: the thread that pushed element (m, n) also finishes it, so no CTA-wide barrier is needed; it polls the
      // word of every source rank in its own copy of the staging area until the word carries this launch's epoch
      const unsigned long long* stage_local =
          reinterpret_cast<const unsigned long long*>(static_cast<const uint8_t*>(p.peers[p.rank]) + p.staging_offset) + stage_base;
      bool timed_out = false;
      // Two token columns per round: the loads of all source ranks go out together, so a round costs about one
      // memory round trip instead of one per (column, rank); words that have not arrived yet are re-read together.
      constexpr int CB = 2;
#pragma unroll 1
      for (int jj0 = 0; jj0 < cols_per; jj0 += CB) {
        unsigned long long w[CB][8];
        const unsigned long long* src[CB];
        bool need[CB];
        float resv[CB];
#pragma unroll
        for (int cb = 0; cb < CB; ++cb) {
          const int m = m0 + j_begin + jj0 + cb;
          need[cb] = (jj0 + cb < cols_per) && n_ok && m < m_end;
          src[cb] = stage_local + static_cast<long long>(m) * p.ldo + n;
          resv[cb] = 0.f;
#pragma unroll
          for (int sr = 0; sr < 8; ++sr)
            w[cb][sr] = (need[cb] && sr < p.world) ? ld_packed_sys(src[cb] + static_cast<long long>(sr) * p.slot_elems)
                                                   : (static_cast<unsigned long long>(epoch) << 32);
          if (need[cb] && p.residual) {
            const long long ri = static_cast<long long>(m) * p.ldr + n;
            resv[cb] = p.dtype == ORTB200_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[ri])
                                               : __half2float(reinterpret_cast<const __half*>(p.residual)[ri]);
          }
        }
        unsigned int spins = 0;
        while (!timed_out) {
          bool all = true;
#pragma unroll
          for (int cb = 0; cb < CB; ++cb)
#pragma unroll
            for (int sr = 0; sr < 8; ++sr) all = all && (static_cast<unsigned int>(w[cb][sr] >> 32) == epoch);
          if (all) break;
          if (++spins > spin_limit) {
            timed_out = true;
            break;
          }
          __nanosleep(32);
#pragma unroll
          for (int cb = 0; cb < CB; ++cb)
#pragma unroll
            for (int sr = 0; sr < 8; ++sr)
              if (static_cast<unsigned int>(w[cb][sr] >> 32) != epoch)
                w[cb][sr] = ld_packed_sys(src[cb] + static_cast<long long>(sr) * p.slot_elems);
        }
#pragma unroll
        for (int cb = 0; cb < CB; ++cb) {
          if (!need[cb]) continue;
          const int m = m0 + j_begin + jj0 + cb;
          float y = 0.f;
#pragma unroll
          for (int sr = 0; sr < 8; ++sr)  // fixed order: every rank adds in the same order and gets the same bits
            if (sr < p.world) y += __uint_as_float(static_cast<unsigned int>(w[cb][sr]));
          y = act_apply(p.act, y + bias_v) + resv[cb];
          if (p.dtype == ORTB200_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.ldo + n] = __float2bfloat16_rn(y);
          else reinterpret_cast<__half*>(p.out)[m * p.ldo + n] = __float2half_rn(y);
        }
      }
      if (timed_out && p.status) atomicExch(p.status, kStatusTimeoutPeer);
      // the CTA that finishes last advances the epoch for the next fused launch
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const unsigned int total = gridDim.x * gridDim.y;
        if (atomicAdd(p.done, 1u) == total - 1) {
          *p.done = 0;
          __threadfence();
          *reinterpret_cast<volatile unsigned int*>(p.epoch) = epoch;
        }
      }
    }
  }

  // nobody leaves while a peer may still read its partial tile
  if (C > 1) cluster_sync_all();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
}

template <int BN, int STAGES, bool DUAL, int NBITS = 0>
int launch_small(const CUtensorMap& tw, const CUtensorMap& tx, const SmallGemmParams& p, dim3 grid, cudaStream_t stream,
                 bool use_pdl) {
  using S = SmallSmem<BN, STAGES, DUAL, NBITS>;
  static_assert(S::kTotal <= 113 * 1024, "two CTAs per SM must fit");
  auto kern = gemm_smallm_kernel<BN, STAGES, DUAL, NBITS>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(NBITS ? kThreadsNBits : kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int nattr = 0;
  if (p.cluster > 1) {
    attrs[nattr].id = cudaLaunchAttributeClusterDimension;
    attrs[nattr].val.clusterDim.x = p.cluster;
    attrs[nattr].val.clusterDim.y = 1;
    attrs[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  if (use_pdl) {
    attrs[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = nattr;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, p) == cudaSuccess ? 0 : -11;
}

}  // namespace

int pick_cluster(int tiles, int num_kb, int bn, int force) {
  int c = 1;
  if (force > 0) {
    c = force >= 8 ? 8 : (force >= 4 ? 4 : (force >= 2 ? 2 : 1));
  } else {
    // aim for about two CTAs per SM; keep at least four k-blocks per CTA
    const int want = (2 * 148) / (tiles > 0 ? tiles : 1);
    while (c * 2 <= want && c < 8) c *= 2;
  }
  while (c > 1 && (num_kb / c < 4 || bn % c != 0)) c /= 2;
  return c;
}

int launch_gemm_smallm(const ortb200_gemm_args* a, int bn, cudaStream_t stream, int* cluster_out, int* stages_out) {
  const bool dual = a->act == ORTB200_ACT_SWIGLU;
  const int num_kb = (a->K + kBK - 1) / kBK;
  const int tiles_n = (a->N + kBM - 1) / kBM, tiles_m = (a->M + bn - 1) / bn;
  const int cluster = pick_cluster(tiles_n * tiles_m, num_kb, bn, a->force_splits);
  CUtensorMap tw, tx;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const bool f8w = a->in_dtype == ORTB200_F8W;
  const bool nbits = a->in_dtype == ORTB200_Q4 || f8w;
  if (nbits) {
    // a->w is the tile-blob array of ortb200_nbits_blob_bytes(N, K) bytes: no tensor map, plain bulk copies
    if (dual || a->K % 64 != 0 || a->rms_eps > 0.f) return -15;
    tw = CUtensorMap{};
  } else if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, a->w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) {
    return -6;
  }
  if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->M, static_cast<int64_t>(a->K) * 2, kBK, bn) != 0) return -6;
  SmallGemmParams p;
  p.nbits_blob = nbits ? a->w : nullptr;
  p.M = a->M; p.N = a->N; p.K = a->K; p.num_kb = num_kb; p.cluster = cluster; p.dual_offset = a->dual_offset;
  p.dtype = a->dtype; p.act = a->act; p.alpha = a->alpha; p.out = a->out; p.ldo = a->ldo; p.bias = a->bias;
  p.residual = a->residual; p.ldr = a->ldr; p.status = a->status;
  p.world = 1; p.rank = 0; p.staging_offset = 0; p.slot_elems = 0; p.epoch = nullptr; p.done = nullptr;
  p.tile_info = nullptr; p.num_tiles = nullptr; p.w_rows_per_expert = 0;
  p.rms_eps = a->rms_eps; p.x_rows = a->x;
  if (a->rms_eps > 0.f && a->world > 1) return -12;
  for (int i = 0; i < 8; ++i) p.peers[i] = nullptr;
  if (a->world > 1) {
    if (a->world > 8 || a->rank < 0 || a->rank >= a->world || dual || a->ldo != a->N) return -12;
    const long long staging_off = 262144;
    const long long slot = (a->symm_bytes / 2 - staging_off) / (2LL * a->world * 8);  // the upper half belongs to the collectives
    if (slot < static_cast<long long>(a->M) * a->ldo) return -13;
    for (int i = 0; i < a->world; ++i) {
      if (!a->peers[i]) return -12;
      p.peers[i] = a->peers[i];
    }
    p.world = a->world; p.rank = a->rank; p.staging_offset = staging_off; p.slot_elems = slot;
    p.epoch = reinterpret_cast<unsigned int*>(a->peers[a->rank]);
    p.done = p.epoch + 1;
  }
  dim3 grid(tiles_n * cluster, tiles_m, 1);
  const bool pdl = a->use_pdl != 0;
  *cluster_out = cluster;
  if (f8w) {
    switch (bn) {
      case 16: *stages_out = 9; return launch_small<16, 9, false, 2>(tw, tx, p, grid, stream, pdl);
      case 32: *stages_out = 8; return launch_small<32, 8, false, 2>(tw, tx, p, grid, stream, pdl);
      case 64: *stages_out = 6; return launch_small<64, 6, false, 2>(tw, tx, p, grid, stream, pdl);
      default: return -8;
    }
  }
  if (nbits) {
    switch (bn) {
      case 16: *stages_out = 12; return launch_small<16, 12, false, 1>(tw, tx, p, grid, stream, pdl);
      case 32: *stages_out = 10; return launch_small<32, 10, false, 1>(tw, tx, p, grid, stream, pdl);
      case 64: *stages_out = 8; return launch_small<64, 8, false, 1>(tw, tx, p, grid, stream, pdl);
      default: return -8;
    }
  }
  switch (bn) {
    case 16:
      *stages_out = dual ? 3 : 5;
      return dual ? launch_small<16, 3, true>(tw, tx, p, grid, stream, pdl) : launch_small<16, 5, false>(tw, tx, p, grid, stream, pdl);
    case 32:
      *stages_out = dual ? 2 : 4;
      return dual ? launch_small<32, 2, true>(tw, tx, p, grid, stream, pdl) : launch_small<32, 4, false>(tw, tx, p, grid, stream, pdl);
    case 64:
      *stages_out = dual ? 2 : 3;
      return dual ? launch_small<64, 2, true>(tw, tx, p, grid, stream, pdl) : launch_small<64, 3, false>(tw, tx, p, grid, stream, pdl);
    default: return -8;
  }
}

int launch_gemm_grouped(const ortb200_gemm_grouped_args* a, cudaStream_t stream) {
  const bool dual = a->act == ORTB200_ACT_SWIGLU;
  const int bn = a->tile_rows;
  if (bn != 16 && bn != 32 && bn != 64) return -8;
  const int num_kb = (a->K + kBK - 1) / kBK;
  const int tiles_n = (a->N + kBM - 1) / kBM;
  CUtensorMap tw, tx;
  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int64_t w_rows = static_cast<int64_t>(a->num_experts) * a->w_rows_per_expert;
  if (make_tensor_map_2d(&tw, a->w, dt, 2, a->K, w_rows, static_cast<int64_t>(a->K) * 2, kBK, kBM) != 0) return -6;
  if (make_tensor_map_2d(&tx, a->x, dt, 2, a->K, a->rows, static_cast<int64_t>(a->K) * 2, kBK, bn) != 0) return -6;
  SmallGemmParams p;
  p.M = a->rows; p.N = a->N; p.K = a->K; p.num_kb = num_kb; p.cluster = 1; p.dual_offset = a->dual_offset;
  p.dtype = a->dtype; p.act = a->act; p.alpha = 1.0f; p.out = a->out; p.ldo = a->N; p.bias = a->bias;
  p.residual = nullptr; p.ldr = 0; p.status = a->status;
  p.world = 1; p.rank = 0; p.staging_offset = 0; p.slot_elems = 0; p.epoch = nullptr; p.done = nullptr;
  for (int i = 0; i < 8; ++i) p.peers[i] = nullptr;
  p.rms_eps = 0.f; p.x_rows = nullptr;
  p.nbits_blob = nullptr;
  p.tile_info = static_cast<const int4*>(a->tile_info);
  p.num_tiles = a->num_tiles;
  p.w_rows_per_expert = a->w_rows_per_expert;
  dim3 grid(tiles_n, a->max_tiles, 1);
  const bool pdl = a->use_pdl != 0;
  switch (bn) {
    case 16: return dual ? launch_small<16, 3, true>(tw, tx, p, grid, stream, pdl) : launch_small<16, 5, false>(tw, tx, p, grid, stream, pdl);
    case 32: return dual ? launch_small<32, 2, true>(tw, tx, p, grid, stream, pdl) : launch_small<32, 4, false>(tw, tx, p, grid, stream, pdl);
    default: return dual ? launch_small<64, 2, true>(tw, tx, p, grid, stream, pdl) : launch_small<64, 3, false>(tw, tx, p, grid, stream, pdl);
  }
}

}  // namespace ortb200

extern "C" int ortb200_gemm_grouped(const ortb200_gemm_grouped_args* a, ortb200_stream_t stream) {
  if (!a || !a->x || !a->w || !a->out || !a->tile_info || !a->num_tiles) return -1;
  if (a->rows <= 0 || a->N <= 0 || a->K <= 0 || a->K % 8 != 0 || a->num_experts <= 0 || a->max_tiles <= 0 || a->max_tiles > 65535) return -1;
  if (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16) return -4;
  if (a->act == ORTB200_ACT_SWIGLU && a->dual_offset <= 0) return -2;
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->w) | reinterpret_cast<uintptr_t>(a->tile_info)) & 15) return -3;
  if (a->tile_rows == 256 && a->act != ORTB200_ACT_SWIGLU) return ortb200::launch_gemm_grouped_2cta(a, static_cast<cudaStream_t>(stream));
  if (a->tile_rows >= 128) return ortb200::launch_gemm_grouped_large(a, static_cast<cudaStream_t>(stream));
  return ortb200::launch_gemm_grouped(a, static_cast<cudaStream_t>(stream));
}

#ifdef ORTB200_NBITS_TRACE
extern "C" int ortb200_debug_nbits_trace(unsigned long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, ortb200::g_nbits_trace, sizeof(ortb200::g_nbits_trace)));
}
#endif
