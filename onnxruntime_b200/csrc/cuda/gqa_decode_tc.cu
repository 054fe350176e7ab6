// Decode attention (one query token per sequence) on the tcgen05 tensor cores, head size 128.
//
// The step is bound by reading the KV cache once; what limits a CUDA-core kernel is the instruction stream that turns
// 16-bit keys into fp32 dot products.  Here both products run on the tensor cores with the problem transposed so that
// the long axis is M:
//   MMA 1  S^T[128 keys, 16]   = K_tile[128 keys, 128 dims] . Q[16 heads, 128 dims]^T       (both K-major)
//   MMA 2  O^T[128 dims, 16]  += V_tile^T[128 dims, 128 keys] . P[16 heads, 128 keys]^T     (V MN-major)
// One CTA owns (batch, kv head, key split) and serves every query head of the kv head (up to 16) as the N columns.
// K/V tiles arrive by TMA (128-byte swizzle) through a 3-stage ring; thread t of the 4 softmax warps owns key t of
// the tile (its TMEM lane of S^T): mask, scale, exponentiate, write the 16-bit probabilities into the swizzled
// K-major layout MMA 2 reads.  The reference maximum of a head is only raised when a tile exceeds it by 2^8
// (probabilities stay below 256), so O^T is rescaled in tensor memory a handful of times per sequence instead of
// every tile.  O^T stays in TMEM for the whole key range; at the end thread t reads dim t.  Splits are merged by the
// last CTA to arrive, as in the CUDA-core kernel.
//
// A paged cache is read through a tensor map over [slots, kv heads, dims]: a tile is fetched in pieces of
// min(128, block_size) rows, one TMA per piece, each landing at its row offset inside the swizzled tile.
//
// Reference counterparts: the XQA decode kernels (onnxruntime/contrib_ops/cuda/bert/xqa/mha_impl.cuh), the
// flash-decoding path (bert/flash_attention/flash_api.cc, mha_fwd_kvcache) and PagedDecodeSplitKV
// (bert/paged_attention_impl.cu).
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <type_traits>
#include "gqa_internal.h"
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "tensor_map.h"

namespace ortb200 {

namespace {

constexpr int kTile = 128;                 // keys per tile
constexpr int kStages = 3;
constexpr int kBox = 128 * 128;            // [128 rows][64 elems] of 16-bit data
constexpr int kTileBytes = 2 * kBox;       // K or V tile: two boxes (dims 0-63, 64-127)
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kQBox = 16 * 128;            // [16 heads][64 dims]
constexpr int kPBox = 16 * 128;            // [16 heads][64 keys]
constexpr int kOffQ = kStages * kStageBytes;
constexpr int kOffP = kOffQ + 2 * kQBox;
constexpr int kOffMax = kOffP + 2 * 2 * kPBox;      // float [2][4][16]
constexpr int kOffSum = kOffMax + 2 * 4 * 16 * 4;   // float [4][16]
constexpr int kOffXch = kOffSum + 4 * 16 * 4;        // float [17][128]: q heads and the new key, for the rotary partner
constexpr int kOffNew = kOffXch + 17 * 128 * 4;      // float [16]: scores of the new key
constexpr int kOffBar = kOffNew + 16 * 4;
constexpr int kSmemBytes = kOffBar + 256 + 1024;
constexpr int kThreads = 160;              // 4 softmax warps + 1 TMA / MMA warp
constexpr int kTmemCols = 64;              // S^T buffers at columns 0 and 16, O^T at 32
constexpr float kRaise = 8.f;              // raise the reference maximum only past 2^8

enum { BAR_Q = 0, BAR_FULL0, BAR_EMPTY0 = BAR_FULL0 + kStages, BAR_S0 = BAR_EMPTY0 + kStages, BAR_S1, BAR_P0, BAR_P1, BAR_O,
       BAR_COUNT };

__device__ __forceinline__ float redux_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const float* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
               "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
               : "memory");
}

// G query heads live in columns [0, G) of S^T and O^T; columns are read eight at a time
template <int G>
__device__ __forceinline__ void tmem_ld_heads(uint32_t taddr, float* v) {
#pragma unroll
  for (int c = 0; c < (G + 7) / 8; ++c) tmem_ld_x8(taddr + c * 8, v + c * 8);
  tmem_ld_wait();
}

template <typename T, int G, bool PAGED>
__global__ void __launch_bounds__(kThreads, 1)
gqa_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const DecodeParams p, const int piece_rows) {
  constexpr int H = 128;
  constexpr int GV = (G + 7) / 8 * 8;   // columns fetched from tensor memory
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
  float* sm_max = reinterpret_cast<float*>(smem + kOffMax);
  float* sm_sum = reinterpret_cast<float*>(smem + kOffSum);
  float* sm_xch = reinterpret_cast<float*>(smem + kOffXch);
  float* sm_new = reinterpret_cast<float*>(smem + kOffNew);
  __shared__ unsigned int sm_last;
  // Fused step 1 (one new token per sequence): q, k and v come from the packed projection output; this kernel
  // rotates q and k, writes the query tile itself, appends k / v to the cache and attends to the new key from
  // registers, so no separate prep launch and no round trip of the rotated query through global memory.
  const bool fused = p.qkv != nullptr;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int group = p.N / p.Nk;
  const int head0 = kvh * group;
  const int n_heads = group;

  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int i = 0; i < BAR_COUNT; ++i) mbar_init(&bars[i], (i == BAR_P0 || i == BAR_P1 || (i == BAR_Q && fused)) ? 128 : 1);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 32;

  pdl_wait_prior_grids();
  int total = p.seqlens_k[b] + 1;
  if (total > p.Smax || total < 0) {
    // a length beyond the cache capacity would read past the buffer: attend to what the cache holds and report it
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusBadLength);
    total = total < 0 ? 0 : p.Smax;
  }
  const int start0 = p.window > 0 ? max(0, total - p.window) : 0;
  const int len = max(total - start0, 0);
  int chunk = (len + p.splits - 1) / p.splits;
  if (PAGED) chunk = (chunk + kTile - 1) / kTile * kTile;   // tiles start on piece boundaries (start0 is 0 when paged)
  const int k_begin = start0 + split * chunk;
  // fused: the newest key (position total - 1) is not in the cache yet; the CTA whose range reaches it takes it
  const bool owns_new = fused && k_begin < total && k_begin + chunk >= total;
  const int k_end = owns_new ? total - 1 : min(total, k_begin + chunk);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + kTile - 1) / kTile : 0;

  if (warp == 4 && p.prefetch != nullptr) {
    // This grid moves a few tens of MB and leaves most of the memory bandwidth idle: ask the L2 for this CTA's slice
    // of the next kernel's weights now, so that kernel finds them on chip.
    const long long cta = (static_cast<long long>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    const long long lo = cta * p.prefetch_per_cta;
    const long long hi = lo + p.prefetch_per_cta < p.prefetch_bytes ? lo + p.prefetch_per_cta : p.prefetch_bytes;
    for (long long off = lo + static_cast<long long>(lane) * 16384; off < hi; off += 32 * 16384) {
      const long long nbytes = hi - off < 16384 ? hi - off : 16384;
      bulk_prefetch_l2(p.prefetch + off, static_cast<uint32_t>(nbytes));
    }
  }
  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer + MMA issuer (lane 0 issues; with a
    // paged cache lane i fetches piece i of a tile)
    const uint32_t idesc_s = umma_idesc_f16(kBf16, kTile, 16);
    const uint32_t idesc_o = umma_idesc_f16(kBf16, H, 16) | (1u << 15);   // A (= V^T) is MN-major
    const uint32_t q_addr = smem_u32(smem + kOffQ);
    const int pieces = PAGED ? kTile / piece_rows : 1;
    auto load_tile = [&](int t) {
      const int s = t % kStages;
      uint8_t* st = smem + s * kStageBytes;
      const int key0 = k_begin + t * kTile;
      if (!PAGED) {
        if (lane == 0) {
          mbar_expect_tx(&bars[BAR_FULL0 + s], kStageBytes);
          const int plane = b * p.Nk + kvh;
#pragma unroll
          for (int bx = 0; bx < 2; ++bx) {
            tma_load_3d(st + bx * kBox, &tm_k, &bars[BAR_FULL0 + s], bx * 64, key0, plane);
            tma_load_3d(st + kTileBytes + bx * kBox, &tm_v, &bars[BAR_FULL0 + s], bx * 64, key0, plane);
          }
        }
      } else {
        // pieces whose first key lies beyond the range are not fetched (their block-table entries may be unset)
        const int live = min(pieces, (k_end - key0 + piece_rows - 1) / piece_rows);
        if (lane == 0) mbar_expect_tx(&bars[BAR_FULL0 + s], static_cast<uint32_t>(live) * piece_rows * 4 * 128);
        __syncwarp();
        if (lane < live) {
          const int key = key0 + lane * piece_rows;
          const int bi = key / p.block_size;
          const int blk = bi < p.max_blocks ? p.block_table[static_cast<long long>(b) * p.max_blocks + bi] : -1;
          // a block index outside the pool reads as zeros (TMA fills out-of-range rows)
          const int row = blk >= 0 ? blk * p.block_size + key % p.block_size : 0x3fffff00;
          uint8_t* dst = st + lane * piece_rows * 128;
#pragma unroll
          for (int bx = 0; bx < 2; ++bx) {
            tma_load_3d(dst + bx * kBox, &tm_k, &bars[BAR_FULL0 + s], bx * 64, row, kvh);
            tma_load_3d(dst + kTileBytes + bx * kBox, &tm_v, &bars[BAR_FULL0 + s], bx * 64, row, kvh);
          }
        }
      }
      __syncwarp();
    };
    auto issue_s = [&](int t) {
      const uint32_t k_addr = smem_u32(smem + (t % kStages) * kStageBytes);
      const uint32_t d = tmem_base + (t & 1) * 16;
#pragma unroll
      for (int kk = 0; kk < H / 16; ++kk) {
        umma_f16(d, umma_desc_sw128(k_addr + (kk / 4) * kBox + (kk % 4) * 32),
                 umma_desc_sw128(q_addr + (kk / 4) * kQBox + (kk % 4) * 32), idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit(&bars[BAR_S0 + (t & 1)]);
    };
    bool ok = true;
    if (n_tiles > 0) {
      if (lane == 0 && !fused) {
        mbar_expect_tx(&bars[BAR_Q], 2 * kQBox);
        tma_load_2d(smem + kOffQ, &tm_q, &bars[BAR_Q], 0, b * p.N + head0);
        tma_load_2d(smem + kOffQ + kQBox, &tm_q, &bars[BAR_Q], 64, b * p.N + head0);
      }
      const int pre = n_tiles < kStages ? n_tiles : kStages;
      for (int t = 0; t < pre; ++t) load_tile(t);
      ok = mbar_wait(&bars[BAR_Q], 0) && mbar_wait(&bars[BAR_FULL0], 0);
      if (ok && lane == 0) {
        tcgen05_fence_after();
        issue_s(0);
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int s = t % kStages;
        if (t + 1 < n_tiles) {
          // S^T buffer (t + 1) & 1 was consumed before P of tile t - 1 was published, which this warp waited for
          if (!mbar_wait(&bars[BAR_FULL0 + (t + 1) % kStages], ((t + 1) / kStages) & 1)) { ok = false; break; }
          if (lane == 0) {
            tcgen05_fence_after();
            issue_s(t + 1);
          }
        }
        if (!mbar_wait(&bars[BAR_P0 + (t & 1)], (t >> 1) & 1)) { ok = false; break; }
        if (lane == 0) {
          tcgen05_fence_after();
          const uint32_t v_addr = smem_u32(smem + s * kStageBytes + kTileBytes);
          const uint32_t p_addr = smem_u32(smem + kOffP + (t & 1) * 2 * kPBox);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            umma_f16(tmem_o, umma_desc_mn_sw128(v_addr + kk * 2048, kBox, 1024),
                     umma_desc_sw128(p_addr + (kk / 4) * kPBox + (kk % 4) * 32), idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&bars[BAR_EMPTY0 + s]);
          umma_commit(&bars[BAR_O]);
        }
        __syncwarp();
        if (t + kStages < n_tiles) {
          if (!mbar_wait(&bars[BAR_EMPTY0 + s], (t / kStages) & 1)) { ok = false; break; }
          load_tile(t + kStages);
        }
      }
      if (!ok && lane == 0 && p.status) atomicExch(p.status, kStatusTimeoutMma);
    }
  }

  // ---------------------------------------------------------------- softmax threads: thread t owns key t of a tile
  float m_ref[G], l_part[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_ref[g] = kNegBig;
    l_part[g] = 0.f;
  }
  bool ok = true;
  const float scale_log2 = p.scale * 1.4426950408889634f;
  float v_new = 0.f;   // fused: this thread's dim of the new value row
  if (warp < 4 && fused) {
    // thread t holds dim t of every query head of the group, of the new key and of the new value
    const int t = tid;
    const T* row = static_cast<const T*>(p.qkv) + static_cast<long long>(b) * (p.N + 2 * p.Nk) * H;
    float c = 1.f, sn = 0.f;
    if (p.do_rotary) {
      const int fi = p.interleaved ? (t >> 1) : (t & (H / 2 - 1));
      const int rpos = p.cos_rows > 0 && total - 1 >= p.cos_rows ? p.cos_rows - 1 : (total > 0 ? total - 1 : 0);  // stay inside the tables
      c = to_float<T>(static_cast<const T*>(p.cos_cache)[static_cast<long long>(rpos) * (H / 2) + fi]);
      sn = to_float<T>(static_cast<const T*>(p.sin_cache)[static_cast<long long>(rpos) * (H / 2) + fi]);
    }
    float qx[G];
#pragma unroll
    for (int g = 0; g < G; ++g) qx[g] = g < n_heads ? to_float<T>(row[static_cast<long long>(head0 + g) * H + t]) : 0.f;
    float kx = to_float<T>(row[static_cast<long long>(p.N + kvh) * H + t]);
    const T v_raw = row[static_cast<long long>(p.N + p.Nk + kvh) * H + t];
    v_new = to_float<T>(v_raw);
    if (p.do_rotary) {
#pragma unroll
      for (int g = 0; g < G; ++g) sm_xch[g * 128 + t] = qx[g];
      sm_xch[16 * 128 + t] = kx;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int partner = p.interleaved ? (t ^ 1) : (t ^ (H / 2));
      const bool second = p.interleaved ? (t & 1) : (t >= H / 2);   // holds the "imaginary" half of its pair
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float o = sm_xch[g * 128 + partner];
        qx[g] = second ? qx[g] * c + o * sn : qx[g] * c - o * sn;
      }
      const float ok_ = sm_xch[16 * 128 + partner];
      kx = second ? kx * c + ok_ * sn : kx * c - ok_ * sn;
    }
    // the query tile in the layout MMA 1 reads (128-byte swizzle, K-major); rows past the group stay zero
    const T k_t = from_float<T>(kx);
    float part[G];
    {
      uint8_t* qb = smem + kOffQ + (t >> 6) * kQBox;
      const int col = t & 63;
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        T qt = from_float<T>(0.f);
        if (g < G) {
          qt = from_float<T>(qx[g < G ? g : 0]);
          part[g < G ? g : 0] = to_float<T>(qt) * to_float<T>(k_t);
        }
        *reinterpret_cast<T*>(qb + g * 128 + (((col >> 3) ^ (g & 7)) << 4) + (col & 7) * 2) = qt;
      }
    }
    fence_proxy_async();
    mbar_arrive(&bars[BAR_Q]);
    // score of the new key for every head: a 128-thread dot product
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float ws = warp_sum(part[g]);
      if (lane == 0) sm_sum[warp * 16 + g] = ws;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (t < G) sm_new[t] = sm_sum[t] + sm_sum[16 + t] + sm_sum[32 + t] + sm_sum[48 + t];
    if (owns_new) {
      long long crow;
      if (PAGED) {
        const int key = total - 1;
        const int bi = key / p.block_size;
        const int blk = bi < p.max_blocks ? p.block_table[static_cast<long long>(b) * p.max_blocks + bi] : -1;
        crow = blk >= 0 ? ((static_cast<long long>(blk) * p.block_size + key % p.block_size) * p.Nk + kvh) * H : -1;
      } else {
        crow = ((static_cast<long long>(b) * p.Nk + kvh) * p.Smax + (total - 1)) * H;
      }
      if (crow >= 0 && total - 1 < p.Smax) {
        static_cast<T*>(const_cast<void*>(p.k_cache))[crow + t] = k_t;
        static_cast<T*>(const_cast<void*>(p.v_cache))[crow + t] = v_raw;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // sm_sum is reused at the end; sm_new is complete
  }
  if (warp < 4) {
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    // A wait that gives up clears `ok`; the loop still runs to its end (without further waits) so that every
    // thread keeps meeting the others at the named barrier and publishes P for the MMA warp.
    for (int t = 0; t < n_tiles; ++t) {
      if (ok && !mbar_wait(&bars[BAR_S0 + (t & 1)], (t >> 1) & 1)) ok = false;
      tcgen05_fence_after();
      float sv[GV];
      tmem_ld_heads<G>(tmem_base + lane_addr + (t & 1) * 16, sv);
      const int key = k_begin + t * kTile + tid;
      const bool valid = key < k_end;
      float* mx = sm_max + (t & 1) * 64;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sc = sv[g];
        if (p.softcap > 0.f) sc = p.softcap * tanhf(sc * p.scale / p.softcap) * 1.4426950408889634f;
        else sc *= scale_log2;
        sv[g] = valid ? sc : kNegBig;
        const float wm = redux_max(sv[g]);
        if (lane == 0) mx[warp * 16 + g] = wm;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float corr[G];
      bool raise = false;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float mt = fmaxf(fmaxf(mx[g], mx[16 + g]), fmaxf(mx[32 + g], mx[48 + g]));
        corr[g] = 1.f;
        if (mt > m_ref[g] + kRaise) {
          corr[g] = m_ref[g] <= kNegBig ? 0.f : exp2f(m_ref[g] - mt);
          m_ref[g] = mt;
          raise = true;
        }
      }
      if (raise) {   // uniform over the CTA: every thread saw the same maxima
#pragma unroll
        for (int g = 0; g < G; ++g) l_part[g] *= corr[g];
        if (t > 0) {
          // O^T holds the sum up to tile t - 1 once its MMA has finished; thread t rescales its dim
          if (ok && !mbar_wait(&bars[BAR_O], (t - 1) & 1)) ok = false;
          tcgen05_fence_after();
          float ov[GV];
          tmem_ld_heads<G>(tmem_o + lane_addr, ov);
#pragma unroll
          for (int g = 0; g < G; ++g) ov[g] *= corr[g];
#pragma unroll
          for (int c = 0; c < GV / 8; ++c) tmem_st_x8(tmem_o + lane_addr + c * 8, ov + c * 8);
          tmem_st_wait();
        }
      }
      // probabilities of this key for every head, rounded to the MMA input type (the sum uses the rounded values)
      uint8_t* pb = smem + kOffP + (t & 1) * 2 * kPBox + (tid >> 6) * kPBox;
      const int col = tid & 63;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = valid ? exp2f(sv[g] - m_ref[g]) : 0.f;
        const T pt = from_float<T>(pr);
        l_part[g] += to_float<T>(pt);
        *reinterpret_cast<T*>(pb + g * 128 + (((col >> 3) ^ (g & 7)) << 4) + (col & 7) * 2) = pt;
      }
      if (k_begin + (t + 1) * kTile > k_end) {
        // last, partial tile: rows past the range hold whatever the cache (or an earlier tile) left there; a
        // non-finite value times a zero probability would poison MMA 2, so those V rows are cleared
        if (ok && !mbar_wait(&bars[BAR_FULL0 + t % kStages], (t / kStages) & 1)) ok = false;
        if (!valid) {
          uint8_t* vrow = smem + (t % kStages) * kStageBytes + kTileBytes + tid * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            *reinterpret_cast<uint4*>(vrow + i * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vrow + kBox + i * 16) = make_uint4(0, 0, 0, 0);
          }
        }
      }
      fence_proxy_async();
      tcgen05_fence_before();
      mbar_arrive(&bars[BAR_P0 + (t & 1)]);
    }
    if (!ok && p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
  }
  // (Letting the next kernel start earlier than this was measured slower: its CTAs and those of the kernels that
  // chain behind it pile onto the SMs while the cache is still being streamed.)
  pdl_launch_dependents();

  // ---------------------------------------------------------------- gather the CTA's state: thread t takes dim t
  float fm[G], fl[G], fa[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float ws = warp_sum(l_part[g]);
    if (warp < 4 && lane == 0) sm_sum[warp * 16 + g] = ws;
  }
  if (warp < 4 && ok && n_tiles > 0) {
    if (!mbar_wait(&bars[BAR_O], (n_tiles - 1) & 1)) {
      ok = false;
      if (p.status) atomicExch(p.status, kStatusTimeoutEpilogue);
    }
  }
  tcgen05_fence_after();
  float ov[GV];
#pragma unroll
  for (int g = 0; g < GV; ++g) ov[g] = 0.f;
  if (warp < 4 && ok && n_tiles > 0) tmem_ld_heads<G>(tmem_o + (static_cast<uint32_t>(warp * 32) << 16), ov);
  tcgen05_fence_before();
  __syncthreads();
  if (warp < 4 && tid == 0) {
    // the maxima are the same in every softmax thread; the TMA / MMA warp reads them from shared memory
#pragma unroll
    for (int g = 0; g < G; ++g) sm_max[g] = m_ref[g];
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float m2 = sm_max[g];
    fm[g] = m2 <= kNegBig ? kNegBig : m2 * 0.6931471805599453f;   // base-2 logits back to the natural-log domain
    fl[g] = ok ? sm_sum[g] + sm_sum[16 + g] + sm_sum[32 + g] + sm_sum[48 + g] : 0.f;
    fa[g] = ov[g];
  }
  if (warp == 4) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (owns_new) {
    // fold the new key, held in registers, into the state of this CTA's key range
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sc = sm_new[g] * p.scale;
      if (p.softcap > 0.f) sc = p.softcap * tanhf(sc / p.softcap);
      const float m_new = fmaxf(fm[g], sc);
      const float c_old = safe_exp_diff(fm[g], m_new);
      const float pn = __expf(sc - m_new);
      fl[g] = fl[g] * c_old + pn;
      fa[g] = fa[g] * c_old + pn * v_new;
      fm[g] = m_new;
    }
  }
  const int tile = b * p.Nk + kvh;
  decode_finish<T, H, G>(p, tile, split, b, head0, n_heads, tid, fm, fl, fa, &sm_last);
}

template <typename T, int G, bool PAGED>
int launch_tc(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p, int piece_rows,
              dim3 grid, cudaStream_t stream, bool use_pdl) {
  auto kern = gqa_decode_tc_kernel<T, G, PAGED>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  if (use_pdl) {
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, p, piece_rows) == cudaSuccess ? 0 : -11;
}

template <typename T, bool PAGED>
int launch_tc_g(int group, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p,
                int piece_rows, dim3 grid, cudaStream_t stream, bool use_pdl) {
  if (group <= 4) return launch_tc<T, 4, PAGED>(tq, tk, tv, p, piece_rows, grid, stream, use_pdl);
  if (group <= 8) return launch_tc<T, 8, PAGED>(tq, tk, tv, p, piece_rows, grid, stream, use_pdl);
  return launch_tc<T, 16, PAGED>(tq, tk, tv, p, piece_rows, grid, stream, use_pdl);
}

}  // namespace

bool gqa_decode_tc_supported(const ortb200_gqa_decode_args* a) {
  if (a->H != 128 || (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16)) return false;
  if (a->qkv == nullptr && a->q == nullptr) return false;
  if (a->qkv != nullptr && (reinterpret_cast<uintptr_t>(a->qkv) & 15)) return false;
  const int group = a->N / a->Nk;
  if (group > 16 || !a->workspace) return false;
  if (a->qkv == nullptr && (reinterpret_cast<uintptr_t>(a->q) & 15)) return false;
  if (a->block_table) {
    const int bs = a->block_size;
    if (bs < 8 || (bs & (bs - 1)) != 0 || a->window > 0 || a->num_blocks <= 0) return false;
  }
  return true;
}

// Launches the tensor-core decode kernel; the caller has checked gqa_decode_tc_supported().
int launch_gqa_decode_tc(const ortb200_gqa_decode_args* a, cudaStream_t stream) {
  constexpr int H = 128;
  const int group = a->N / a->Nk;
  const int G = group <= 4 ? 4 : (group <= 8 ? 8 : 16);
  const int base = a->B * a->Nk;
  int splits = a->splits;
  if (splits <= 0) {
    // One CTA per SM at most.  Merging splits costs about as much as four tiles, so a grid that already covers a
    // good part of the machine with short key ranges is not split; otherwise at least two tiles per split.
    const int tiles = (a->Smax + kTile - 1) / kTile;
    if (base >= 32 && tiles <= 12) {
      splits = 1;
    } else {
      splits = 148 / base;
      if (splits > (tiles + 1) / 2) splits = (tiles + 1) / 2;
      if (splits > 32) splits = 32;
      if (splits < 1) splits = 1;
    }
  }
  if (base > 16384) return -4;
  while (splits > 1 && 65536 + static_cast<int64_t>(base) * splits * G * (H + 4) * 4 > a->workspace_bytes) --splits;
  if (a->workspace_bytes < 65536) return -4;

  const CUtensorMapDataType dt = a->dtype == ORTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tq, tk, tv;
  // fused launches build the query tile themselves; the map then only has to be a valid one
  const void* q_base = a->qkv != nullptr ? a->k_cache : a->q;
  if (make_tensor_map_2d(&tq, q_base, dt, 2, H, static_cast<int64_t>(a->B) * a->N, H * 2, 64, 16) != 0) return -5;
  int piece_rows = kTile;
  if (a->block_table) {
    piece_rows = a->block_size < kTile ? a->block_size : kTile;
    const int64_t slots = static_cast<int64_t>(a->num_blocks) * a->block_size;
    // [slots, kv heads, dims] seen as planes = kv heads, rows = slots
    if (make_tensor_map_3d(&tk, a->k_cache, dt, 2, H, slots, a->Nk, static_cast<int64_t>(a->Nk) * H * 2, H * 2, 64, piece_rows) != 0 ||
        make_tensor_map_3d(&tv, a->v_cache, dt, 2, H, slots, a->Nk, static_cast<int64_t>(a->Nk) * H * 2, H * 2, 64, piece_rows) != 0)
      return -5;
  } else {
    const int64_t planes = static_cast<int64_t>(a->B) * a->Nk;
    if (make_tensor_map_3d(&tk, a->k_cache, dt, 2, H, a->Smax, planes, H * 2, static_cast<int64_t>(a->Smax) * H * 2, 64, kTile) != 0 ||
        make_tensor_map_3d(&tv, a->v_cache, dt, 2, H, a->Smax, planes, H * 2, static_cast<int64_t>(a->Smax) * H * 2, 64, kTile) != 0)
      return -5;
  }
  DecodeParams p{};
  p.q = a->q; p.k_cache = a->k_cache; p.v_cache = a->v_cache; p.seqlens_k = a->seqlens_k; p.head_sink = a->head_sink;
  p.out = a->out;
  p.counters = reinterpret_cast<unsigned int*>(a->workspace);
  p.ws = reinterpret_cast<float*>(static_cast<char*>(a->workspace) + 65536);
  p.status = a->status;
  p.B = a->B; p.N = a->N; p.Nk = a->Nk; p.Smax = a->Smax; p.splits = splits; p.window = a->window; p.gparts = 1;
  p.scale = a->scale != 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(H));
  p.softcap = a->softcap;
  p.block_table = a->block_table; p.block_size = a->block_size; p.max_blocks = a->max_blocks;
  p.qkv = a->qkv; p.cos_cache = a->cos_cache; p.sin_cache = a->sin_cache; p.cos_rows = a->cos_rows;
  p.do_rotary = a->do_rotary; p.interleaved = a->rotary_interleaved;
  dim3 grid(splits, a->Nk, a->B);
  p.prefetch = nullptr; p.prefetch_bytes = 0; p.prefetch_per_cta = 0;
  if (a->prefetch != nullptr && a->prefetch_bytes >= 16 && (reinterpret_cast<uintptr_t>(a->prefetch) & 15) == 0) {
    const long long bytes = (a->prefetch_bytes < (48LL << 20) ? a->prefetch_bytes : (48LL << 20)) & ~15LL;
    const long long ctas = static_cast<long long>(grid.x) * grid.y * grid.z;
    p.prefetch = static_cast<const unsigned char*>(a->prefetch);
    p.prefetch_bytes = bytes;
    p.prefetch_per_cta = static_cast<int>(((bytes + ctas - 1) / ctas + 15) & ~15LL);
  }
  const bool pdl = a->use_pdl != 0;
  if (a->dtype == ORTB200_BF16) {
    return a->block_table ? launch_tc_g<__nv_bfloat16, true>(group, tq, tk, tv, p, piece_rows, grid, stream, pdl)
                          : launch_tc_g<__nv_bfloat16, false>(group, tq, tk, tv, p, piece_rows, grid, stream, pdl);
  }
  return a->block_table ? launch_tc_g<__half, true>(group, tq, tk, tv, p, piece_rows, grid, stream, pdl)
                        : launch_tc_g<__half, false>(group, tq, tk, tv, p, piece_rows, grid, stream, pdl);
}

}  // namespace ortb200
