// GroupQueryAttention for sm_100a: the fused "unpack packed QKV + rotary + KV
// append" kernel and the split-KV decode attention kernel.
//
// Reference counterparts: UnpackRoPEAppend
// (onnxruntime/contrib_ops/cuda/bert/group_query_attention_qkv.cuh:43), the XQA /
// flash-decoding decode paths (bert/xqa/mha_impl.cuh, flash_api.cc:441
// mha_fwd_kvcache) and PagedDecodeSplitKV + PagedDecodeReduce
// (bert/paged_attention_impl.cu:719,963).
//
// Decode attention is bound by reading the KV cache once.  One CTA owns one
// (batch, kv head, split) and serves all query heads of that kv head, so K and V
// are streamed exactly once; 8 lanes share a key (32-byte vector loads, 3 shuffle
// steps per dot product), the online-softmax state lives in registers, and the
// CTA that arrives last on a per-(batch, kv head) counter merges the splits - no
// second launch, grid size independent of the current sequence length so the
// launch can be captured in a CUDA graph.
#include <cuda_runtime.h>
#include <math.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"
#include "gqa_internal.h"

namespace ortb200 {

// ------------------------------------------------------------------ prep
template <typename T>
__global__ void __launch_bounds__(256) gqa_prep_kernel(const ortb200_gqa_prep_args a) {
  const int b = blockIdx.x / a.S, s = blockIdx.x % a.S;
  const int H = a.H, halfH = H / 2;
  const int rot = a.rot_dim > 0 ? a.rot_dim : H;
  const int half = rot / 2;
  const int heads = a.N + 2 * a.Nk;
  pdl_launch_dependents();  // the attention kernel may set up; it waits for this grid before reading q or the caches
  pdl_wait_prior_grids();
  const int past = a.first_prompt ? 0 : a.seqlens_k[b] + 1 - a.S;
  long long pos = a.position_ids ? a.position_ids[static_cast<long long>(b) * a.S + s] : past + s;
  if (a.cos_rows > 0) pos = pos < 0 ? 0 : (pos >= a.cos_rows ? a.cos_rows - 1 : pos);  // never read past the rotary tables
  const int cache_pos = past + s;
  const long long tok = static_cast<long long>(b) * a.S + s;
  const T* cosr = a.do_rotary ? static_cast<const T*>(a.cos_cache) + pos * half : nullptr;
  const T* sinr = a.do_rotary ? static_cast<const T*>(a.sin_cache) + pos * half : nullptr;
  // blockIdx.y selects a group of heads so that few tokens still fill the machine
  const int heads_per_block = (heads + gridDim.y - 1) / gridDim.y;
  const int head_lo = blockIdx.y * heads_per_block;
  const int head_hi = min(heads, head_lo + heads_per_block);
  for (int idx = head_lo * halfH + threadIdx.x; idx < head_hi * halfH; idx += blockDim.x) {
    const int head = idx / halfH, i = idx % halfH;
    const T* src;
    if (a.k != nullptr) {
      if (head < a.N) src = static_cast<const T*>(a.qkv) + tok * (a.N * H) + head * H;
      else if (head < a.N + a.Nk) src = static_cast<const T*>(a.k) + tok * (a.Nk * H) + (head - a.N) * H;
      else src = static_cast<const T*>(a.v) + tok * (a.Nk * H) + (head - a.N - a.Nk) * H;
    } else {
      src = static_cast<const T*>(a.qkv) + tok * (static_cast<long long>(heads) * H) + head * H;
    }
    T* dst;
    if (head < a.N) {
      dst = static_cast<T*>(a.q_out) + tok * (a.N * H) + head * H;
    } else {
      if (cache_pos < 0 || cache_pos >= a.Smax) continue;
      const bool is_k = head < a.N + a.Nk;
      const int kh = is_k ? head - a.N : head - a.N - a.Nk;
      T* base = static_cast<T*>(is_k ? a.k_cache : a.v_cache);
      dst = base + ((static_cast<long long>(b) * a.Nk + kh) * a.Smax + cache_pos) * H;
    }
    const bool rotate = a.do_rotary && head < a.N + a.Nk && i < half;
    int e0, e1;
    if (i < half) {
      e0 = a.interleaved ? 2 * i : i;
      e1 = a.interleaved ? 2 * i + 1 : i + half;
    } else {
      e0 = rot + 2 * (i - half);
      e1 = e0 + 1;
    }
    if (!a.do_rotary || head >= a.N + a.Nk) {
      e0 = 2 * i;
      e1 = 2 * i + 1;
    }
    const float x0 = to_float<T>(src[e0]), x1 = to_float<T>(src[e1]);
    if (rotate) {
      const float c = to_float<T>(cosr[i]), sn = to_float<T>(sinr[i]);
      dst[e0] = from_float<T>(x0 * c - x1 * sn);
      dst[e1] = from_float<T>(x1 * c + x0 * sn);
    } else {
      dst[e0] = src[e0];
      dst[e1] = src[e1];
    }
  }
}

// ------------------------------------------------------------ paged prep
// One CTA per packed token: find its sequence, rotate Q and K at position past + offset, store Q and write K / V
// into the cache slot named by slot_mapping (when given) or by the block table.
template <typename T>
__global__ void __launch_bounds__(256) paged_prep_kernel(const ortb200_paged_prep_args a) {
  const int t = blockIdx.x;
  const int H = a.H, halfH = H / 2;
  const int rot = a.rot_dim > 0 ? a.rot_dim : H;
  const int half = rot / 2;
  const int heads = a.N + 2 * a.Nk;
  pdl_wait_prior_grids();
  // sequence of this token: last b with cu_seqlens[b] <= t
  int lo = 0, hi = a.B;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (a.cu_seqlens[mid] <= t) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int pos = a.past_seqlens[b] + (t - a.cu_seqlens[b]);
  long long slot;
  if (a.slot_mapping) {
    slot = a.slot_mapping[t];
  } else {
    const int bi = pos / a.block_size;
    slot = bi < a.max_blocks ? static_cast<long long>(a.block_table[static_cast<long long>(b) * a.max_blocks + bi]) * a.block_size + pos % a.block_size : -1;
  }
  const bool slot_ok = slot >= 0 && slot < static_cast<long long>(a.num_blocks) * a.block_size;
  if (!a.slot_mapping && !slot_ok && threadIdx.x == 0 && a.status) atomicExch(a.status, kStatusBadArgument);
  const int rpos = a.cos_rows > 0 ? (pos < 0 ? 0 : (pos >= a.cos_rows ? a.cos_rows - 1 : pos)) : pos;  // never read past the rotary tables
  const T* cosr = a.do_rotary ? static_cast<const T*>(a.cos_cache) + static_cast<long long>(rpos) * half : nullptr;
  const T* sinr = a.do_rotary ? static_cast<const T*>(a.sin_cache) + static_cast<long long>(rpos) * half : nullptr;
  for (int idx = threadIdx.x; idx < heads * halfH; idx += blockDim.x) {
    const int head = idx / halfH, i = idx % halfH;
    const T* src;
    if (a.k != nullptr) {
      if (head < a.N) src = static_cast<const T*>(a.qkv) + static_cast<long long>(t) * (a.N * H) + head * H;
      else if (head < a.N + a.Nk) src = static_cast<const T*>(a.k) + static_cast<long long>(t) * (a.Nk * H) + (head - a.N) * H;
      else src = static_cast<const T*>(a.v) + static_cast<long long>(t) * (a.Nk * H) + (head - a.N - a.Nk) * H;
    } else {
      src = static_cast<const T*>(a.qkv) + static_cast<long long>(t) * (static_cast<long long>(heads) * H) + head * H;
    }
    T* dst;
    if (head < a.N) {
      dst = static_cast<T*>(a.q_out) + static_cast<long long>(t) * (a.N * H) + head * H;
    } else {
      if (!slot_ok) continue;  // slot_mapping -1: the token is not cached
      const bool is_k = head < a.N + a.Nk;
      const int kh = is_k ? head - a.N : head - a.N - a.Nk;
      dst = static_cast<T*>(is_k ? a.k_cache : a.v_cache) + (slot * a.Nk + kh) * H;
    }
    const bool rotate = a.do_rotary && head < a.N + a.Nk && i < half;
    int e0, e1;
    if (rotate) {
      e0 = a.interleaved ? 2 * i : i;
      e1 = a.interleaved ? 2 * i + 1 : i + half;
    } else if (a.do_rotary && head < a.N + a.Nk) {
      e0 = rot + 2 * (i - half);
      e1 = e0 + 1;
    } else {
      e0 = 2 * i;
      e1 = 2 * i + 1;
    }
    const float x0 = to_float<T>(src[e0]), x1 = to_float<T>(src[e1]);
    if (rotate) {
      const float c = to_float<T>(cosr[i]), sn = to_float<T>(sinr[i]);
      dst[e0] = from_float<T>(x0 * c - x1 * sn);
      dst[e1] = from_float<T>(x1 * c + x0 * sn);
    } else {
      dst[e0] = src[e0];
      dst[e1] = src[e1];
    }
  }
  pdl_launch_dependents();
}

// ---------------------------------------------------------------- decode
constexpr int kDecTile = 32;    // keys per pipeline stage
constexpr int kDecStages = 4;

template <typename T, int H, int G, bool PAGED>
__global__ void __launch_bounds__(128) gqa_decode_kernel(const DecodeParams p) {
  constexpr int DPL = H / 8;          // dims per lane (8 lanes share a key)
  constexpr int VEC = DPL * sizeof(T) / 16;  // 16-byte loads per lane per row
  constexpr int kRowBytes = H * sizeof(T);
  constexpr int kTileBytes = kDecTile * kRowBytes;
  static_assert(VEC >= 1, "head size too small");
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / p.gparts, gp = blockIdx.y % p.gparts;
  const int b = blockIdx.z;
  const int group = p.N / p.Nk;
  const int head0 = kvh * group + gp * G;       // first query head served here
  const int n_heads = min(G, group - gp * G);   // query heads actually present
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = lane >> 3, sub = lane & 7, d0 = sub * DPL;

  // K/V tiles stream through shared memory with bulk asynchronous copies (kDecStages tiles in flight per CTA)
  extern __shared__ __align__(128) uint8_t dec_smem[];
  uint8_t* stage_base = dec_smem;                                             // [stages][K tile | V tile]
  float* sm_acc = reinterpret_cast<float*>(dec_smem + kDecStages * 2 * kTileBytes);  // [4][G][H]
  float* sm_m = sm_acc + 4 * G * H;                                            // [4][G]
  float* sm_l = sm_m + 4 * G;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sm_l + 4 * G);
  __shared__ unsigned int sm_last;

  if (tid == 0) {
    for (int i = 0; i < kDecStages; ++i) mbar_init(&full_bar[i], 1);
    fence_mbar_init();
  }
  __syncthreads();

  pdl_wait_prior_grids();
  int total = p.seqlens_k[b] + 1;
  if (total > p.Smax || total < 0) {
    // a length beyond the cache capacity would read past the buffer: attend to what the cache holds and report it
    if (tid == 0 && p.status) atomicExch(p.status, kStatusBadLength);
    total = total < 0 ? 0 : p.Smax;
  }
  const int start0 = p.window > 0 ? max(0, total - p.window) : 0;
  const int len = max(total - start0, 0);
  const int chunk = (len + p.splits - 1) / p.splits;
  const int k_begin = start0 + split * chunk;
  const int k_end_all = min(total, k_begin + chunk);
  // fused prep: the newest key is not in the cache yet; the CTA whose range reaches it handles it from registers
  const bool owns_new = (p.qkv != nullptr) && k_end_all == total && k_begin < total;
  const int k_end = owns_new ? k_end_all - 1 : k_end_all;
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + kDecTile - 1) / kDecTile : 0;

  const T* kbase = static_cast<const T*>(p.k_cache) + (static_cast<long long>(b) * p.Nk + kvh) * p.Smax * H;
  const T* vbase = static_cast<const T*>(p.v_cache) + (static_cast<long long>(b) * p.Nk + kvh) * p.Smax * H;

  auto issue_tile = [&](int t) {
    const int s = t % kDecStages;
    const int key0 = k_begin + t * kDecTile;
    const int rows = min(kDecTile, k_end - key0);
    const uint32_t bytes = static_cast<uint32_t>(rows) * kRowBytes;
    uint8_t* dst = stage_base + s * 2 * kTileBytes;
    mbar_expect_tx(&full_bar[s], 2 * bytes);
    bulk_load(dst, kbase + static_cast<long long>(key0) * H, bytes, &full_bar[s]);
    bulk_load(dst + kTileBytes, vbase + static_cast<long long>(key0) * H, bytes, &full_bar[s]);
  };
  // paged cache: the rows of a tile are scattered over blocks, so the 32 lanes of warp 0 fetch one row pair each
  auto issue_tile_paged = [&](int t) {
    const int s = t % kDecStages;
    const int key0 = k_begin + t * kDecTile;
    const int rows = min(kDecTile, k_end - key0);
    uint8_t* dst = stage_base + s * 2 * kTileBytes;
    if (lane == 0) mbar_expect_tx(&full_bar[s], 2u * static_cast<uint32_t>(rows) * kRowBytes);
    __syncwarp();
    if (lane < rows) {
      const int key = key0 + lane;
      const int blk = p.block_table[static_cast<long long>(b) * p.max_blocks + key / p.block_size];
      const long long row = ((static_cast<long long>(blk) * p.block_size + key % p.block_size) * p.Nk + kvh) * H;
      bulk_load(dst + lane * kRowBytes, static_cast<const T*>(p.k_cache) + row, kRowBytes, &full_bar[s]);
      bulk_load(dst + kTileBytes + lane * kRowBytes, static_cast<const T*>(p.v_cache) + row, kRowBytes, &full_bar[s]);
    }
  };
  if (PAGED) {
    if (warp == 0) {
      const int pre = n_tiles < kDecStages ? n_tiles : kDecStages;
      for (int t = 0; t < pre; ++t) issue_tile_paged(t);
    }
  } else if (tid == 0) {
    const int pre = n_tiles < kDecStages ? n_tiles : kDecStages;
    for (int t = 0; t < pre; ++t) issue_tile(t);
  }

  const bool fused = p.qkv != nullptr;
  // rotary factors of the new position for this lane's dims (non-interleaved: dim i pairs with i +- H/2, held by the
  // lane 4 further on; interleaved: neighbouring dims, held by this lane)
  float rc[DPL], rs[DPL];
  if (fused && p.do_rotary) {
    const int rpos = p.cos_rows > 0 && total - 1 >= p.cos_rows ? p.cos_rows - 1 : (total > 0 ? total - 1 : 0);
    const T* cosr = static_cast<const T*>(p.cos_cache) + static_cast<long long>(rpos) * (H / 2);
    const T* sinr = static_cast<const T*>(p.sin_cache) + static_cast<long long>(rpos) * (H / 2);
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = d0 + i;
      const int fi = p.interleaved ? (d >> 1) : (d % (H / 2));
      rc[i] = to_float<T>(cosr[fi]);
      rs[i] = to_float<T>(sinr[fi]);
    }
  }
  // x[DPL] holds this lane's dims of one head vector; returns it rotated
  auto rope = [&](float* x) {
    if (p.interleaved) {
#pragma unroll
      for (int i = 0; i < DPL; i += 2) {
        const float a = x[i], bb = x[i + 1];
        x[i] = a * rc[i] - bb * rs[i];
        x[i + 1] = bb * rc[i + 1] + a * rs[i + 1];
      }
    } else {
      const bool upper = sub >= 4;  // dims [H/2, H)
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, x[i], 4);
        x[i] = upper ? x[i] * rc[i] + other * rs[i] : x[i] * rc[i] - other * rs[i];
      }
    }
  };
  const long long qkv_row = static_cast<long long>(b) * (p.N + 2 * p.Nk) * H;
  float qf[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int hd = head0 + (g < n_heads ? g : 0);
    const T* qp = fused ? static_cast<const T*>(p.qkv) + qkv_row + static_cast<long long>(hd) * H + d0
                        : static_cast<const T*>(p.q) + (static_cast<long long>(b) * p.N + hd) * H + d0;
    float x[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) x[i] = to_float<T>(qp[i]);
    if (fused && p.do_rotary) rope(x);
#pragma unroll
    for (int i = 0; i < DPL; ++i) qf[g][i] = x[i] * p.scale;
  }
  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = kNegBig;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }

  bool ok = true;
  for (int t = 0; t < n_tiles; ++t) {
    const int s = t % kDecStages;
    if (ok && !mbar_wait(&full_bar[s], (t / kDecStages) & 1)) ok = false;  // bounded; a failed wait skips the math below
    const uint8_t* ktile = stage_base + s * 2 * kTileBytes;
    const uint8_t* vtile = ktile + kTileBytes;
    const int key0 = k_begin + t * kDecTile;
    // 16 key slots per CTA (4 warps x 4 lane groups), two keys per slot per tile.  Everything below is
    // branch-free so that the 2 x G dot-product / shuffle / exp chains overlap (the loop is latency-bound).
    float kf[2][DPL], vf[2][DPL];
    bool valid[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int row = u * 16 + warp * 4 + slot;
      valid[u] = ok && (key0 + row) < k_end;
      const int rr = valid[u] ? row : 0;  // row 0 of a started tile always holds data
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        const uint4 kq = *reinterpret_cast<const uint4*>(ktile + rr * kRowBytes + d0 * sizeof(T) + v * 16);
        const uint4 vq = *reinterpret_cast<const uint4*>(vtile + rr * kRowBytes + d0 * sizeof(T) + v * 16);
        const T* kp = reinterpret_cast<const T*>(&kq);
        const T* vp = reinterpret_cast<const T*>(&vq);
#pragma unroll
        for (int i = 0; i < 16 / static_cast<int>(sizeof(T)); ++i) {
          kf[u][v * (16 / sizeof(T)) + i] = to_float<T>(kp[i]);
          vf[u][v * (16 / sizeof(T)) + i] = to_float<T>(vp[i]);
        }
      }
    }
    float sc[2][G];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float a0 = 0.f, a1 = 0.f;  // two partial sums halve the FMA dependency chain
#pragma unroll
        for (int i = 0; i < DPL; i += 2) {
          a0 += qf[g][i] * kf[u][i];
          a1 += qf[g][i + 1] * kf[u][i + 1];
        }
        sc[u][g] = a0 + a1;
      }
    }
#pragma unroll
    for (int off = 1; off <= 4; off <<= 1) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int g = 0; g < G; ++g) sc[u][g] += __shfl_xor_sync(0xffffffffu, sc[u][g], off);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s0 = sc[0][g], s1 = sc[1][g];
      if (p.softcap > 0.f) {
        s0 = p.softcap * tanhf(s0 / p.softcap);
        s1 = p.softcap * tanhf(s1 / p.softcap);
      }
      s0 = valid[0] ? s0 : kNegBig;
      s1 = valid[1] ? s1 : kNegBig;
      const float m_new = fmaxf(m[g], fmaxf(s0, s1));
      const float corr = __expf(m[g] - m_new);
      const float p0 = valid[0] ? __expf(s0 - m_new) : 0.f;
      const float p1 = valid[1] ? __expf(s1 - m_new) : 0.f;
      l[g] = l[g] * corr + p0 + p1;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[g][i] = acc[g][i] * corr + p0 * vf[0][i] + p1 * vf[1][i];
      m[g] = m_new;
    }
    __syncthreads();  // every warp is done with stage s
    if (PAGED) {
      if (warp == 0 && ok && t + kDecStages < n_tiles) issue_tile_paged(t + kDecStages);
    } else if (tid == 0 && ok && t + kDecStages < n_tiles) {
      issue_tile(t + kDecStages);
    }
  }
  if (!ok && tid == 0 && p.status) atomicExch(p.status, kStatusTimeoutEpilogue);

  if (owns_new) {
    // the new token: rotate its key, store key and value at cache position total - 1, attend to them.  All lanes run
    // the shuffles; only lane group 0 of warp 0 stores and accumulates.
    const T* kp = static_cast<const T*>(p.qkv) + qkv_row + static_cast<long long>(p.N + kvh) * H + d0;
    const T* vp = static_cast<const T*>(p.qkv) + qkv_row + static_cast<long long>(p.N + p.Nk + kvh) * H + d0;
    float kx[DPL], vx[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      kx[i] = to_float<T>(kp[i]);
      vx[i] = to_float<T>(vp[i]);
    }
    if (p.do_rotary) rope(kx);
    const bool mine = warp == 0 && slot == 0;
    if (mine) {
      long long row;
      if (PAGED) {
        const int key = total - 1;
        const int blk = p.block_table[static_cast<long long>(b) * p.max_blocks + key / p.block_size];
        row = ((static_cast<long long>(blk) * p.block_size + key % p.block_size) * p.Nk + kvh) * H;
      } else {
        row = ((static_cast<long long>(b) * p.Nk + kvh) * p.Smax + (total - 1)) * H;
      }
      T* kd = static_cast<T*>(const_cast<void*>(p.k_cache)) + row + d0;
      T* vd = static_cast<T*>(const_cast<void*>(p.v_cache)) + row + d0;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        kd[i] = from_float<T>(kx[i]);
        vd[i] = vp[i];
        kx[i] = to_float<T>(kd[i]);  // attend to the stored (rounded) key, as later steps will
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float a0 = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) a0 += qf[g][i] * kx[i];
#pragma unroll
      for (int off = 1; off <= 4; off <<= 1) a0 += __shfl_xor_sync(0xffffffffu, a0, off);
      if (p.softcap > 0.f) a0 = p.softcap * tanhf(a0 / p.softcap);
      if (mine) {
        const float m_new = fmaxf(m[g], a0);
        const float corr = __expf(m[g] - m_new);
        const float pr = __expf(a0 - m_new);
        l[g] = l[g] * corr + pr;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = acc[g][i] * corr + pr * vx[i];
        m[g] = m_new;
      }
    }
  }

  // merge the 4 key slots of a warp (lanes differing in bits 3 and 4)
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float m_new = fmaxf(m[g], m_o);
      const float c_s = safe_exp_diff(m[g], m_new), c_o = safe_exp_diff(m_o, m_new);
      l[g] = l[g] * c_s + l_o * c_o;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
        acc[g][i] = acc[g][i] * c_s + a_o * c_o;
      }
      m[g] = m_new;
    }
  }
  if (slot == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (sub == 0) {
        sm_m[warp * G + g] = m[g];
        sm_l[warp * G + g] = l[g];
      }
#pragma unroll
      for (int i = 0; i < DPL; ++i) sm_acc[(warp * G + g) * H + d0 + i] = acc[g][i];
    }
  }
  __syncthreads();

  // merge the 4 warps: thread t owns dim t (H <= 128 == blockDim)
  const int tile = (b * p.Nk + kvh) * p.gparts + gp;
  const bool owner = tid < H;
  float fm[G], fl[G], fa[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mm = kNegBig;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w * G + g]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = safe_exp_diff(sm_m[w * G + g], mm);
      ll += sm_l[w * G + g] * c;
      if (owner) aa += sm_acc[(w * G + g) * H + tid] * c;
    }
    fm[g] = mm;
    fl[g] = ll;
    fa[g] = aa;
  }

  decode_finish<T, H, G>(p, tile, split, b, head0, n_heads, tid, fm, fl, fa, &sm_last);
}


template <typename T, int H, int G, bool PAGED>
static int launch_decode_g(const DecodeParams& p, dim3 grid, cudaStream_t stream, bool use_pdl) {
  constexpr int kSmem = kDecStages * 2 * kDecTile * H * static_cast<int>(sizeof(T)) + (4 * G * H + 8 * G) * 4 + 8 * kDecStages;
  auto kern = gqa_decode_kernel<T, H, G, PAGED>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -10;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(128, 1, 1);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  if (use_pdl) {
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, p) == cudaSuccess ? 0 : -11;
}

template <typename T, int H>
static int launch_decode(const ortb200_gqa_decode_args* a, cudaStream_t stream) {
  const int group = a->N / a->Nk;
  const int G = group >= 4 ? 4 : (group >= 2 ? 2 : 1);
  const int gparts = (group + G - 1) / G;
  int splits = a->splits;
  if (splits <= 0) {
    // about three resident CTAs per SM, but at least two key tiles per CTA at full cache occupancy
    const int ctas = a->B * a->Nk * gparts;
    splits = (2 * 148) / ctas;  // one wave of (register-limited) two CTAs per SM
    const int max_by_len = (a->Smax + 2 * kDecTile - 1) / (2 * kDecTile);
    if (splits > max_by_len) splits = max_by_len;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
  }
  const int tiles = a->B * a->Nk * gparts;
  const int64_t need = 65536 + static_cast<int64_t>(tiles) * splits * G * (H + 4) * 4;
  if (splits > 1 && (!a->workspace || a->workspace_bytes < need || tiles > 16384)) splits = 1;
  DecodeParams p;
  p.q = a->q; p.k_cache = a->k_cache; p.v_cache = a->v_cache; p.seqlens_k = a->seqlens_k; p.head_sink = a->head_sink;
  p.out = a->out;
  p.counters = reinterpret_cast<unsigned int*>(a->workspace);
  p.ws = a->workspace ? reinterpret_cast<float*>(static_cast<char*>(a->workspace) + 65536) : nullptr;
  p.status = a->status;
  p.B = a->B; p.N = a->N; p.Nk = a->Nk; p.Smax = a->Smax; p.splits = splits; p.window = a->window; p.gparts = gparts;
  p.scale = a->scale != 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(H));
  p.softcap = a->softcap;
  p.block_table = a->block_table; p.block_size = a->block_size; p.max_blocks = a->max_blocks;
  p.qkv = a->qkv; p.cos_cache = a->cos_cache; p.sin_cache = a->sin_cache; p.cos_rows = a->cos_rows;
  p.prefetch = nullptr; p.prefetch_bytes = 0; p.prefetch_per_cta = 0;
  p.do_rotary = a->do_rotary; p.interleaved = a->rotary_interleaved;
  dim3 grid(splits, a->Nk * gparts, a->B);
  if (a->block_table) {
    if (G == 4) return launch_decode_g<T, H, 4, true>(p, grid, stream, a->use_pdl != 0);
    if (G == 2) return launch_decode_g<T, H, 2, true>(p, grid, stream, a->use_pdl != 0);
    return launch_decode_g<T, H, 1, true>(p, grid, stream, a->use_pdl != 0);
  }
  if (G == 4) return launch_decode_g<T, H, 4, false>(p, grid, stream, a->use_pdl != 0);
  if (G == 2) return launch_decode_g<T, H, 2, false>(p, grid, stream, a->use_pdl != 0);
  return launch_decode_g<T, H, 1, false>(p, grid, stream, a->use_pdl != 0);
}

}  // namespace ortb200

using namespace ortb200;

extern "C" int64_t ortb200_gqa_decode_workspace_bytes(int B, int N, int H) {
  // tiles * G <= B * N ; at most 32 splits
  return 65536 + static_cast<int64_t>(B) * N * 32 * (H + 4) * 4;
}

extern "C" int ortb200_gqa_decode(const ortb200_gqa_decode_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || (!a->q && !a->qkv) || !a->k_cache || !a->v_cache || !a->seqlens_k || !a->out) return -1;
  if (a->qkv && a->do_rotary && (!a->cos_cache || !a->sin_cache)) return -2;
  if (a->B <= 0 || a->N <= 0 || a->Nk <= 0 || a->N % a->Nk != 0 || a->Smax <= 0) return -1;
  if (a->block_table && (a->block_size <= 0 || a->max_blocks <= 0)) return -1;
  if (a->H != 64 && a->H != 128) return -2;
  if ((reinterpret_cast<uintptr_t>(a->k_cache) | reinterpret_cast<uintptr_t>(a->v_cache)) & 15) return -3;
  if (a->algo == 2 && !gqa_decode_tc_supported(a)) return -6;
  if (a->algo != 1 && gqa_decode_tc_supported(a)) return launch_gqa_decode_tc(a, stream);
  if (a->dtype == ORTB200_BF16) {
    return a->H == 128 ? launch_decode<__nv_bfloat16, 128>(a, stream) : launch_decode<__nv_bfloat16, 64>(a, stream);
  } else if (a->dtype == ORTB200_F16) {
    return a->H == 128 ? launch_decode<__half, 128>(a, stream) : launch_decode<__half, 64>(a, stream);
  }
  return -4;
}

extern "C" int ortb200_paged_prep(const ortb200_paged_prep_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->qkv || !a->q_out || !a->k_cache || !a->v_cache || !a->cu_seqlens || !a->past_seqlens) return -1;
  if (!a->slot_mapping && !a->block_table) return -1;
  if (a->T < 0 || a->B <= 0 || a->H % 2 != 0 || a->block_size <= 0 || a->num_blocks <= 0) return -1;
  if (a->do_rotary && (!a->cos_cache || !a->sin_cache)) return -2;
  if ((a->k != nullptr) != (a->v != nullptr)) return -2;
  const int rot = a->rot_dim > 0 ? a->rot_dim : a->H;
  if (rot > a->H || rot % 2 != 0) return -2;
  if (a->T == 0) return 0;
  if (a->dtype == ORTB200_BF16) paged_prep_kernel<__nv_bfloat16><<<a->T, 256, 0, stream>>>(*a);
  else if (a->dtype == ORTB200_F16) paged_prep_kernel<__half><<<a->T, 256, 0, stream>>>(*a);
  else return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_gqa_prep(const ortb200_gqa_prep_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->qkv || !a->q_out || !a->k_cache || !a->v_cache || !a->seqlens_k) return -1;
  if (a->B <= 0 || a->S <= 0 || a->H % 2 != 0) return -1;
  if (a->do_rotary && (!a->cos_cache || !a->sin_cache)) return -2;
  if ((a->k != nullptr) != (a->v != nullptr)) return -2;
  const int rot = a->rot_dim > 0 ? a->rot_dim : a->H;
  if (rot > a->H || rot % 2 != 0) return -2;
  const int tokens = a->B * a->S, heads = a->N + 2 * a->Nk;
  int ygroups = 1;
  if (tokens < 296) {
    ygroups = (296 + tokens - 1) / tokens;
    if (ygroups > heads) ygroups = heads;
  }
  dim3 grid(static_cast<unsigned>(tokens), static_cast<unsigned>(ygroups));
  const int threads = ygroups > 1 ? 128 : 256;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  if (a->use_pdl) {
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
  }
  cudaError_t e;
  if (a->dtype == ORTB200_BF16) e = cudaLaunchKernelEx(&cfg, gqa_prep_kernel<__nv_bfloat16>, *a);
  else if (a->dtype == ORTB200_F16) e = cudaLaunchKernelEx(&cfg, gqa_prep_kernel<__half>, *a);
  else return -4;
  return e == cudaSuccess ? 0 : -11;
}
