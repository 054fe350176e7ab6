// Mixture-of-experts plumbing for sm_100a: routing, the device-side tile plan for the grouped GEMM, the token
// permutation and the weighted combine.  Nothing here reads a count back to the host, so a MoE layer is a fixed
// sequence of launches that a CUDA graph can hold.
//
// Reference counterparts: the softmax + top-k router, permutation and finalize kernels of
// onnxruntime/contrib_ops/cuda/moe/ft_moe/moe_kernel.cu (topk_gating_softmax, initialize_moe_routing,
// finalize_moe_routing) and the op contract in onnxruntime/contrib_ops/cuda/moe/moe.cc.
#include <cuda_runtime.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace ortb200 {
namespace {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

// One warp per token: softmax over the expert logits, the k largest probabilities (ties: lower expert index),
// optional renormalisation over the chosen k, and the per-expert histogram.
template <typename T>
__global__ void __launch_bounds__(128) moe_route_kernel(const T* __restrict__ logits, int tokens, int E, int k, int normalize,
                                                        int expert_begin, int expert_end, int* __restrict__ topk_idx,
                                                        float* __restrict__ topk_w, int* __restrict__ counts) {
  pdl_wait_prior_grids();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= tokens) return;
  constexpr int PER = kMaxExperts / 32;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? to_float<T>(logits[static_cast<long long>(t) * E + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (i * 32 + lane) < E ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  float chosen_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    // warp arg-max over the remaining probabilities
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (e < E && (v[i] > best)) {
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;  // taken
    if (lane == j) {
      my_w = best * inv;
      my_e = best_e;
    }
    chosen_sum += best * inv;
  }
  if (lane < k) {
    if (normalize) my_w /= chosen_sum;
    topk_idx[t * k + lane] = my_e;
    topk_w[t * k + lane] = my_w;
    if (my_e >= expert_begin && my_e < expert_end) atomicAdd(&counts[my_e - expert_begin], 1);
  }
}

// One CTA: exclusive scan of the per-expert counts, the tile list of the grouped GEMM, and zeroed cursors.
__global__ void __launch_bounds__(256) moe_plan_kernel(const int* __restrict__ counts, int E_local, int tile_rows, int max_tiles,
                                                       int* __restrict__ offsets, int* __restrict__ cursors,
                                                       int4* __restrict__ tile_info, int* __restrict__ num_tiles) {
  __shared__ int s_off[kMaxExperts + 1], s_tile[kMaxExperts + 1];
  pdl_wait_prior_grids();
  if (threadIdx.x == 0) {
    int acc = 0, tacc = 0;
    for (int e = 0; e < E_local; ++e) {
      s_off[e] = acc;
      s_tile[e] = tacc;
      acc += counts[e];
      tacc += (counts[e] + tile_rows - 1) / tile_rows;
    }
    s_off[E_local] = acc;
    s_tile[E_local] = tacc;
    *num_tiles = tacc < max_tiles ? tacc : max_tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E_local; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E_local) cursors[e] = 0;
  }
  for (int e = threadIdx.x; e < E_local; e += blockDim.x) {
    const int first = s_off[e], end = s_off[e + 1];
    int ti = s_tile[e];
    for (int r = first; r < end && ti < max_tiles; r += tile_rows, ++ti) tile_info[ti] = make_int4(e, r, min(end, r + tile_rows), 0);
  }
}

// One CTA per (token, choice): claim a row in the expert's segment and copy the token there.
__global__ void __launch_bounds__(128) moe_permute_kernel(const uint4* __restrict__ x, int vecs_per_row, int k, int expert_begin,
                                                          int expert_end, const int* __restrict__ topk_idx,
                                                          const int* __restrict__ offsets, int* __restrict__ cursors,
                                                          uint4* __restrict__ xp, int* __restrict__ row_of) {
  __shared__ int s_row;
  pdl_wait_prior_grids();
  const int tj = blockIdx.x;
  const int e = topk_idx[tj];
  if (e < expert_begin || e >= expert_end) {
    if (threadIdx.x == 0) row_of[tj] = -1;  // another rank's expert
    return;
  }
  if (threadIdx.x == 0) {
    const int le = e - expert_begin;
    s_row = offsets[le] + atomicAdd(&cursors[le], 1);
    row_of[tj] = s_row;
  }
  __syncthreads();
  const long long src = static_cast<long long>(tj / k) * vecs_per_row, dst = static_cast<long long>(s_row) * vecs_per_row;
  for (int v = threadIdx.x; v < vecs_per_row; v += blockDim.x) xp[dst + v] = x[src + v];
}

// One CTA per token: out[t] = sum_j w[t, j] * (y[row_of[t, j]] + bias[expert(t, j)]) in the order j = 0 .. k-1.
// Rows move as 16-byte vectors (H is a multiple of 8), all k rows of a vector in flight before the first add.
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* __restrict__ y, const T* __restrict__ bias, int H, int k,
                                                          int expert_begin, const int* __restrict__ topk_idx,
                                                          const float* __restrict__ topk_w, const int* __restrict__ row_of,
                                                          T* __restrict__ out) {
  pdl_wait_prior_grids();
  const int t = blockIdx.x;
  constexpr int EPV = 16 / static_cast<int>(sizeof(T));
  const int hvecs = H / EPV;
  int rows[kMaxTopK];
  float ws[kMaxTopK];
  int experts[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) {
    rows[j] = j < k ? row_of[t * k + j] : -1;
    ws[j] = j < k ? topk_w[t * k + j] : 0.f;
    experts[j] = j < k ? topk_idx[t * k + j] - expert_begin : 0;
  }
  for (int hv = threadIdx.x; hv < hvecs; hv += blockDim.x) {
    uint4 v[kMaxTopK], b[kMaxTopK];
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) {
      v[j] = rows[j] >= 0 ? __ldg(reinterpret_cast<const uint4*>(y + static_cast<long long>(rows[j]) * H) + hv) : make_uint4(0u, 0u, 0u, 0u);
      b[j] = (bias != nullptr && rows[j] >= 0) ? __ldg(reinterpret_cast<const uint4*>(bias + static_cast<long long>(experts[j]) * H) + hv)
                                                : make_uint4(0u, 0u, 0u, 0u);
    }
    float acc[EPV];
#pragma unroll
    for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) {
      if (rows[j] < 0) continue;
      const T* ve = reinterpret_cast<const T*>(&v[j]);
      const T* be = reinterpret_cast<const T*>(&b[j]);
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] += ws[j] * (to_float<T>(ve[e]) + to_float<T>(be[e]));
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < EPV; ++e) oe[e] = from_float<T>(acc[e]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[hv] = o;
  }
}

}  // namespace
}  // namespace ortb200

using namespace ortb200;

extern "C" int ortb200_moe_tile_rows(int64_t rows, int experts) {
  const int64_t per = experts > 0 ? rows / experts : rows;
  if (per <= 16) return 16;
  if (per <= 32) return 32;
  if (per <= 96) return 64;
  return per <= 512 ? 128 : 256;  // prompt-sized batches: the large-tile persistent kernel
}

extern "C" int ortb200_moe_max_tiles(int64_t rows, int experts, int tile_rows) {
  return static_cast<int>((rows + tile_rows - 1) / tile_rows + experts);
}

extern "C" int ortb200_moe_route(const ortb200_moe_route_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->logits || !a->x || !a->topk_idx || !a->topk_w || !a->counts || !a->offsets || !a->cursors || !a->tile_info ||
      !a->num_tiles || !a->xp || !a->row_of)
    return -1;
  if (a->tokens <= 0 || a->E <= 0 || a->E > kMaxExperts || a->k <= 0 || a->k > kMaxTopK || a->k > a->E) return -2;
  if (a->expert_begin < 0 || a->expert_end > a->E || a->expert_end <= a->expert_begin) return -2;
  if ((a->H * 2) % 16 != 0 || ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->xp)) & 15)) return -3;
  if (a->tile_rows != 16 && a->tile_rows != 32 && a->tile_rows != 64 && a->tile_rows != 128 && a->tile_rows != 256) return -2;
  const int E_local = a->expert_end - a->expert_begin;
  if (cudaMemsetAsync(a->counts, 0, sizeof(int) * E_local, stream) != cudaSuccess) return -11;
  const unsigned gblocks = static_cast<unsigned>((a->tokens + 3) / 4);
  if (a->dtype == ORTB200_BF16)
    moe_route_kernel<__nv_bfloat16><<<gblocks, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(a->logits), a->tokens, a->E, a->k,
                                                                 a->normalize, a->expert_begin, a->expert_end, a->topk_idx, a->topk_w, a->counts);
  else if (a->dtype == ORTB200_F16)
    moe_route_kernel<__half><<<gblocks, 128, 0, stream>>>(static_cast<const __half*>(a->logits), a->tokens, a->E, a->k, a->normalize,
                                                          a->expert_begin, a->expert_end, a->topk_idx, a->topk_w, a->counts);
  else if (a->dtype == ORTB200_F32)
    moe_route_kernel<float><<<gblocks, 128, 0, stream>>>(static_cast<const float*>(a->logits), a->tokens, a->E, a->k, a->normalize,
                                                         a->expert_begin, a->expert_end, a->topk_idx, a->topk_w, a->counts);
  else
    return -4;
  moe_plan_kernel<<<1, 256, 0, stream>>>(a->counts, E_local, a->tile_rows, a->max_tiles, a->offsets, a->cursors,
                                         static_cast<int4*>(a->tile_info), a->num_tiles);
  moe_permute_kernel<<<static_cast<unsigned>(a->tokens * a->k), 128, 0, stream>>>(
      static_cast<const uint4*>(a->x), a->H * 2 / 16, a->k, a->expert_begin, a->expert_end, a->topk_idx, a->offsets, a->cursors,
      static_cast<uint4*>(a->xp), a->row_of);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_moe_combine(const void* y, const void* bias, void* out, int tokens, int H, int k, int expert_begin,
                                   const int* topk_idx, const float* topk_w, const int* row_of, int dtype, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!y || !out || !topk_idx || !topk_w || !row_of || tokens <= 0 || H <= 0 || k <= 0 || k > kMaxTopK) return -1;
  if (H % 8 != 0 || ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15)) return -3;
  if (dtype == ORTB200_BF16)
    moe_combine_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(bias), H, k,
                                                                  expert_begin, topk_idx, topk_w, row_of, static_cast<__nv_bfloat16*>(out));
  else if (dtype == ORTB200_F16)
    moe_combine_kernel<__half><<<tokens, 256, 0, stream>>>(static_cast<const __half*>(y), static_cast<const __half*>(bias), H, k, expert_begin,
                                                           topk_idx, topk_w, row_of, static_cast<__half*>(out));
  else
    return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
