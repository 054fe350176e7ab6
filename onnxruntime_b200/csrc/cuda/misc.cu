// Small bandwidth-bound utility kernels: embedding row gather, arg-max over
// the vocabulary (greedy sampling), bias + activation, SwiGLU gating and the
// standalone rotary embedding.
//
// Reference counterparts: core/providers/cuda/tensor/gather_impl.cu,
// contrib_ops/cuda/transformers/greedy_search_top_one.cu:47,
// core/providers/cuda/tensor/gelu_approximate_impl.cu:40-119 (FastGelu),
// contrib_ops/cuda/math/bias_gelu_impl.cu:22, contrib_ops/cuda/bert/rotary_embedding_impl.cu:24.
#include <cuda_runtime.h>
#include <math.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace ortb200 {

__global__ void gather_rows_kernel(const uint4* __restrict__ table, const int64_t* __restrict__ ids, uint4* __restrict__ out,
                                   int64_t vocab, int vecs_per_row) {
  pdl_wait_prior_grids();
  const int64_t row = blockIdx.x;
  int64_t id = ids[row];
  if (id < 0) id += vocab;
  const bool ok = id >= 0 && id < vocab;
  for (int v = threadIdx.x; v < vecs_per_row; v += blockDim.x)
    out[row * vecs_per_row + v] = ok ? table[id * vecs_per_row + v] : make_uint4(0, 0, 0, 0);
  pdl_launch_dependents();
}

template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ x, int64_t* __restrict__ out, int64_t n) {
  __shared__ float sv[32];
  __shared__ int64_t si[32];
  pdl_wait_prior_grids();
  const T* row = x + static_cast<int64_t>(blockIdx.x) * n;
  float best = -INFINITY;
  int64_t best_i = 0x7fffffffffffffffLL;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float<T>(row[i]);
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    best_i = lane < nw ? si[lane] : 0x7fffffffffffffffLL;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffffffffffffLL ? 0 : best_i;
  }
  pdl_launch_dependents();
}

__device__ __forceinline__ float act_fn(int act, float v, float alpha) {
  switch (act) {
    case ORTB200_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    case ORTB200_ACT_FASTGELU: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
    case ORTB200_ACT_RELU: return fmaxf(v, 0.0f);
    case ORTB200_ACT_SILU: return v / (1.0f + __expf(-v));
    case ORTB200_ACT_QUICKGELU: return v / (1.0f + __expf(-alpha * v));
    default: return v;
  }
}

template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, int64_t total, int cols,
                                int act, float alpha) {
  pdl_wait_prior_grids();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    float v = to_float<T>(x[i]);
    if (bias) v += to_float<T>(bias[i % cols]);
    y[i] = from_float<T>(act_fn(act, v, alpha));
  }
  pdl_launch_dependents();
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols) {
  pdl_wait_prior_grids();
  const int64_t total = rows * cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / cols, c = i % cols;
    const float g = to_float<T>(x[r * 2 * cols + c]), u = to_float<T>(x[r * 2 * cols + cols + c]);
    y[i] = from_float<T>(g / (1.0f + __expf(-g)) * u);
  }
  pdl_launch_dependents();
}

template <typename T>
__global__ void rotary_kernel(const T* __restrict__ x, T* __restrict__ y, const int64_t* __restrict__ position_ids,
                              int64_t position_offset, const T* __restrict__ cos_cache, const T* __restrict__ sin_cache,
                              int B, int S, int N, int H, int rot, int interleaved, int bnsh) {
  // one block per (b, s, n); thread i handles one pair
  const int n = blockIdx.x % N, s = (blockIdx.x / N) % S, b = blockIdx.x / (N * S);
  const int half = rot / 2;
  const int64_t pos = position_ids ? position_ids[static_cast<int64_t>(b) * S + s] : position_offset + s;
  const int64_t off = bnsh ? ((static_cast<int64_t>(b) * N + n) * S + s) * H : ((static_cast<int64_t>(b) * S + s) * N + n) * H;
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
    int e0, e1;
    if (i < half) {
      e0 = interleaved ? 2 * i : i;
      e1 = interleaved ? 2 * i + 1 : i + half;
      const float c = to_float<T>(cos_cache[pos * half + i]), sn = to_float<T>(sin_cache[pos * half + i]);
      const float x0 = to_float<T>(x[off + e0]), x1 = to_float<T>(x[off + e1]);
      y[off + e0] = from_float<T>(x0 * c - x1 * sn);
      y[off + e1] = from_float<T>(x1 * c + x0 * sn);
    } else {
      e0 = rot + 2 * (i - half);
      e1 = e0 + 1;
      const T a0 = x[off + e0], a1 = x[off + e1];
      y[off + e0] = a0;
      y[off + e1] = a1;
    }
  }
}

static int grid_for(int64_t total, int threads) {
  int64_t blocks = (total + threads - 1) / threads;
  const int64_t cap = 148 * 16;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace ortb200

using namespace ortb200;

extern "C" int ortb200_gather_rows(const void* table, const int64_t* ids, void* out, int64_t n, int64_t vocab, int hidden,
                                   int elem_bytes, ortb200_stream_t stream) {
  if (!table || !ids || !out || n < 0 || hidden <= 0) return -1;
  if (n == 0) return 0;
  const int64_t row_bytes = static_cast<int64_t>(hidden) * elem_bytes;
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -3;
  const int vecs = static_cast<int>(row_bytes / 16);
  const int threads = vecs >= 256 ? 256 : (vecs >= 128 ? 128 : 64);
  gather_rows_kernel<<<static_cast<unsigned>(n), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(table), ids, static_cast<uint4*>(out), vocab, vecs);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_argmax(const void* x, int64_t* out, int64_t rows, int64_t n, int dtype, ortb200_stream_t stream) {
  if (!x || !out || rows < 0 || n <= 0) return -1;
  if (rows == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned g = static_cast<unsigned>(rows);
  if (dtype == ORTB200_BF16) argmax_kernel<__nv_bfloat16><<<g, 1024, 0, st>>>(static_cast<const __nv_bfloat16*>(x), out, n);
  else if (dtype == ORTB200_F16) argmax_kernel<__half><<<g, 1024, 0, st>>>(static_cast<const __half*>(x), out, n);
  else if (dtype == ORTB200_F32) argmax_kernel<float><<<g, 1024, 0, st>>>(static_cast<const float*>(x), out, n);
  else return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_bias_act(const void* x, const void* bias, void* y, int64_t rows, int cols, int act, float alpha,
                                int dtype, ortb200_stream_t stream) {
  if (!x || !y || rows < 0 || cols <= 0) return -1;
  if (rows == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * cols;
  const int g = grid_for(total, 256);
  if (dtype == ORTB200_BF16)
    bias_act_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(bias),
                                                      static_cast<__nv_bfloat16*>(y), total, cols, act, alpha);
  else if (dtype == ORTB200_F16)
    bias_act_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), static_cast<const __half*>(bias),
                                               static_cast<__half*>(y), total, cols, act, alpha);
  else if (dtype == ORTB200_F32)
    bias_act_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), static_cast<const float*>(bias),
                                              static_cast<float*>(y), total, cols, act, alpha);
  else return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_swiglu(const void* x, void* y, int64_t rows, int cols, int dtype, ortb200_stream_t stream) {
  if (!x || !y || rows < 0 || cols <= 0) return -1;
  if (rows == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = grid_for(rows * cols, 256);
  if (dtype == ORTB200_BF16)
    swiglu_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, cols);
  else if (dtype == ORTB200_F16)
    swiglu_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), rows, cols);
  else if (dtype == ORTB200_F32)
    swiglu_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), rows, cols);
  else return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_rotary(const void* x, void* y, const int64_t* position_ids, int64_t position_offset,
                              const void* cos_cache, const void* sin_cache, int B, int S, int N, int H, int rot_dim,
                              int interleaved, int bnsh, int dtype, ortb200_stream_t stream) {
  if (!x || !y || !cos_cache || !sin_cache || B <= 0 || S <= 0 || N <= 0 || H <= 0 || H % 2) return -1;
  const int rot = rot_dim > 0 ? rot_dim : H;
  if (rot > H || rot % 2) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned g = static_cast<unsigned>(B) * S * N;
  const int threads = H / 2 >= 64 ? 64 : 32;
  if (dtype == ORTB200_BF16)
    rotary_kernel<__nv_bfloat16><<<g, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), position_ids,
                                                        position_offset, static_cast<const __nv_bfloat16*>(cos_cache),
                                                        static_cast<const __nv_bfloat16*>(sin_cache), B, S, N, H, rot, interleaved, bnsh);
  else if (dtype == ORTB200_F16)
    rotary_kernel<__half><<<g, threads, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), position_ids, position_offset,
                                                 static_cast<const __half*>(cos_cache), static_cast<const __half*>(sin_cache), B, S, N, H,
                                                 rot, interleaved, bnsh);
  else if (dtype == ORTB200_F32)
    rotary_kernel<float><<<g, threads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), position_ids, position_offset,
                                                static_cast<const float*>(cos_cache), static_cast<const float*>(sin_cache), B, S, N, H, rot,
                                                interleaved, bnsh);
  else return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
