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

// Orderable 64-bit key: larger value wins, ties go to the smaller index.
__device__ __forceinline__ unsigned long long argmax_key(float v, long long idx) {
  unsigned int u = __float_as_uint(v + 0.0f);  // -0.0 + 0.0 = +0.0: the two zeros compare equal, the first index wins
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return (static_cast<unsigned long long>(u) << 32) | static_cast<unsigned long long>(0xFFFFFFFFu - static_cast<unsigned int>(idx));
}

// grid (chunks, rows).  Each CTA reduces its chunk, merges into ws[row] with a 64-bit atomicMax, and the CTA
// that arrives last on counters[row] writes the index and leaves ws / counters zeroed for the next launch.
template <typename T>
__global__ void __launch_bounds__(256) argmax_kernel(const T* __restrict__ x, int64_t* __restrict__ out, int64_t n,
                                                     unsigned long long* __restrict__ ws, unsigned int* __restrict__ counters) {
  __shared__ unsigned long long sk[8];
  pdl_wait_prior_grids();
  const int64_t rowi = blockIdx.y;
  const T* row = x + rowi * n;
  const int64_t per = (n + gridDim.x - 1) / gridDim.x;
  const int64_t lo = blockIdx.x * per, hi = lo + per < n ? lo + per : n;
  unsigned long long best = 0;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = to_float<T>(row[i]);
    if (v == v) {  // NaN never wins
      const unsigned long long k = argmax_key(v, i);
      best = k > best ? k : best;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
    best = ok > best ? ok : best;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sk[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) best = sk[w] > best ? sk[w] : best;
    atomicMax(&ws[rowi], best);
    __threadfence();
    const unsigned int old = atomicAdd(&counters[rowi], 1u);
    if (old == gridDim.x - 1) {
      __threadfence();
      const unsigned long long k = atomicExch(&ws[rowi], 0ull);
      counters[rowi] = 0;
      out[rowi] = k == 0 ? 0 : static_cast<int64_t>(0xFFFFFFFFu - static_cast<unsigned int>(k & 0xFFFFFFFFull));
    }
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

// 16-bit types, cols a multiple of 8: one thread combines 8 gate values with 8 up values (16-byte accesses)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_vec8_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t rows, int cols8) {
  pdl_wait_prior_grids();
  const int64_t total = rows * cols8;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / cols8, c = i % cols8;
    const uint4 g4 = x[r * 2 * cols8 + c], u4 = x[r * 2 * cols8 + cols8 + c];
    const T* g = reinterpret_cast<const T*>(&g4);
    const T* u = reinterpret_cast<const T*>(&u4);
    __align__(16) T o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gv = to_float<T>(g[e]);
      o[e] = from_float<T>(gv / (1.0f + __expf(-gv)) * to_float<T>(u[e]));
    }
    y[i] = *reinterpret_cast<const uint4*>(o);
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

extern "C" int64_t ortb200_argmax_workspace_bytes(int64_t rows) { return rows * 16; }

extern "C" int ortb200_argmax(const void* x, int64_t* out, int64_t rows, int64_t n, int dtype, void* workspace,
                              int64_t workspace_bytes, ortb200_stream_t stream) {
  if (!x || !out || rows < 0 || n <= 0 || n > 0xFFFFFFFFll) return -1;
  if (rows == 0) return 0;
  if (!workspace || workspace_bytes < rows * 16 || (reinterpret_cast<uintptr_t>(workspace) & 7)) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned long long* ws = static_cast<unsigned long long*>(workspace);
  unsigned int* counters = reinterpret_cast<unsigned int*>(ws + rows);
  int chunks = static_cast<int>((n + 4095) / 4096);
  const int64_t want = (2 * 148 + rows - 1) / rows;
  if (chunks > want) chunks = static_cast<int>(want);
  if (chunks < 1) chunks = 1;
  dim3 g(static_cast<unsigned>(chunks), static_cast<unsigned>(rows));
  if (dtype == ORTB200_BF16) argmax_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), out, n, ws, counters);
  else if (dtype == ORTB200_F16) argmax_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), out, n, ws, counters);
  else if (dtype == ORTB200_F32) argmax_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), out, n, ws, counters);
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
  if (dtype != ORTB200_F32 && cols % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    const int gv = grid_for(rows * (cols / 8), 256);
    if (dtype == ORTB200_BF16)
      swiglu_vec8_kernel<__nv_bfloat16><<<gv, 256, 0, st>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y), rows, cols / 8);
    else
      swiglu_vec8_kernel<__half><<<gv, 256, 0, st>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y), rows, cols / 8);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
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
