// LayerNorm / RMSNorm family with the residual add fused in:
//   s   = x (+ skip) (+ bias)            -> optionally written back as the residual stream
//   out = (s - mean) * rstd * gamma + beta     (LayerNorm)
//   out = s * rsqrt(mean(s^2) + eps) * gamma   (simplified / RMS)
// fp32 statistics, 16-byte vector loads, the row stays in registers between the
// two passes so every byte is read once and written once (HBM-bound).
//
// Replaces SkipLayerNormKernel(Small) and cuApplyLayerNorm of the reference
// (onnxruntime/contrib_ops/cuda/bert/skip_layer_norm_impl.cu:74-248,
// onnxruntime/core/providers/cuda/nn/layer_norm_impl.cu:438).
#include <cuda_runtime.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace ortb200 {

template <typename T>
struct Vec16 {
  static constexpr int kElems = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ float get(int i) const { return to_float<T>(reinterpret_cast<const T*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = from_float<T>(v); }
};

__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? smem[lane] : 0.0f;
  return warp_sum(t);
}

// VPT = 16-byte vectors per thread kept in registers; H == VPT * blockDim.x * kElems exactly or padded (guarded).
template <typename T, int VPT>
__global__ void __launch_bounds__(256) norm_kernel(const T* __restrict__ x, const T* __restrict__ skip,
                                                   const T* __restrict__ bias, const T* __restrict__ gamma,
                                                   const T* __restrict__ beta, T* __restrict__ out,
                                                   T* __restrict__ sum_out, int H, float eps, int simplified) {
  constexpr int E = Vec16<T>::kElems;
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * H;
  const T* sr = skip ? skip + row * H : nullptr;
  float vals[VPT][E];
  float s1 = 0.f, s2 = 0.f;
  pdl_wait_prior_grids();
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * E;
    if (col < H) {
      Vec16<T> a;
      a.raw = *reinterpret_cast<const uint4*>(xr + col);
#pragma unroll
      for (int i = 0; i < E; ++i) vals[v][i] = a.get(i);
      if (sr) {
        Vec16<T> b;
        b.raw = *reinterpret_cast<const uint4*>(sr + col);
#pragma unroll
        for (int i = 0; i < E; ++i) vals[v][i] += b.get(i);
      }
      if (bias) {
        Vec16<T> b;
        b.raw = *reinterpret_cast<const uint4*>(bias + col);
#pragma unroll
        for (int i = 0; i < E; ++i) vals[v][i] += b.get(i);
      }
      if (sum_out) {
        Vec16<T> o;
#pragma unroll
        for (int i = 0; i < E; ++i) {
          o.set(i, vals[v][i]);
          vals[v][i] = o.get(i);  // statistics see the stored (rounded) residual, as a later reader would
        }
        *reinterpret_cast<uint4*>(sum_out + row * H + col) = o.raw;
      }
#pragma unroll
      for (int i = 0; i < E; ++i) {
        s1 += vals[v][i];
        s2 += vals[v][i] * vals[v][i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < E; ++i) vals[v][i] = 0.f;
    }
  }
  pdl_launch_dependents();
  float mean = 0.f, rstd;
  if (simplified) {
    const float ms = block_sum(s2, red) / H;
    rstd = rsqrtf(ms + eps);
  } else {
    mean = block_sum(s1, red) / H;
    // two-pass variance from registers: numerically safer than E[x^2] - mean^2
    float sq = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int col = (v * blockDim.x + threadIdx.x) * E;
      if (col < H) {
#pragma unroll
        for (int i = 0; i < E; ++i) {
          const float d = vals[v][i] - mean;
          sq += d * d;
        }
      }
    }
    rstd = rsqrtf(block_sum(sq, red) / H + eps);
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * E;
    if (col < H) {
      Vec16<T> g, b, o;
      g.raw = *reinterpret_cast<const uint4*>(gamma + col);
      if (beta) b.raw = *reinterpret_cast<const uint4*>(beta + col);
#pragma unroll
      for (int i = 0; i < E; ++i) {
        float y = (vals[v][i] - mean) * rstd * g.get(i);
        if (beta) y += b.get(i);
        o.set(i, y);
      }
      *reinterpret_cast<uint4*>(out + row * H + col) = o.raw;
    }
  }
}

template <typename T>
static int launch_norm(const ortb200_norm_args* a, cudaStream_t stream) {
  constexpr int E = 16 / sizeof(T);
  const int H = a->hidden;
  if (H % E != 0) return -2;
  const int vecs = H / E;
  int threads = 256;
  if (vecs <= 32) threads = 32;
  else if (vecs <= 64) threads = 64;
  else if (vecs <= 128) threads = 128;
  const int vpt = (vecs + threads - 1) / threads;
  dim3 grid(static_cast<unsigned>(a->rows));
  const T* x = static_cast<const T*>(a->x);
  const T* skip = static_cast<const T*>(a->skip);
  const T* bias = static_cast<const T*>(a->bias);
  const T* gamma = static_cast<const T*>(a->gamma);
  const T* beta = static_cast<const T*>(a->beta);
  T* out = static_cast<T*>(a->out);
  T* sum_out = static_cast<T*>(a->sum_out);
#define ORTB200_NORM(V)                                                                                     \
  norm_kernel<T, V><<<grid, threads, 0, stream>>>(x, skip, bias, gamma, beta, out, sum_out, H, a->epsilon, a->simplified)
  if (vpt <= 1) ORTB200_NORM(1);
  else if (vpt <= 2) ORTB200_NORM(2);
  else if (vpt <= 4) ORTB200_NORM(4);
  else if (vpt <= 8) ORTB200_NORM(8);
  else if (vpt <= 16) ORTB200_NORM(16);
  else return -3;
#undef ORTB200_NORM
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ortb200

extern "C" int ortb200_norm(const ortb200_norm_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->x || !a->gamma || !a->out || a->rows < 0 || a->hidden <= 0) return -1;
  if (a->rows == 0) return 0;
  const uintptr_t align = reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->out) |
                          reinterpret_cast<uintptr_t>(a->gamma) | reinterpret_cast<uintptr_t>(a->skip) |
                          reinterpret_cast<uintptr_t>(a->bias) | reinterpret_cast<uintptr_t>(a->beta) |
                          reinterpret_cast<uintptr_t>(a->sum_out);
  if (align & 15) return -3;
  switch (a->dtype) {
    case ORTB200_F16: return ortb200::launch_norm<__half>(a, stream);
    case ORTB200_BF16: return ortb200::launch_norm<__nv_bfloat16>(a, stream);
    case ORTB200_F32: return ortb200::launch_norm<float>(a, stream);
    default: return -4;
  }
}
