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

// ---------------------------------------------------------------------------------------------------------------
// EmbedLayerNormalization: out[b, s, :] = LayerNorm(word[ids[b, s]] + pos[position] + seg[segment_ids[b, s]]).
// One block per token; the three rows are gathered with 16-byte loads, summed in registers, normalised with fp32
// statistics and written once (reference: EmbedLayerNormKernel, contrib_ops/cuda/bert/embed_layer_norm_impl.cu:123).
namespace ortb200 {

template <typename T, int VPT>
__global__ void __launch_bounds__(128) embed_layernorm_kernel(const ortb200_embed_layernorm_args a) {
  constexpr int E = Vec16<T>::kElems;
  __shared__ float red[32];
  const int64_t tok = blockIdx.x;
  const int H = a.hidden;
  const int s = static_cast<int>(tok % a.S);
  auto id_at = [&](const void* p, int64_t i) -> int64_t {
    return a.id_bytes == 8 ? static_cast<const int64_t*>(p)[i] : static_cast<int64_t>(static_cast<const int32_t*>(p)[i]);
  };
  int64_t wid = id_at(a.input_ids, tok);
  int64_t pid = a.position_ids ? id_at(a.position_ids, a.position_broadcast ? s : tok) : s;
  int64_t sid = (a.segment_ids && a.segment_emb) ? id_at(a.segment_ids, tok) : -1;
  // ids outside the tables read row 0 and flag the launch (the reference fails the run on such ids)
  if (wid < 0 || wid >= a.word_rows || pid < 0 || pid >= a.pos_rows || (sid >= a.seg_rows)) {
    if (a.status && threadIdx.x == 0) atomicExch(a.status, kStatusBadArgument);
    wid = wid < 0 || wid >= a.word_rows ? 0 : wid;
    pid = pid < 0 || pid >= a.pos_rows ? 0 : pid;
    sid = sid >= a.seg_rows ? 0 : sid;
  }
  const T* wr = static_cast<const T*>(a.word_emb) + wid * H;
  const T* pr = static_cast<const T*>(a.pos_emb) + pid * H;
  const T* sr = sid >= 0 ? static_cast<const T*>(a.segment_emb) + sid * H : nullptr;
  float vals[VPT][E];
  float s1 = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * E;
    if (col < H) {
      Vec16<T> w, p, g;
      w.raw = *reinterpret_cast<const uint4*>(wr + col);
      p.raw = *reinterpret_cast<const uint4*>(pr + col);
      if (sr) g.raw = *reinterpret_cast<const uint4*>(sr + col);
#pragma unroll
      for (int i = 0; i < E; ++i) {
        // the sum is rounded to T first, as the reference does before normalising (and as embedding_sum stores it)
        const float e = to_float<T>(from_float<T>(w.get(i) + p.get(i) + (sr ? g.get(i) : 0.f)));
        vals[v][i] = e;
        s1 += e;
      }
      if (a.sum_out) {
        Vec16<T> o;
#pragma unroll
        for (int i = 0; i < E; ++i) o.set(i, vals[v][i]);
        *reinterpret_cast<uint4*>(static_cast<T*>(a.sum_out) + tok * H + col) = o.raw;
      }
    } else {
#pragma unroll
      for (int i = 0; i < E; ++i) vals[v][i] = 0.f;
    }
  }
  const float mean = block_sum(s1, red) / static_cast<float>(H);
  float s2 = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * E;
    if (col < H) {
#pragma unroll
      for (int i = 0; i < E; ++i) {
        const float c = vals[v][i] - mean;
        s2 += c * c;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(s2, red) / static_cast<float>(H) + a.epsilon);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int col = (v * blockDim.x + threadIdx.x) * E;
    if (col < H) {
      Vec16<T> g, bt, o;
      g.raw = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.gamma) + col);
      bt.raw = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.beta) + col);
#pragma unroll
      for (int i = 0; i < E; ++i) o.set(i, (vals[v][i] - mean) * rstd * g.get(i) + bt.get(i));
      *reinterpret_cast<uint4*>(static_cast<T*>(a.out) + tok * H + col) = o.raw;
    }
  }
}

template <typename T>
int launch_embed_ln(const ortb200_embed_layernorm_args* a, cudaStream_t stream) {
  constexpr int E = Vec16<T>::kElems;
  if (a->hidden % E != 0) return -3;
  const int per_pass = 128 * E;
  const int vpt = (a->hidden + per_pass - 1) / per_pass;
  const dim3 grid(static_cast<unsigned>(a->B) * static_cast<unsigned>(a->S));
  switch (vpt) {
    case 1: embed_layernorm_kernel<T, 1><<<grid, 128, 0, stream>>>(*a); break;
    case 2: embed_layernorm_kernel<T, 2><<<grid, 128, 0, stream>>>(*a); break;
    case 3: case 4: embed_layernorm_kernel<T, 4><<<grid, 128, 0, stream>>>(*a); break;
    default: return -2;   // hidden sizes above 4096 (fp16) take the generic path
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ortb200

extern "C" int ortb200_embed_layernorm(const ortb200_embed_layernorm_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->input_ids || !a->word_emb || !a->pos_emb || !a->gamma || !a->beta || !a->out) return -1;
  if (a->B <= 0 || a->S <= 0 || a->hidden <= 0 || (a->id_bytes != 4 && a->id_bytes != 8)) return -1;
  const uintptr_t align = reinterpret_cast<uintptr_t>(a->word_emb) | reinterpret_cast<uintptr_t>(a->pos_emb) |
                          reinterpret_cast<uintptr_t>(a->segment_emb) | reinterpret_cast<uintptr_t>(a->gamma) |
                          reinterpret_cast<uintptr_t>(a->beta) | reinterpret_cast<uintptr_t>(a->out) |
                          reinterpret_cast<uintptr_t>(a->sum_out);
  if (align & 15) return -3;
  switch (a->dtype) {
    case ORTB200_F16: return ortb200::launch_embed_ln<__half>(a, stream);
    case ORTB200_BF16: return ortb200::launch_embed_ln<__nv_bfloat16>(a, stream);
    case ORTB200_F32: return ortb200::launch_embed_ln<float>(a, stream);
    default: return -4;
  }
}
