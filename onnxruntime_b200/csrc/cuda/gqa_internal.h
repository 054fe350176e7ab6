// Shared by the two decode-attention kernels (CUDA-core split-KV kernel and the tcgen05 kernel): launch
// parameters and the tail that merges the splits and writes the output.
#pragma once
#include <cuda_runtime.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace ortb200 {

struct DecodeParams {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int* seqlens_k;
  const void* head_sink;
  void* out;
  float* ws;
  unsigned int* counters;
  int* status;
  int B, N, Nk, Smax, splits, window, gparts;
  float scale, softcap;
  // paged cache [num_blocks, block_size, Nk, H]: key j of sequence b lives in block block_table[b, j / block_size]
  const int* block_table;
  int block_size, max_blocks;
  // fused "unpack + rotary + append" (one new token per sequence): q, k and v are read from the packed projection
  // output qkv [B, (N + 2 Nk) H]; the CTA whose key range ends at the new position rotates the new key, writes
  // key and value into the cache and attends to them from registers
  const void* qkv;
  int cos_rows;
  const void* cos_cache;
  const void* sin_cache;
  int do_rotary, interleaved;
  // L2 prefetch of the next kernel's weights: CTA i asks for bytes [i, i + 1) * prefetch_per_cta of the range
  const unsigned char* prefetch;
  long long prefetch_bytes;
  int prefetch_per_cta;
};

// Running maxima start at a large negative finite value so that exp(m_old - m_new) never sees inf - inf.
constexpr float kNegBig = -1.0e30f;
__device__ __forceinline__ float safe_exp_diff(float a, float b) {
  return a <= kNegBig ? 0.f : __expf(a - b);
}


// tcgen05 decode kernel (gqa_decode_tc.cu)
bool gqa_decode_tc_supported(const ortb200_gqa_decode_args* a);
int launch_gqa_decode_tc(const ortb200_gqa_decode_args* a, cudaStream_t stream);

// Tail of a decode-attention CTA.  On entry thread tid < H holds, for each of the G query heads, its dim of the
// unnormalised output (fa), and every thread holds the running maximum (fm, natural-log domain) and the sum of
// exponentials (fl) of the CTA's key range.  With splits > 1 the state goes to the workspace and the CTA that
// arrives last on the tile's counter merges all splits; that CTA (or the only one) normalises and stores.
template <typename T, int H, int G>
__device__ __forceinline__ void decode_finish(const DecodeParams& p, int tile, int split, int b, int head0, int n_heads,
                                              int tid, float (&fm)[G], float (&fl)[G], float (&fa)[G],
                                              unsigned int* sm_last_ptr) {
  const bool owner = tid < H;
  unsigned int& sm_last = *sm_last_ptr;
  bool finalize = true;
  if (p.splits > 1) {
    // publish partial state: ws[tile][split][g][H + 2]
    float* my = p.ws + ((static_cast<size_t>(tile) * p.splits + split) * G) * (H + 2);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (owner) my[g * (H + 2) + tid] = fa[g];
      if (tid == 0) {
        my[g * (H + 2) + H] = fm[g];
        my[g * (H + 2) + H + 1] = fl[g];
      }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned int old = atomicAdd(&p.counters[tile], 1u);
      const unsigned int last = old == static_cast<unsigned int>(p.splits - 1) ? 1u : 0u;
      if (last) p.counters[tile] = 0;
      sm_last = last;
    }
    __syncthreads();
    finalize = sm_last != 0;
    if (finalize) {
      __threadfence();
      const float* base = p.ws + (static_cast<size_t>(tile) * p.splits * G) * (H + 2);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float mm = kNegBig;
        for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, __ldcg(&base[(s * G + g) * (H + 2) + H]));
        float ll = 0.f, aa = 0.f;
        for (int s = 0; s < p.splits; ++s) {
          const float* ps = base + (s * G + g) * (H + 2);
          const float c = safe_exp_diff(__ldcg(&ps[H]), mm);
          ll += __ldcg(&ps[H + 1]) * c;
          if (owner) aa += __ldcg(&ps[tid]) * c;
        }
        fm[g] = mm;
        fl[g] = ll;
        fa[g] = aa;
      }
    }
  }
  pdl_launch_dependents();
  if (finalize && owner) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (g >= n_heads) break;
      float ll = fl[g];
      if (p.head_sink) {
        const float sink = to_float<T>(static_cast<const T*>(p.head_sink)[head0 + g]);
        const float mm = fmaxf(fm[g], sink);
        const float c = safe_exp_diff(fm[g], mm);
        ll = ll * c + __expf(sink - mm);
        fa[g] *= c;
      }
      const float o = ll > 0.f ? fa[g] / ll : 0.f;
      static_cast<T*>(p.out)[(static_cast<long long>(b) * p.N + head0 + g) * H + tid] = from_float<T>(o);
    }
  }
}

}  // namespace ortb200
