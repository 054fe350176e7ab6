// Internal interface between the GEMM dispatcher (gemm_tcgen05.cu) and the decode-shaped kernel (gemm_smallm.cu).
#pragma once
#include <cuda_runtime.h>
#include "ortb200_kernels.h"

namespace ortb200 {

struct SmallGemmParams {
  int M, N, K;
  int num_kb;
  int cluster;       // CTAs per cluster == split-K factor
  int dual_offset;
  int dtype;
  int act;
  float alpha;
  void* out;
  long long ldo;
  const void* bias;
  const void* residual;
  long long ldr;
  int* status;
  // ---- fused all-reduce over peer memory (world > 1): see ortb200_symm_layout in ortb200_kernels.h
  int world, rank;
  void* peers[8];          // base of every rank's symmetric workspace (peers[rank] is the local one)
  long long staging_offset;  // bytes from the workspace base to staging[2][world][slot_elems] (64-bit words: value | epoch << 32)
  long long slot_elems;      // elements per (parity, source rank) slot, >= M * ldo
  unsigned int* epoch;       // local: number of completed fused launches
  unsigned int* done;        // local: CTAs finished in the current launch
  // ---- grouped mode (mixture of experts): blockIdx.y indexes a device-side tile list instead of a row block
  const int4* tile_info;     // {expert, first row, end row, unused}; null = ordinary GEMM
  const int* num_tiles;      // device scalar: entries of tile_info in use
  int w_rows_per_expert;     // rows of W (and entries of bias: N) that belong to one expert
  // ---- fused RMS normalisation of the activations (rms_eps > 0): out = (W x) / rms(x) with gamma folded into W
  float rms_eps;
  const void* x_rows;        // the activation matrix [M, K] itself (read with plain loads for the row statistics)
  // ---- packed 4-bit weights (NBITS kernels): per (weight tile, k-block) one contiguous 4864-byte blob
  const void* nbits_blob;
};

// Grouped GEMM over a device-side tile list (see ortb200_gemm_grouped).
int launch_gemm_grouped(const ortb200_gemm_grouped_args* a, cudaStream_t stream);
// The same on the persistent large-tile kernel (tile_rows 128 or 256).
int launch_gemm_grouped_large(const ortb200_gemm_grouped_args* a, cudaStream_t stream);

// Large-M GEMM on CTA pairs (gemm_2cta.cu): 256 x 256 tiles, tcgen05 cta_group::2.
int launch_gemm_2cta(const ortb200_gemm_args* a, cudaStream_t stream);
// Second half of the prefill-sized fused GEMM + all-reduce (collectives.cu): the products already sit in the scatter
// areas of the symmetric workspace (the GEMM epilogue pushed them there); adds them in rank order, adds the residual,
// replicates the sums and copies them to `out` [M, N].
int launch_allreduce_prescattered(const ortb200_gemm_args* a, cudaStream_t stream);
int launch_gemm_grouped_2cta(const ortb200_gemm_grouped_args* a, cudaStream_t stream);

// bn in {16, 32, 64}.  Returns 0 or a negative launch error; reports the cluster size and pipeline depth used.
int launch_gemm_smallm(const ortb200_gemm_args* a, int bn, cudaStream_t stream, int* cluster_out, int* stages_out);

#ifdef __CUDACC__
}  // namespace ortb200
#include "ptx_sm100.cuh"
namespace ortb200 {
// ---- epilogue store pass shared by the large-M GEMM kernels (device code)
template <int ACT>
__device__ __forceinline__ float act_const(float v) {
  if (ACT == ORTB200_ACT_GELU) return gelu_erf_fast(v);
  if (ACT == ORTB200_ACT_FASTGELU) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
  if (ACT == ORTB200_ACT_RELU) return fmaxf(v, 0.0f);
  if (ACT == ORTB200_ACT_SILU) return v / (1.0f + __expf(-v));
  if (ACT == ORTB200_ACT_QUICKGELU) return v / (1.0f + __expf(-1.702f * v));
  return v;
}

// One pass of the staged 16-bit tile -> global memory in 16-byte chunks, with activation and residual.
// stg[row][128] holds `rows` token rows starting at m_base by 128 output features starting at nrow0; STRIDE threads
// share the pass (thread et takes chunks et, et + STRIDE, ...).
struct StoreArgs {
  void* out;
  const void* residual;
  long long ldo, ldr;
  int N;
};

template <bool BF16, int ACT, int STRIDE>
__device__ __forceinline__ void store_pass(const StoreArgs& p, const uint16_t* stg, int rows, int et, int m_base, int m_end, int nrow0,
                                           bool vec_ok) {
  const bool has_res = p.residual != nullptr;
  for (int idx = et; idx < rows * 16; idx += STRIDE) {
    const int row = idx >> 4, ch = idx & 15;
    const int m = m_base + row;
    const int nn = nrow0 + ch * 8;
    if (m >= m_end || nn >= p.N) continue;
    const uint4 val = *reinterpret_cast<const uint4*>(stg + row * 128 + ch * 8);
    const long long o = static_cast<long long>(m) * p.ldo + nn;
    if (vec_ok && nn + 8 <= p.N) {
      uint4 res = val;
      if (has_res || ACT != ORTB200_ACT_NONE) {
        uint4 rr = make_uint4(0u, 0u, 0u, 0u);
        if (has_res)
          rr = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) + static_cast<long long>(m) * p.ldr + nn));
        const uint32_t a4[4] = {val.x, val.y, val.z, val.w};
        const uint32_t b4[4] = {rr.x, rr.y, rr.z, rr.w};
        uint32_t o4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi, rlo, rhi;
          if (BF16) {
            lo = __uint_as_float(a4[e] << 16); hi = __uint_as_float(a4[e] & 0xffff0000u);
            rlo = __uint_as_float(b4[e] << 16); rhi = __uint_as_float(b4[e] & 0xffff0000u);
          } else {
            const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&a4[e]));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&b4[e]));
            lo = fa.x; hi = fa.y; rlo = fb.x; rhi = fb.y;
          }
          lo = act_const<ACT>(lo) + rlo;
          hi = act_const<ACT>(hi) + rhi;
          if (BF16) {
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
            o4[e] = *reinterpret_cast<const uint32_t*>(&h2);
          } else {
            const __half2 h2 = __floats2half2_rn(lo, hi);
            o4[e] = *reinterpret_cast<const uint32_t*>(&h2);
          }
        }
        res = make_uint4(o4[0], o4[1], o4[2], o4[3]);
      }
      *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + o) = res;
    } else {
      const uint16_t* sv = stg + row * 128 + ch * 8;
      for (int e = 0; e < 8 && nn + e < p.N; ++e) {
        float y = BF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sv + e)) : __half2float(*reinterpret_cast<const __half*>(sv + e));
        y = act_const<ACT>(y);
        if (has_res) {
          const long long ri = static_cast<long long>(m) * p.ldr + nn + e;
          y += BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[ri]) : __half2float(reinterpret_cast<const __half*>(p.residual)[ri]);
        }
        if (BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[o + e] = __float2bfloat16_rn(y);
        else reinterpret_cast<__half*>(p.out)[o + e] = __float2half_rn(y);
      }
    }
  }
}

// Tensor-parallel variant of the store pass: instead of `out`, every 16-byte chunk of the staged tile goes straight to
// the rank that will reduce it - slice `g / row_vecs` of the flattened [M, N] product, at scatter[this rank][g % row_vecs]
// in that rank's symmetric workspace (the layout ortb200_symm_collective's all-reduce sums from).  Needs N % 8 == 0.
struct ScatterArgs {
  void* peers[8];
  long long area_offset;   // byte offset of the scatter area of this launch's parity within every workspace
  unsigned int row_vecs;   // 16-byte vectors per slice
  int rank, N;
};

template <int STRIDE>
__device__ __forceinline__ void scatter_pass(const ScatterArgs& p, const uint16_t* stg, int rows, int et, int m_base, int m_end, int nrow0) {
  for (int idx = et; idx < rows * 16; idx += STRIDE) {
    const int row = idx >> 4, ch = idx & 15;
    const int m = m_base + row;
    const int nn = nrow0 + ch * 8;
    if (m >= m_end || nn >= p.N) continue;
    const uint4 val = *reinterpret_cast<const uint4*>(stg + row * 128 + ch * 8);
    const unsigned int g = static_cast<unsigned int>((static_cast<long long>(m) * p.N + nn) >> 3);
    const unsigned int dst = g / p.row_vecs, i = g - dst * p.row_vecs;
    uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.peers[dst]) + p.area_offset) + static_cast<long long>(p.rank) * p.row_vecs + i;
    *d = val;
  }
}

template <bool BF16, int STRIDE>
__device__ __noinline__ void store_pass_act(const StoreArgs& p, int act, const uint16_t* stg, int rows, int et, int m_base, int m_end,
                                            int nrow0, bool vec_ok) {
  switch (act) {
    case ORTB200_ACT_GELU: store_pass<BF16, ORTB200_ACT_GELU, STRIDE>(p, stg, rows, et, m_base, m_end, nrow0, vec_ok); break;
    case ORTB200_ACT_FASTGELU: store_pass<BF16, ORTB200_ACT_FASTGELU, STRIDE>(p, stg, rows, et, m_base, m_end, nrow0, vec_ok); break;
    case ORTB200_ACT_RELU: store_pass<BF16, ORTB200_ACT_RELU, STRIDE>(p, stg, rows, et, m_base, m_end, nrow0, vec_ok); break;
    case ORTB200_ACT_SILU: store_pass<BF16, ORTB200_ACT_SILU, STRIDE>(p, stg, rows, et, m_base, m_end, nrow0, vec_ok); break;
    case ORTB200_ACT_QUICKGELU: store_pass<BF16, ORTB200_ACT_QUICKGELU, STRIDE>(p, stg, rows, et, m_base, m_end, nrow0, vec_ok); break;
    default: store_pass<BF16, ORTB200_ACT_NONE, STRIDE>(p, stg, rows, et, m_base, m_end, nrow0, vec_ok); break;
  }
}

#endif  // __CUDACC__

}  // namespace ortb200
