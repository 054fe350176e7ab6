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
int launch_gemm_grouped_2cta(const ortb200_gemm_grouped_args* a, cudaStream_t stream);

// bn in {16, 32, 64}.  Returns 0 or a negative launch error; reports the cluster size and pipeline depth used.
int launch_gemm_smallm(const ortb200_gemm_args* a, int bn, cudaStream_t stream, int* cluster_out, int* stages_out);

}  // namespace ortb200
