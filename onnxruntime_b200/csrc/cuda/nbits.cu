// MatMulNBits support for sm_100a: block-quantised int4 / int8 weights -> bf16 / fp16 rows.
//
// Reference counterparts: Dequantize4Bits / DequantizeBlockwise
// (onnxruntime/contrib_ops/cuda/quantization/dequantize_blockwise.cu) and the
// weight layout of MatMulNBits (docs/ContribOperators.md, "com.microsoft.MatMulNBits"):
//   B      uint8 [N, n_blocks, block_size * bits / 8]   low nibble = even k
//   scales T     [N, n_blocks]
//   zp     uint8 [N, ceil(n_blocks * bits / 8)] packed like B, or T [N, n_blocks]; default 2^(bits-1)
//   W[n, k] = (q[n, k] - zp[n, k / block_size]) * scales[n, k / block_size]
//
// One thread expands 8 consecutive weights (a 32-bit word of nibbles, or 8 bytes) and writes 16 bytes, so both the
// packed read and the expanded write are fully coalesced; the kernel runs at the write bandwidth of the output.
#include <cuda_runtime.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace ortb200 {
namespace {

template <typename T, int BITS>
__global__ void __launch_bounds__(256) nbits_dequant_kernel(const uint8_t* __restrict__ B, const T* __restrict__ scales,
                                                            const uint8_t* __restrict__ zp_packed, const T* __restrict__ zp_full,
                                                            T* __restrict__ out, int64_t N, int K, int block_size, int n_blocks,
                                                            int64_t ldo) {
  pdl_wait_prior_grids();
  const int groups_per_row = (K + 7) / 8;
  const int64_t total = N * groups_per_row;
  const int blob = block_size * BITS / 8;  // bytes per block
  const int zp_row = (n_blocks * BITS + 7) / 8;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total;
       g += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = g / groups_per_row;
    const int k0 = static_cast<int>(g % groups_per_row) * 8;
    const int blk = k0 / block_size, in_blk = k0 % block_size;  // block_size >= 16 and a power of two: 8 weights share a block
    const float s = to_float<T>(scales[n * n_blocks + blk]);
    float z;
    if (zp_full) {
      z = to_float<T>(zp_full[n * n_blocks + blk]);
    } else if (zp_packed) {
      if (BITS == 4) {
        const uint8_t zb = zp_packed[n * zp_row + (blk >> 1)];
        z = static_cast<float>((blk & 1) ? (zb >> 4) : (zb & 0xF));
      } else {
        z = static_cast<float>(zp_packed[n * zp_row + blk]);
      }
    } else {
      z = static_cast<float>(1 << (BITS - 1));
    }
    const uint8_t* src = B + (n * n_blocks + blk) * blob + in_blk * BITS / 8;
    float w[8];
    if (BITS == 4) {
      const uint32_t q = *reinterpret_cast<const uint32_t*>(src);
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = (static_cast<float>((q >> (4 * i)) & 0xF) - z) * s;
    } else {
      const uint2 q = *reinterpret_cast<const uint2*>(src);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w[i] = (static_cast<float>((q.x >> (8 * i)) & 0xFF) - z) * s;
        w[4 + i] = (static_cast<float>((q.y >> (8 * i)) & 0xFF) - z) * s;
      }
    }
    T* dst = out + n * ldo + k0;
    if (k0 + 8 <= K) {
      __align__(16) T v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = from_float<T>(w[i]);
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
    } else {
      for (int i = 0; i < 8 && k0 + i < K; ++i) dst[i] = from_float<T>(w[i]);
    }
  }
  pdl_launch_dependents();
}

__global__ void __launch_bounds__(256) nbits_prepack_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int64_t words) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint32_t w = in[i];
    uint32_t o = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o |= ((w >> (8 * j)) & 0xFu) << (4 * j);             // weight 2j   (low nibble of byte j)
      o |= ((w >> (8 * j + 4)) & 0xFu) << (16 + 4 * j);    // weight 2j+1 (high nibble of byte j)
    }
    out[i] = o;
  }
}

}  // namespace
}  // namespace ortb200

using namespace ortb200;

extern "C" int ortb200_nbits_prepack(const void* B, void* out, int64_t bytes, ortb200_stream_t stream_) {
  if (!B || !out || bytes < 0 || bytes % 4 != 0 || B == out) return -1;
  if ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 3) return -3;
  if (bytes == 0) return 0;
  const int64_t words = bytes / 4;
  int64_t blocks = (words + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  nbits_prepack_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint32_t*>(B), static_cast<uint32_t*>(out), words);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int ortb200_nbits_dequant(const void* B, const void* scales, const void* zero_points, int zp_is_packed, void* out,
                                     int64_t N, int K, int bits, int block_size, int64_t ldo, int dtype,
                                     ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!B || !scales || !out || N < 0 || K <= 0) return -1;
  if (bits != 4 && bits != 8) return -2;
  if (block_size < 16 || (block_size & (block_size - 1)) != 0) return -2;
  if (ldo < K || (ldo % 8) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(B) & 7)) return -3;
  if (N == 0) return 0;
  const int n_blocks = (K + block_size - 1) / block_size;
  const int64_t total = N * ((K + 7) / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const uint8_t* zp_p = (zero_points && zp_is_packed) ? static_cast<const uint8_t*>(zero_points) : nullptr;
  const void* zp_f = (zero_points && !zp_is_packed) ? zero_points : nullptr;
  const uint8_t* b = static_cast<const uint8_t*>(B);
  const unsigned g = static_cast<unsigned>(blocks);
  if (dtype == ORTB200_BF16) {
    using T = __nv_bfloat16;
    if (bits == 4) nbits_dequant_kernel<T, 4><<<g, 256, 0, stream>>>(b, static_cast<const T*>(scales), zp_p, static_cast<const T*>(zp_f), static_cast<T*>(out), N, K, block_size, n_blocks, ldo);
    else nbits_dequant_kernel<T, 8><<<g, 256, 0, stream>>>(b, static_cast<const T*>(scales), zp_p, static_cast<const T*>(zp_f), static_cast<T*>(out), N, K, block_size, n_blocks, ldo);
  } else if (dtype == ORTB200_F16) {
    using T = __half;
    if (bits == 4) nbits_dequant_kernel<T, 4><<<g, 256, 0, stream>>>(b, static_cast<const T*>(scales), zp_p, static_cast<const T*>(zp_f), static_cast<T*>(out), N, K, block_size, n_blocks, ldo);
    else nbits_dequant_kernel<T, 8><<<g, 256, 0, stream>>>(b, static_cast<const T*>(scales), zp_p, static_cast<const T*>(zp_f), static_cast<T*>(out), N, K, block_size, n_blocks, ldo);
  } else {
    return -4;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
