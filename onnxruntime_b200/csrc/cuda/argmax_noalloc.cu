// Arg-max that carries its own scratch memory; see argmax_noalloc.h for the contract.
#include <cuda_runtime.h>

#include <mutex>

#include "argmax_noalloc.h"
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace {

using ortb200::to_float;

// Per row: one 64-bit running maximum and one 32-bit arrival counter (padded to 8 bytes).
constexpr int kMaxRows = ORTB200_ARGMAX_NOALLOC_MAX_ROWS;
constexpr size_t kScratchBytes = static_cast<size_t>(kMaxRows) * 16;  // 64 KiB
static __device__ __align__(256) unsigned char g_argmax_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

// value in the high half (made orderable as an unsigned integer), inverted index in the low half:
// the larger value wins and, between equal values, the smaller index
__device__ __forceinline__ unsigned long long make_key(float v, long long idx) {
  unsigned int u = __float_as_uint(v + 0.0f);  // -0.0 + 0.0 = +0.0: the two zeros compare equal, the first index wins
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return (static_cast<unsigned long long>(u) << 32) | static_cast<unsigned long long>(0xFFFFFFFFu - static_cast<unsigned int>(idx));
}

// grid (chunks, rows).  The scratch is zero when the kernel starts (the host enqueues the clear in front of it).
template <typename T>
__global__ void __launch_bounds__(256) argmax_noalloc_kernel(const T* __restrict__ x, int64_t* __restrict__ out, int64_t n,
                                                             unsigned long long* __restrict__ best_of_row,
                                                             unsigned int* __restrict__ arrived) {
  __shared__ unsigned long long warp_best[8];
  const int64_t r = blockIdx.y;
  const T* row = x + r * n;
  const int64_t per = (n + gridDim.x - 1) / gridDim.x;
  const int64_t lo = blockIdx.x * per;
  const int64_t hi = lo + per < n ? lo + per : n;
  unsigned long long best = 0;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = to_float<T>(row[i]);
    if (v == v) {
      const unsigned long long k = make_key(v, i);
      best = k > best ? k : best;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) best = warp_best[w] > best ? warp_best[w] : best;
    atomicMax(&best_of_row[r], best);
    __threadfence();
    if (atomicAdd(&arrived[r], 1u) == gridDim.x - 1) {  // last chunk of this row: every maximum has been merged
      __threadfence();
      const unsigned long long k = atomicMax(&best_of_row[r], 0ull);
      out[r] = k == 0 ? 0 : static_cast<int64_t>(0xFFFFFFFFu - static_cast<unsigned int>(k & 0xFFFFFFFFull));
    }
  }
}

int scratch_for_current_device(void** addr) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ORTB200_NOALLOC_E_NO_SCRATCH;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_argmax_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return ORTB200_NOALLOC_E_NO_SCRATCH;
    }
    g_scratch_addr[dev] = p;
  }
  *addr = g_scratch_addr[dev];
  return ORTB200_NOALLOC_OK;
}

}  // namespace

extern "C" int ortb200_argmax_noalloc_prepare(void) {
  void* p = nullptr;
  return scratch_for_current_device(&p);
}

extern "C" int ortb200_argmax_noalloc(const void* x, int64_t* out, int64_t rows, int64_t n, int dtype, void* stream) {
  if (!x || !out || rows < 0 || n <= 0 || n > 0xFFFFFFFFll) return ORTB200_NOALLOC_E_BAD_ARGUMENT;
  if (rows > kMaxRows) return ORTB200_NOALLOC_E_TOO_LARGE;
  if (dtype != ORTB200_BF16 && dtype != ORTB200_F16 && dtype != ORTB200_F32) return ORTB200_NOALLOC_E_BAD_DTYPE;
  if (rows == 0) return ORTB200_NOALLOC_OK;
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != ORTB200_NOALLOC_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned long long* best_of_row = static_cast<unsigned long long*>(scratch);
  unsigned int* arrived = reinterpret_cast<unsigned int*>(best_of_row + rows);
  // both the running maxima and the arrival counters have to start at zero
  if (cudaMemsetAsync(scratch, 0, static_cast<size_t>(rows) * 16, st) != cudaSuccess) {
    (void)cudaGetLastError();
    return ORTB200_NOALLOC_E_LAUNCH;
  }
  int chunks = static_cast<int>((n + 4095) / 4096);
  const int64_t want = (2 * 148 + rows - 1) / rows;  // about two CTAs per SM over all rows
  if (chunks > want) chunks = static_cast<int>(want);
  if (chunks < 1) chunks = 1;
  const dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(rows));
  if (dtype == ORTB200_BF16)
    argmax_noalloc_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), out, n, best_of_row, arrived);
  else if (dtype == ORTB200_F16)
    argmax_noalloc_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), out, n, best_of_row, arrived);
  else
    argmax_noalloc_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), out, n, best_of_row, arrived);
  return cudaGetLastError() == cudaSuccess ? ORTB200_NOALLOC_OK : ORTB200_NOALLOC_E_LAUNCH;
}

extern "C" const char* ortb200_argmax_noalloc_strerror(int code) {
  switch (code) {
    case ORTB200_NOALLOC_OK: return "ok";
    case ORTB200_NOALLOC_E_BAD_ARGUMENT: return "bad argument: x and out must be non-null, rows >= 0 and 1 <= n <= 4294967295";
    case ORTB200_NOALLOC_E_BAD_DTYPE: return "unsupported dtype: use ORTB200_F16, ORTB200_BF16 or ORTB200_F32";
    case ORTB200_NOALLOC_E_LAUNCH: return "the CUDA runtime rejected the scratch clear or the kernel launch";
    case ORTB200_NOALLOC_E_TOO_LARGE:
      return "rows exceeds ORTB200_ARGMAX_NOALLOC_MAX_ROWS (4096): the built-in scratch array holds 16 bytes per row; "
             "use ortb200_argmax() with caller-provided scratch";
    case ORTB200_NOALLOC_E_NO_SCRATCH: return "the address of the built-in scratch array could not be obtained on the current device";
    default: return "unknown code";
  }
}
