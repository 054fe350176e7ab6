// All-reduce / all-gather / all-to-all as single kernels over peer-mapped (symmetric) memory.
//
// Every rank runs the same kernel with the same grid.  Data moves with plain 16-byte peer stores over
// NVLink / NVSwitch; CTA b of one rank only ever depends on CTA b of the other ranks (the vectors are dealt to CTAs
// the same way on every rank), so one flag per (source rank, CTA) is the whole synchronisation - no grid-wide
// barrier and no host round trip, and the launch can sit in a CUDA graph.  Every wait is bounded and reports
// through the status word.
//
// Reference counterparts: the NCCL wrappers of onnxruntime/contrib_ops/cuda/collective/nccl_kernels.cc
// (AllReduce :379, AllGather :430, AllToAll :497) and the IPC-based custom all-reduce
// (collective/custom_reduce_impl.cu).
//
// Workspace layout (bytes from the base of each rank's buffer; see also ortb200_gemm_args):
//   64, 68                 epoch / done words of this file's kernels
//   [64 KiB, 256 KiB)      flags[src rank < 8][CTA < 4096] uint32
//   [bytes / 2, bytes)     two halves used alternately by epoch parity; each half = [scatter area | result area]
#include <cuda_runtime.h>
#include "ortb200_kernels.h"
#include "ptx_sm100.cuh"

namespace ortb200 {
namespace {

constexpr long long kFlagsOffset = 65536;
constexpr int kFlagsPerRank = 4096;
constexpr unsigned int kSpinLimit = 1u << 22;

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct CollParams {
  int op;                 // ORTB200_COLL_*
  int world, rank;
  void* peers[8];
  long long half_bytes;   // size of one parity half
  long long region_offset;  // bytes / 2
  const uint4* in;
  uint4* out;
  long long rows;         // all-gather: rows of the local piece;   others: 1
  long long row_vecs;     // 16-byte vectors per row of the local piece (all-to-all: per destination chunk;
                          // all-reduce: per slice, slices padded to whole vectors)
  long long total_vecs;   // all-reduce: vectors in the whole tensor
  int dtype;
  int* status;
};

// CTA-wide: tell every rank that this CTA's stores for `value` are done, then wait for the same CTA of every rank.
__device__ __forceinline__ bool cta_exchange_flags(const CollParams& p, unsigned int value) {
  __shared__ int s_ok;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_ok = 1;
  if (threadIdx.x < p.world) {
    unsigned int* f = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(p.peers[threadIdx.x]) + kFlagsOffset) +
                      p.rank * kFlagsPerRank + blockIdx.x;
    st_release_sys(f, value);
  }
  __syncthreads();
  if (threadIdx.x < p.world) {
    const unsigned int* f = reinterpret_cast<const unsigned int*>(static_cast<const uint8_t*>(p.peers[p.rank]) + kFlagsOffset) +
                            threadIdx.x * kFlagsPerRank + blockIdx.x;
    unsigned int spins = 0;
    while (static_cast<int>(ld_acquire_sys(f) - value) < 0) {
      if (++spins > kSpinLimit) {
        s_ok = 0;
        if (p.status) atomicExch(p.status, kStatusTimeoutPeer);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  __threadfence_system();
  return s_ok != 0;
}

template <typename T>
__device__ __forceinline__ void add_vec(float* acc, const uint4& v) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < 16 / static_cast<int>(sizeof(T)); ++i) acc[i] += to_float<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 sum_vecs(const uint4* const* src, int world, long long idx) {
  float acc[16 / sizeof(T)];
#pragma unroll
  for (int i = 0; i < 16 / static_cast<int>(sizeof(T)); ++i) acc[i] = 0.f;
  for (int s = 0; s < world; ++s) add_vec<T>(acc, __ldcg(src[s] + idx));  // rank order: same bits on every rank
  uint4 r;
  T* e = reinterpret_cast<T*>(&r);
#pragma unroll
  for (int i = 0; i < 16 / static_cast<int>(sizeof(T)); ++i) e[i] = from_float<T>(acc[i]);
  return r;
}

__global__ void __launch_bounds__(256) symm_collective_kernel(const CollParams p) {
  pdl_wait_prior_grids();
  unsigned int* hdr = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(p.peers[p.rank]) + 64);
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(hdr) + 1;
  const long long half_off = p.region_offset + static_cast<long long>(epoch & 1) * p.half_bytes;
  const long long scatter_vecs = p.half_bytes / 32;  // vectors in the scatter area (= half of the half)
  auto scatter_of = [&](int r) { return reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.peers[r]) + half_off); };
  auto result_of = [&](int r) { return scatter_of(r) + scatter_vecs; };
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  bool ok = true;

  if (p.op == ORTB200_COLL_ALLGATHER) {
    // result[row][src rank][row_vecs]
    const long long n = p.rows * p.row_vecs;
    for (long long i = t0; i < n; i += stride) {
      const uint4 v = p.in[i];
      const long long row = i / p.row_vecs, c = i % p.row_vecs;
      const long long dst = (row * p.world + p.rank) * p.row_vecs + c;
      for (int d = 0; d < p.world; ++d) result_of((p.rank + d) % p.world)[dst] = v;
    }
    ok = cta_exchange_flags(p, 2 * epoch + 1);
    const long long total = n * p.world;
    const uint4* res = result_of(p.rank);
    // a CTA reads back exactly the vectors that its namesakes wrote: same (row, c) set for every source rank
    for (long long i = t0; i < n; i += stride) {
      const long long row = i / p.row_vecs, c = i % p.row_vecs;
      for (int s = 0; s < p.world; ++s) {
        const long long idx = (row * p.world + s) * p.row_vecs + c;
        p.out[idx] = __ldcg(res + idx);
      }
    }
    (void)total;
  } else if (p.op == ORTB200_COLL_ALLTOALL) {
    // in = [world][row_vecs]; chunk d goes to rank d, which stores it at result[src rank]
    for (long long i = t0; i < p.row_vecs; i += stride)
      for (int d = 0; d < p.world; ++d) {
        const int dst = (p.rank + d) % p.world;
        result_of(dst)[static_cast<long long>(p.rank) * p.row_vecs + i] = p.in[static_cast<long long>(dst) * p.row_vecs + i];
      }
    ok = cta_exchange_flags(p, 2 * epoch + 1);
    const uint4* res = result_of(p.rank);
    for (long long i = t0; i < p.row_vecs; i += stride)
      for (int s = 0; s < p.world; ++s) p.out[static_cast<long long>(s) * p.row_vecs + i] = __ldcg(res + static_cast<long long>(s) * p.row_vecs + i);
  } else {
    // all-reduce in two steps: slice d of every rank's input is pushed to rank d (scatter[src rank][row_vecs]),
    // rank d adds the slices in rank order and pushes the sums to everyone's result area, everyone copies out
    for (long long i = t0; i < p.row_vecs; i += stride)
      for (int d = 0; d < p.world; ++d) {
        const int dst = (p.rank + d) % p.world;
        const long long g = static_cast<long long>(dst) * p.row_vecs + i;
        if (g < p.total_vecs) scatter_of(dst)[static_cast<long long>(p.rank) * p.row_vecs + i] = p.in[g];
      }
    ok = cta_exchange_flags(p, 2 * epoch + 1);
    const uint4* src[8];
    for (int s = 0; s < p.world; ++s) src[s] = scatter_of(p.rank) + static_cast<long long>(s) * p.row_vecs;
    for (long long i = t0; i < p.row_vecs; i += stride) {
      const long long g = static_cast<long long>(p.rank) * p.row_vecs + i;
      if (g >= p.total_vecs) continue;
      uint4 r;
      if (p.dtype == ORTB200_BF16) r = sum_vecs<__nv_bfloat16>(src, p.world, i);
      else if (p.dtype == ORTB200_F16) r = sum_vecs<__half>(src, p.world, i);
      else r = sum_vecs<float>(src, p.world, i);
      for (int d = 0; d < p.world; ++d) result_of((p.rank + d) % p.world)[g] = r;
    }
    ok = cta_exchange_flags(p, 2 * epoch + 2) && ok;
    const uint4* res = result_of(p.rank);
    for (long long i = t0; i < p.row_vecs; i += stride)
      for (int s = 0; s < p.world; ++s) {
        const long long g = static_cast<long long>(s) * p.row_vecs + i;
        if (g < p.total_vecs) p.out[g] = __ldcg(res + g);
      }
  }
  (void)ok;
  pdl_launch_dependents();
  // the CTA that finishes last closes the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(hdr + 1, 1u) == gridDim.x - 1) {
      hdr[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(hdr) = epoch;
    }
  }
}

}  // namespace
}  // namespace ortb200

using namespace ortb200;

extern "C" int64_t ortb200_symm_collective_max_bytes(int op, int world, int64_t symm_bytes) {
  // one parity half = symm_bytes / 4; its scatter and result areas are half of that each
  const int64_t area = symm_bytes / 8;
  if (op == ORTB200_COLL_ALLGATHER) return area / (world > 0 ? world : 1);  // per-rank input bytes
  if (op == ORTB200_COLL_ALLTOALL) return area;                            // whole input
  return area / 2;                                                         // all-reduce: whole tensor (slices are padded)
}

extern "C" int ortb200_symm_collective(const ortb200_symm_collective_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->in || !a->out || a->world < 2 || a->world > 8 || a->rank < 0 || a->rank >= a->world) return -1;
  for (int i = 0; i < a->world; ++i)
    if (!a->peers[i]) return -1;
  if ((reinterpret_cast<uintptr_t>(a->in) | reinterpret_cast<uintptr_t>(a->out)) & 15) return -3;
  if (a->symm_bytes < (1 << 20) || (a->symm_bytes % 256) != 0) return -3;
  CollParams p;
  p.op = a->op; p.world = a->world; p.rank = a->rank;
  for (int i = 0; i < 8; ++i) p.peers[i] = i < a->world ? a->peers[i] : nullptr;
  p.region_offset = a->symm_bytes / 2;
  p.half_bytes = a->symm_bytes / 4;
  p.in = static_cast<const uint4*>(a->in);
  p.out = static_cast<uint4*>(a->out);
  p.dtype = a->dtype;
  p.status = a->status;
  p.rows = 1; p.row_vecs = 0; p.total_vecs = 0;
  const int64_t limit = ortb200_symm_collective_max_bytes(a->op, a->world, a->symm_bytes);
  long long work_vecs = 0;
  if (a->op == ORTB200_COLL_ALLGATHER) {
    if (a->rows <= 0 || a->row_bytes <= 0 || a->row_bytes % 16 != 0 || a->rows * a->row_bytes > limit) return -13;
    p.rows = a->rows; p.row_vecs = a->row_bytes / 16;
    work_vecs = p.rows * p.row_vecs;
  } else if (a->op == ORTB200_COLL_ALLTOALL) {
    if (a->row_bytes <= 0 || a->row_bytes % 16 != 0 || a->row_bytes * a->world > limit) return -13;
    p.row_vecs = a->row_bytes / 16;  // bytes per destination chunk
    work_vecs = p.row_vecs;
  } else if (a->op == ORTB200_COLL_ALLREDUCE) {
    if (a->row_bytes <= 0 || a->row_bytes % 16 != 0 || a->row_bytes > limit) return -13;
    if (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16 && a->dtype != ORTB200_F32) return -4;
    p.total_vecs = a->row_bytes / 16;  // bytes of the whole tensor
    p.row_vecs = (p.total_vecs + a->world - 1) / a->world;
    work_vecs = p.row_vecs;
  } else {
    return -2;
  }
  long long ctas = (work_vecs + 255) / 256;
  if (ctas > 2 * 148) ctas = 2 * 148;  // all CTAs resident at once: a CTA waits for its namesakes on the other ranks
  if (ctas < 1) ctas = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  if (a->use_pdl) {
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, symm_collective_kernel, p) == cudaSuccess ? 0 : -11;
}
