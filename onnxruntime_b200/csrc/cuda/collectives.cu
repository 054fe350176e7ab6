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
//   64, 68, 72             epoch / done words of this file's kernels; polling-limit override (0 = default)
//   [64 KiB, 256 KiB)      flags[src rank < 8][CTA < 4096] uint32
//   [bytes / 2, bytes)     two halves used alternately by epoch parity; each half = [scatter area | result area]
#include <cuda_runtime.h>
#include "gemm_internal.h"
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
  // all-reduce that finishes a tensor-parallel GEMM: the scatter areas were filled by the GEMM's epilogue
  // (prescattered), and residual [M, N] (row pitch ldr elements, N = row_elems) is added to the sums
  int prescattered;
  const void* residual;
  long long ldr;
  int row_elems;
  // NVLS: multicast address of the workspace (every rank's buffer behind one address).  With it the sums are
  // replicated by one multimem.st per 16 bytes (the switch copies them to every rank: 1 / world of the tensor leaves
  // the GPU instead of (world - 1) / world).  A stand-alone all-reduce also lets the switch add: the inputs stay at
  // home and one multimem.ld_reduce per 16 bytes of the rank's slice returns the sum.  The all-reduce that finishes a
  // GEMM keeps its peer-store scatter, because those stores overlap the GEMM's remaining tiles while a reduction in
  // the switch can only start after the GEMM (measured on 4 GPUs: 42.1 ms time to first token with ld_reduce
  // against 39.6 ms with the overlapped scatter).  16-bit and 32-bit float types.
  void* mc;
};

// 16 bytes summed over all ranks by the switch (fp32 accumulation for the 16-bit types)
__device__ __forceinline__ uint4 multimem_ld_reduce(const void* mc_addr, int dtype) {
  uint4 v;
  if (dtype == ORTB200_BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  else if (dtype == ORTB200_F16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
// 16 bytes stored into every rank's copy
__device__ __forceinline__ void multimem_st(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

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
    // word 2 of this file's header (byte 72 of the local workspace) overrides the polling limit (0 = default);
    // failure-detection tests set a small one so that a rank that never answers costs milliseconds
    const unsigned int lim_override = *reinterpret_cast<const volatile unsigned int*>(static_cast<const uint8_t*>(p.peers[p.rank]) + 72);
    const unsigned int limit = lim_override != 0 ? lim_override : kSpinLimit;
    unsigned int spins = 0;
    while (static_cast<int>(ld_acquire_sys(f) - value) < 0) {
      if (++spins > limit) {
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
__device__ __forceinline__ uint4 sum_vecs(const uint4* const* src, int world, long long idx, const uint4* residual = nullptr) {
  float acc[16 / sizeof(T)];
#pragma unroll
  for (int i = 0; i < 16 / static_cast<int>(sizeof(T)); ++i) acc[i] = 0.f;
  for (int s = 0; s < world; ++s) add_vec<T>(acc, __ldcg(src[s] + idx));  // rank order: same bits on every rank
  if (residual) add_vec<T>(acc, __ldg(residual));
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
  } else if (p.mc != nullptr && !p.prescattered) {
    // stand-alone all-reduce through the switch: every rank leaves its whole input in its OWN scatter area, then
    // reduces its slice with multimem.ld_reduce and replicates the sums with multimem.st into every rank's result area
    uint4* mine = scatter_of(p.rank);
    for (long long i = t0; i < p.row_vecs; i += stride)
      for (int d = 0; d < p.world; ++d) {
        const long long g = static_cast<long long>(d) * p.row_vecs + i;
        if (g < p.total_vecs) mine[g] = p.in[g];
      }
    ok = cta_exchange_flags(p, 2 * epoch + 1);
    uint8_t* mc_scatter = static_cast<uint8_t*>(p.mc) + half_off;
    uint8_t* mc_result = mc_scatter + scatter_vecs * 16;
    // four reductions in flight per thread: one switch round trip costs microseconds, so the loop is unrolled with
    // all loads (and residual loads) issued before the first result is touched
    constexpr int kUnroll = 4;
    for (long long i0 = t0; i0 < p.row_vecs; i0 += kUnroll * stride) {
      uint4 r[kUnroll], rv[kUnroll];
      long long gs[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = i0 + u * stride;
        const long long g = static_cast<long long>(p.rank) * p.row_vecs + i;
        gs[u] = (i < p.row_vecs && g < p.total_vecs) ? g : -1;
        if (gs[u] >= 0) {
          r[u] = multimem_ld_reduce(mc_scatter + g * 16, p.dtype);
          if (p.residual) {
            const long long el = g * 8;  // 16-bit types only
            const long long m = el / p.row_elems, n = el - m * p.row_elems;
            rv[u] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) + m * p.ldr + n));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (gs[u] < 0) continue;
        if (p.residual) {
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
          if (p.dtype == ORTB200_BF16) {
            add_vec<__nv_bfloat16>(acc, r[u]);
            add_vec<__nv_bfloat16>(acc, rv[u]);
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&r[u]);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(acc[e]);
          } else {
            add_vec<__half>(acc, r[u]);
            add_vec<__half>(acc, rv[u]);
            __half* o = reinterpret_cast<__half*>(&r[u]);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __float2half_rn(acc[e]);
          }
        }
        multimem_st(mc_result + gs[u] * 16, r[u]);
      }
    }
    ok = cta_exchange_flags(p, 2 * epoch + 2) && ok;
    const uint4* res = result_of(p.rank);
    for (long long i = t0; i < p.row_vecs; i += stride)
      for (int s = 0; s < p.world; ++s) {
        const long long g = static_cast<long long>(s) * p.row_vecs + i;
        if (g < p.total_vecs) p.out[g] = __ldcg(res + g);
      }
  } else {
    // all-reduce in two steps: slice d of every rank's input is pushed to rank d (scatter[src rank][row_vecs]),
    // rank d adds the slices in rank order and pushes the sums to everyone's result area, everyone copies out
    if (!p.prescattered) {
      for (long long i = t0; i < p.row_vecs; i += stride)
        for (int d = 0; d < p.world; ++d) {
          const int dst = (p.rank + d) % p.world;
          const long long g = static_cast<long long>(dst) * p.row_vecs + i;
          if (g < p.total_vecs) scatter_of(dst)[static_cast<long long>(p.rank) * p.row_vecs + i] = p.in[g];
        }
    }
    ok = cta_exchange_flags(p, 2 * epoch + 1);
    const uint4* src[8];
    for (int s = 0; s < p.world; ++s) src[s] = scatter_of(p.rank) + static_cast<long long>(s) * p.row_vecs;
    for (long long i = t0; i < p.row_vecs; i += stride) {
      const long long g = static_cast<long long>(p.rank) * p.row_vecs + i;
      if (g >= p.total_vecs) continue;
      uint4 r;
      const uint4* res_vec = nullptr;
      if (p.residual) {
        const long long el = g * 8;  // 16-bit types only
        const long long m = el / p.row_elems, n = el - m * p.row_elems;
        res_vec = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) + m * p.ldr + n);
      }
      if (p.dtype == ORTB200_BF16) r = sum_vecs<__nv_bfloat16>(src, p.world, i, res_vec);
      else if (p.dtype == ORTB200_F16) r = sum_vecs<__half>(src, p.world, i, res_vec);
      else r = sum_vecs<float>(src, p.world, i);
      if (p.mc != nullptr) {
        // one store, replicated by the switch into every rank's result area
        multimem_st(static_cast<uint8_t*>(p.mc) + half_off + (scatter_vecs + g) * 16, r);
      } else {
        for (int d = 0; d < p.world; ++d) result_of((p.rank + d) % p.world)[g] = r;
      }
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

// ---------------------------------------------------------------------------------------------------------------
// Expert-parallel mixture of experts: un-permute + routing-weight scale + cross-rank sum + replication in one kernel.
//
// Every rank has run its local experts on the (replicated) tokens routed to them; y holds those expert outputs in
// permuted order.  Token t is owned by rank t / T_own.  Step 1: each rank adds up ITS experts' weighted rows of token t
// and stores that one row straight into the owner's scatter area (slot = position of the rank's first expert in the
// token's top-k list, so no two ranks share a slot and nobody needs a count).  Step 2: the owner adds the slots of the
// token in top-k order and stores the finished row into every rank's result area.  Step 3: copy out.  CTA b handles
// the tokens t = b (mod grid) on every rank, so the two flag exchanges between namesake CTAs are the only
// synchronisation.  Per GPU this moves (routed rows / world) * 7/8 rows out in step 1 and its token shard to 7 peers in
// step 2, against a broadcast of every permuted row in the reference
// (onnxruntime/contrib_ops/cuda/collective/sharded_moe.cc:159-176).
struct MoeCombineParams {
  CollParams c;             // world, rank, peers, half_bytes, region_offset, status (op / in / out unused)
  const void* y;            // [rows, H] expert outputs of this rank, permuted order
  const void* bias;         // optional [E_local, H]
  void* out;                // [T, H]
  const int* topk_idx;      // [T, k] global expert ids
  const float* topk_w;      // [T, k]
  const int* row_of;        // [T, k] row of y, or -1 when the expert lives on another rank
  int T, H, k, E_local, expert_begin, T_own;
};

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_symm_kernel(const MoeCombineParams p) {
  pdl_wait_prior_grids();
  const CollParams& c = p.c;
  unsigned int* hdr = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(c.peers[c.rank]) + 64);
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(hdr) + 1;
  const long long half_off = c.region_offset + static_cast<long long>(epoch & 1) * c.half_bytes;
  const long long scatter_vecs = c.half_bytes / 32;
  auto scatter_of = [&](int r) { return reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.peers[r]) + half_off); };
  auto result_of = [&](int r) { return scatter_of(r) + scatter_vecs; };
  constexpr int EPV = 16 / static_cast<int>(sizeof(T));  // elements per 16-byte vector
  const int hvecs = p.H / EPV;
  const T* y = static_cast<const T*>(p.y);
  const T* bias = static_cast<const T*>(p.bias);

  // ---- step 1: this rank's share of every token of this CTA, pushed to the token's owner
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    int slot = -1;
    for (int j = 0; j < p.k; ++j)
      if (p.row_of[t * p.k + j] >= 0) {
        slot = j;
        break;
      }
    if (slot < 0) continue;  // none of this token's experts live here
    const int owner = t / p.T_own, tl = t - owner * p.T_own;
    uint4* dst = scatter_of(owner) + (static_cast<long long>(tl) * p.k + slot) * hvecs;
    for (int hv = threadIdx.x; hv < hvecs; hv += blockDim.x) {
      float acc[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
      for (int j = slot; j < p.k; ++j) {
        const int row = p.row_of[t * p.k + j];
        if (row < 0) continue;
        const float w = p.topk_w[t * p.k + j];
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * p.H) + hv);
        const T* ve = reinterpret_cast<const T*>(&v);
        if (bias) {
          const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + static_cast<long long>(p.topk_idx[t * p.k + j] - p.expert_begin) * p.H) + hv);
          const T* be = reinterpret_cast<const T*>(&bv);
#pragma unroll
          for (int e = 0; e < EPV; ++e) acc[e] += w * (to_float<T>(ve[e]) + to_float<T>(be[e]));
        } else {
#pragma unroll
          for (int e = 0; e < EPV; ++e) acc[e] += w * to_float<T>(ve[e]);
        }
      }
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int e = 0; e < EPV; ++e) oe[e] = from_float<T>(acc[e]);
      dst[hv] = o;
    }
  }
  bool ok = cta_exchange_flags(c, 2 * epoch + 1);

  // ---- step 2: the owner adds the slots of its tokens in top-k order and replicates the row
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    if (t / p.T_own != c.rank) continue;
    const int tl = t - c.rank * p.T_own;
    const uint4* src = scatter_of(c.rank) + static_cast<long long>(tl) * p.k * hvecs;
    // slot j carries data when expert j's rank does not already appear earlier in the list
    unsigned int use = 0;
    for (int j = 0; j < p.k; ++j) {
      const int rj = p.topk_idx[t * p.k + j] / p.E_local;
      bool first = true;
      for (int i = 0; i < j; ++i) first = first && (p.topk_idx[t * p.k + i] / p.E_local != rj);
      if (first) use |= 1u << j;
    }
    for (int hv = threadIdx.x; hv < hvecs; hv += blockDim.x) {
      float acc[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
      for (int j = 0; j < p.k; ++j) {
        if (!((use >> j) & 1u)) continue;
        const uint4 v = __ldcg(src + static_cast<long long>(j) * hvecs + hv);
        const T* ve = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int e = 0; e < EPV; ++e) acc[e] += to_float<T>(ve[e]);
      }
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int e = 0; e < EPV; ++e) oe[e] = from_float<T>(acc[e]);
      const long long idx = static_cast<long long>(t) * hvecs + hv;
      for (int d = 0; d < c.world; ++d) result_of((c.rank + d) % c.world)[idx] = o;
    }
  }
  ok = cta_exchange_flags(c, 2 * epoch + 2) && ok;

  // ---- step 3: copy this CTA's tokens out of the local result area
  const uint4* res = result_of(c.rank);
  uint4* out = static_cast<uint4*>(p.out);
  for (int t = blockIdx.x; t < p.T; t += gridDim.x)
    for (int hv = threadIdx.x; hv < hvecs; hv += blockDim.x) out[static_cast<long long>(t) * hvecs + hv] = __ldcg(res + static_cast<long long>(t) * hvecs + hv);
  (void)ok;
  pdl_launch_dependents();
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

namespace ortb200 {
int launch_allreduce_prescattered(const ortb200_gemm_args* a, cudaStream_t stream) {
  if (a->world < 2 || a->world > 8 || !a->out || a->ldo != a->N || a->N % 8 != 0) return -12;
  if (a->residual && ((a->ldr % 8) != 0 || (reinterpret_cast<uintptr_t>(a->residual) & 15))) return -3;
  if (reinterpret_cast<uintptr_t>(a->out) & 15) return -3;
  CollParams p;
  p.op = ORTB200_COLL_ALLREDUCE; p.world = a->world; p.rank = a->rank;
  for (int i = 0; i < 8; ++i) p.peers[i] = i < a->world ? a->peers[i] : nullptr;
  p.region_offset = a->symm_bytes / 2;
  p.half_bytes = a->symm_bytes / 4;
  p.in = nullptr;
  p.out = static_cast<uint4*>(a->out);
  p.dtype = a->dtype;
  p.status = a->status;
  p.rows = 1;
  p.total_vecs = static_cast<long long>(a->M) * a->N / 8;
  p.row_vecs = (p.total_vecs + a->world - 1) / a->world;
  p.prescattered = 1; p.residual = a->residual; p.ldr = a->ldr; p.row_elems = a->N;
  p.mc = a->mc_ptr;
  long long ctas = (p.row_vecs + 255) / 256;
  if (ctas > 2 * 148) ctas = 2 * 148;
  if (ctas < 1) ctas = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  return cudaLaunchKernelEx(&cfg, symm_collective_kernel, p) == cudaSuccess ? 0 : -11;
}
}  // namespace ortb200

extern "C" int ortb200_moe_combine_symm(const ortb200_moe_combine_symm_args* a, ortb200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->y || !a->out || !a->topk_idx || !a->topk_w || !a->row_of) return -1;
  if (a->world < 2 || a->world > 8 || a->rank < 0 || a->rank >= a->world || a->T <= 0 || a->H <= 0 || a->k <= 0 || a->k > 8 || a->E_local <= 0) return -1;
  if (a->dtype != ORTB200_BF16 && a->dtype != ORTB200_F16) return -4;
  if (a->H % 8 != 0) return -3;
  if ((reinterpret_cast<uintptr_t>(a->y) | reinterpret_cast<uintptr_t>(a->out) | reinterpret_cast<uintptr_t>(a->bias)) & 15) return -3;
  if (a->symm_bytes < (1 << 20) || (a->symm_bytes % 256) != 0) return -3;
  for (int i = 0; i < a->world; ++i)
    if (!a->peers[i]) return -1;
  MoeCombineParams p{};
  p.c.world = a->world; p.c.rank = a->rank;
  for (int i = 0; i < 8; ++i) p.c.peers[i] = i < a->world ? a->peers[i] : nullptr;
  p.c.region_offset = a->symm_bytes / 2;
  p.c.half_bytes = a->symm_bytes / 4;
  p.c.status = a->status;
  p.y = a->y; p.bias = a->bias; p.out = a->out; p.topk_idx = a->topk_idx; p.topk_w = a->topk_w; p.row_of = a->row_of;
  p.T = a->T; p.H = a->H; p.k = a->k; p.E_local = a->E_local; p.expert_begin = a->expert_begin;
  p.T_own = (a->T + a->world - 1) / a->world;
  const long long area = p.c.half_bytes / 2;  // scatter area == result area
  if (static_cast<long long>(p.T_own) * a->k * a->H * 2 > area || static_cast<long long>(a->T) * a->H * 2 > area) return -13;
  int ctas = a->T < 2 * 148 ? a->T : 2 * 148;  // all CTAs resident at once: a CTA waits for its namesakes on the other ranks
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
  cudaError_t e;
  if (a->dtype == ORTB200_BF16) e = cudaLaunchKernelEx(&cfg, moe_combine_symm_kernel<__nv_bfloat16>, p);
  else e = cudaLaunchKernelEx(&cfg, moe_combine_symm_kernel<__half>, p);
  return e == cudaSuccess ? 0 : -11;
}

extern "C" int64_t ortb200_moe_combine_symm_max_tokens(int world, int k, int H, int64_t symm_bytes) {
  const int64_t area = symm_bytes / 8;
  const int64_t by_result = area / (static_cast<int64_t>(H) * 2);
  const int64_t by_scatter = area / (static_cast<int64_t>(H) * 2 * k) * world - world;  // T_own is rounded up
  return by_result < by_scatter ? by_result : by_scatter;
}

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
  p.prescattered = 0; p.residual = nullptr; p.ldr = 0; p.row_elems = 0;
  p.mc = a->op == ORTB200_COLL_ALLREDUCE ? a->mc_ptr : nullptr;
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
