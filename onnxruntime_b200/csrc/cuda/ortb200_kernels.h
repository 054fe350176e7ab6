// C ABI of the sm_100a kernel library (libortb200_kernels.so).
//
// Every function takes raw device pointers plus a cudaStream_t and returns 0
// on success or a negative code when the arguments are rejected on the host
// (nothing is launched in that case).  Device-side problems (a bounded wait
// that ran out) are reported through the int status word the caller passes;
// 0 means the launch completed normally.
//
// The library does not depend on PyTorch; the torch extension and ctypes-based
// tests both call it through these symbols.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* ortb200_stream_t;  // cudaStream_t

enum ortb200_dtype { ORTB200_F16 = 0, ORTB200_BF16 = 1, ORTB200_F32 = 2 };

enum ortb200_act {
  ORTB200_ACT_NONE = 0,
  ORTB200_ACT_GELU = 1,      // erf form
  ORTB200_ACT_FASTGELU = 2,  // tanh form
  ORTB200_ACT_RELU = 3,
  ORTB200_ACT_SILU = 4,
  ORTB200_ACT_SWIGLU = 5,    // silu(W1 x) * (W2 x); W2 rows start `dual_offset` rows after W1 rows
  ORTB200_ACT_QUICKGELU = 6,
};

// out[M, N] = act(alpha * X[M, K] * W[N, K]^T + bias[N]) + residual[M, N]
// X and W are row-major with K contiguous (K % 8 == 0, 16-byte aligned bases).
// tcgen05 / TMEM tensor-core GEMM; weights ride the 128-lane M side of the MMA
// and tokens the N side, so decode (M = 1..16) streams W once at HBM speed and
// prefill uses 128x{128,256} tiles.  `workspace` holds split-K partial tiles and
// tile counters; ortb200_gemm_workspace_bytes() gives an upper bound for a
// problem.  The counters must be zero before the first launch (the kernel leaves
// them zero again).
typedef struct {
  const void* x;        // [M, K]
  const void* w;        // [N_total, K]; N rows used for the first operand
  void* out;            // [M, ldo]
  const void* bias;     // [N] or null, same dtype as out
  const void* residual; // [M, ldr] or null, same dtype as out
  int64_t ldo, ldr;
  int M, N, K;
  int w_rows;           // total rows in w (>= N, or >= dual_offset + N for SWIGLU)
  int dual_offset;      // SWIGLU only
  int dtype;            // ortb200_dtype of x, w, out, bias, residual (F16 or BF16)
  int act;              // ortb200_act
  float alpha;
  void* workspace;      // device scratch, may be null when splits == 1 is forced
  int64_t workspace_bytes;
  int* status;          // device int, may be null
  int force_splits;     // 0 = heuristic
  int force_bn;         // 0 = heuristic; else 16/32/64/128/256
  int use_pdl;          // launch with programmatic stream serialization
} ortb200_gemm_args;

int ortb200_gemm(const ortb200_gemm_args* args, ortb200_stream_t stream);
int64_t ortb200_gemm_workspace_bytes(int M, int N, int K, int act);
// Number of kernels one ortb200_gemm call launches (always 1).
int ortb200_gemm_last_config(int* bn, int* splits, int* stages);

#ifdef __cplusplus
}
#endif
