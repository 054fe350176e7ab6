// Helpers shared by the GPU op wrappers (kernels_cuda*.cc).
#pragma once
#include <ATen/ATen.h>

#include "kernel.h"

namespace ortb {

void CheckLaunch(int rc, const char* what);

// out[M,N] = act(alpha * x[M,K] @ w_nk[N,K]^T + bias) + residual on the tcgen05 GEMM kernel.
// act == SWIGLU: w_nk holds gate rows then up rows, `dual_offset` rows apart.
// fused_allreduce: the kernel also sums the result over all ranks through the session's symmetric workspace.
// x2d / w_nk of type Float8_e4m3fn run the tensor cores in 8-bit mode; out_type (fp16 / bf16) is then required.
at::Tensor LaunchGemm(OpKernelContext& ctx, const at::Tensor& x2d, const at::Tensor& w_nk, int64_t n_out,
                      int64_t dual_offset, const at::Tensor& bias, const at::Tensor& residual2d, int act, float alpha,
                      bool fused_allreduce = false, at::ScalarType out_type = at::ScalarType::Undefined, float rms_eps = 0.f,
                      const at::Tensor& alpha_dev = at::Tensor());
// MatMulNBits (4-bit) weights as the tile-blob array the decode GEMM expands in shared memory, and that GEMM (M <= 64).
at::Tensor NbitsBuildBlobs(const at::Tensor& B, const at::Tensor& scales, const at::Tensor& zp_bytes, int64_t N, int64_t K,
                           int64_t block);
at::Tensor LaunchGemmQ4(OpKernelContext& ctx, const at::Tensor& x2d, const at::Tensor& blobs, int64_t n_out, const at::Tensor& bias,
                        const at::Tensor& residual2d, bool fused_allreduce = false, int in_dtype = 4 /* ORTB200_Q4 */);
// Weight-only fp8 (e4m3 [N, K] + fp32 scales [N, K / block]) as the tile-blob array of the decode GEMM's fp8 mode
// (layout: ortb200_gemm_args, in_dtype F8W).  K and block must be multiples of 64.
at::Tensor Fp8WeightBuildBlobs(const at::Tensor& B, const at::Tensor& scales, int64_t block);
// True when the fused GEMM + all-reduce kernel can take an [M, N] row-parallel product in this session.
bool CanFuseAllReduce(OpKernelContext& ctx, int64_t M, int64_t N);

// Sum `partial` over the ranks of the session's process group and add `residual` (may be undefined).
at::Tensor GemmAllReduce(OpKernelContext& ctx, const at::Tensor& partial, const at::Tensor& residual);

void RegisterMoreCudaKernels(KernelRegistry& r);
void RegisterCudaKernels3(KernelRegistry& r);

}  // namespace ortb
