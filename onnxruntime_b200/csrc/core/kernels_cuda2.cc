#include "collective.h"
#include "cuda_ops.h"
#include "session.h"

namespace ortb {

at::Tensor GemmAllReduce(OpKernelContext& ctx, const at::Tensor& partial, const at::Tensor& residual) {
  at::Tensor y = AllReduceSum(ctx.session(), partial);
  if (residual.defined()) y = y + residual;
  return y;
}

void RegisterMoreCudaKernels(KernelRegistry&) {}

}  // namespace ortb
