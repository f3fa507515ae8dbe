// tcgen05 forward kernels (placeholder until the tensor-core path lands).
#include "common.cuh"
namespace fdmla {
bool fwd_tensor_supported(const FwdProblem &, int) { return false; }
int launch_fwd_tensor(const FwdProblem &, int, cudaStream_t) { return FDMLA_ERR_UNSUPPORTED; }
}  // namespace fdmla
