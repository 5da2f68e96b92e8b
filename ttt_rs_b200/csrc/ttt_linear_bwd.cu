// placeholder until the backward kernel lands
#include "ttt_kernels.h"
namespace ttt {
cudaError_t launch_linear_bwd(int, const CUtensorMap*, const LinBwdParams&, int, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_linear_bwd_reduce(const ReduceParams&, cudaStream_t) { return cudaErrorNotSupported; }
}
