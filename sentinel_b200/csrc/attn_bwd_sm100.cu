// placeholder until the tcgen05 backward lands
#include "common.cuh"
#include "sm100_ptx.cuh"
namespace sntl {
bool tc_bwd_supported(const AttnShape&) { return false; }
size_t tc_backward_workspace_bytes(const AttnShape&) { return 0; }
cudaError_t tc_backward(const TcArgs&, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t read_and_clear_bwd_status(cudaStream_t, uint32_t* w) { *w = 0; return cudaSuccess; }
}
