#include "common.cuh"
namespace flexattn {
int launch_sm100_dq(cudaStream_t, const DevParams&, int, int) { return FLEXATTN_ERR_UNSUPPORTED_BACKEND; }
int launch_sm100_dkv(cudaStream_t, const DevParams&, int, int) { return FLEXATTN_ERR_UNSUPPORTED_BACKEND; }
}
