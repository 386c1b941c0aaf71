// Per-device kernel set-up, run once per context creation.
#include "backend.h"

namespace st {

cudaError_t configure_gemv_kernels();
cudaError_t configure_gemm_tc_kernels();
cudaError_t configure_gemm_pair_kernels();
cudaError_t configure_grouped_kernels();

cudaError_t configure_device() {
    cudaError_t e = configure_gemv_kernels();
    if (e == cudaSuccess) e = configure_gemm_tc_kernels();
    if (e == cudaSuccess) e = configure_gemm_pair_kernels();
    if (e == cudaSuccess) e = configure_grouped_kernels();
    return e;
}

}  // namespace st
