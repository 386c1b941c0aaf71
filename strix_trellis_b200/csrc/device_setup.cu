// Per-device kernel set-up, run once per context creation.
#include "backend.h"

#include <atomic>

namespace st {

cudaError_t configure_gemv_kernels();
cudaError_t configure_gemm_tc_kernels();
cudaError_t configure_gemm_pair_kernels();
cudaError_t configure_grouped_kernels();

// SM count of the current device, looked up once per device ordinal.
int device_sm_count() {
    constexpr int kDevices = 64;
    static std::atomic<int> known[kDevices];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDevices) return 1;
    int sms = known[device].load(std::memory_order_relaxed);
    if (sms == 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1) return 1;
        known[device].store(sms, std::memory_order_relaxed);
    }
    return sms;
}

cudaError_t configure_device() {
    cudaError_t e = configure_gemv_kernels();
    if (e == cudaSuccess) e = configure_gemm_tc_kernels();
    if (e == cudaSuccess) e = configure_gemm_pair_kernels();
    if (e == cudaSuccess) e = configure_grouped_kernels();
    return e;
}

}  // namespace st
