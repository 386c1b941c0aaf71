// What the recording launch layer of the contract tests remembers.
#pragma once
#include <vector>

#include "backend.h"

namespace mock {
struct Record {
    int launches = 0;
    int scratch_resets = 0;
    bool fail_launch = false;
    bool last_was_gemm = false;
    st::LinearCall last{};
    void* last_workspace = nullptr;
    cudaStream_t last_stream = nullptr;
    std::vector<int> configured_devices;  // st::configure_device calls, in order
};
Record& record();
}  // namespace mock
