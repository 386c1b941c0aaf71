// A CUDA runtime made of counters, for the host-side contract tests only.  The real host
// API sources (strix_trellis_b200/csrc/api_*.cpp) are compiled against this header instead of
// the toolkit's, so every allocation, copy, synchronisation, pointer or stream query they
// make is counted and any of them can be made to fail.  "Device memory" is host memory that
// this runtime remembers the owner device of.  Nothing here touches a GPU.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <vector>

typedef int cudaError_t;
enum : int {
    cudaSuccess = 0,
    cudaErrorInvalidValue = 1,
    cudaErrorMemoryAllocation = 2,
    cudaErrorInvalidDevice = 101,
    cudaErrorLaunchFailure = 719,
};
struct fake_stream_tag;
typedef fake_stream_tag* cudaStream_t;
enum cudaMemcpyKind { cudaMemcpyHostToHost, cudaMemcpyHostToDevice, cudaMemcpyDeviceToHost, cudaMemcpyDeviceToDevice };
enum cudaDeviceAttr { cudaDevAttrComputeCapabilityMajor = 75, cudaDevAttrMultiProcessorCount = 16 };
enum cudaMemoryType { cudaMemoryTypeUnregistered = 0, cudaMemoryTypeHost = 1, cudaMemoryTypeDevice = 2, cudaMemoryTypeManaged = 3 };
struct cudaPointerAttributes { cudaMemoryType type; int device; void* devicePointer; void* hostPointer; };
enum cudaStreamCaptureStatus { cudaStreamCaptureStatusNone = 0, cudaStreamCaptureStatusActive = 1 };
enum cudaDriverEntryPointQueryResult { cudaDriverEntryPointSuccess = 0, cudaDriverEntryPointSymbolNotFound = 1 };
constexpr unsigned long long cudaEnableDefault = 0;

namespace fake {
struct Block { size_t bytes; int device; };
struct State {
    // what the "machine" looks like
    int current_device = 0;
    int device_count = 2;
    int capability_major = 10;
    int sm_count = 148;
    // streams other than the null stream that exist, with their device
    std::map<void*, int> streams;
    // live device allocations
    std::map<uintptr_t, Block> blocks;
    // counters
    int allocs = 0, frees = 0, copies = 0, memsets = 0, syncs = 0;
    int pointer_queries = 0, range_queries = 0, stream_queries = 0, device_queries = 0;
    std::vector<const void*> copy_sources;
    // failure injection: a call whose running number equals *_failure_at fails once
    int alloc_failure_at = -1, copy_failure_at = -1;
    bool fail_sync = false;
    bool capturing = false;
};
State& state();
void reset();
}  // namespace fake

cudaError_t cudaGetDevice(int* device);
cudaError_t cudaGetLastError();
cudaError_t cudaDeviceGetAttribute(int* value, cudaDeviceAttr attr, int device);
cudaError_t cudaMalloc(void** out, size_t bytes);
cudaError_t cudaFree(void* p);
cudaError_t cudaMemcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind);
cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t s);
cudaError_t cudaMemset(void* dst, int value, size_t bytes);
cudaError_t cudaMemsetAsync(void* dst, int value, size_t bytes, cudaStream_t s);
cudaError_t cudaStreamSynchronize(cudaStream_t s);
cudaError_t cudaDeviceSynchronize();
cudaError_t cudaStreamGetDevice(cudaStream_t s, int* device);
cudaError_t cudaStreamGetFlags(cudaStream_t s, unsigned int* flags);
cudaError_t cudaStreamIsCapturing(cudaStream_t s, cudaStreamCaptureStatus* status);
cudaError_t cudaPointerGetAttributes(cudaPointerAttributes* out, const void* p);
cudaError_t cudaGetDriverEntryPoint(const char* symbol, void** fn, unsigned long long flags,
                                    cudaDriverEntryPointQueryResult* result);
