// Device-side objects of libkhcuda_gqa shared by its CUDA translation units: the device and stream handles
// behind the opaque C types, CUDA error mapping and buffer-size checks.
#pragma once

#include <cuda_runtime.h>

#include "common.h"

struct kh_device {
    int32_t ordinal;
    int32_t sm_count;
    uint32_t* status;     // device status word
    uint32_t wait_limit;  // polls a bounded wait inside a kernel makes before it gives up (kh_device_set_wait_limit)
};

struct kh_stream {
    kh_device* device;
    cudaStream_t stream;
    bool owned;
    kh_buffer_ref active_counts;  // bound by kh_stream_bind_active_counts: launches read their counts from it
};

struct kh_event {
    kh_device* device;
    cudaEvent_t event;
};

namespace kh {

#define KH_CUDA(call)                                                                                         \
    do {                                                                                                      \
        cudaError_t kh_cuda_err = (call);                                                                     \
        if (kh_cuda_err != cudaSuccess) {                                                                     \
            ::kh::raise(kh_cuda_err == cudaErrorMemoryAllocation ? KH_RESOURCE_EXHAUSTED : KH_UNAVAILABLE,    \
                        "%s failed: %s", #call, cudaGetErrorString(kh_cuda_err));                             \
        }                                                                                                     \
    } while (0)

inline void use_device(const kh_device* device) {
    KH_REQUIRE(device != nullptr, "device is null");
    KH_CUDA(cudaSetDevice(device->ordinal));
}

inline void need(kh_buffer_ref buffer, uint64_t bytes, const char* name) {
    KH_REQUIRE(buffer.ptr != nullptr, "%s buffer is null", name);
    KH_REQUIRE(buffer.bytes >= bytes, "%s buffer holds %llu bytes but %llu are required", name,
               (unsigned long long)buffer.bytes, (unsigned long long)bytes);
}

}  // namespace kh
