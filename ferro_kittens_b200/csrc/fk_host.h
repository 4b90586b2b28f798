// Internal host-side helpers shared by the launchers: thread-local error
// text, the CUDA-call guard, per-device scratch for the host-buffer entry points.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <mutex>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/ferro_kittens.h"

/// Record a formatted message as this thread's last error and return `code`.
int fk_fail(int code, const char* format, ...);

#define FK_CUDA(call)                                                                      \
    do {                                                                                   \
        cudaError_t fk_cuda_status = (call);                                               \
        if (fk_cuda_status != cudaSuccess)                                                 \
            return fk_fail(FK_ERR_DRIVER, "%s failed: %s", #call,                          \
                           cudaGetErrorString(fk_cuda_status));                            \
    } while (0)

namespace fk {

/// A device buffer cached per (device, slot) for the host-buffer entry points;
/// grown when a call needs more, released at process exit by the runtime.
int scratch(int slot, size_t bytes, void** out);

/// 8 status words per device for the host-buffer entry points.
int scratch_status(uint32_t** out);

/// Everything queued on `stream` has completed, or FK_ERR_TIMEOUT past the launch budget
/// (`fk_launch_budget_ms`): the library's replacement for cudaStreamSynchronize.
int wait_stream(cudaStream_t stream);

/// One lock per device, held for the whole of a host-buffer entry point: those calls share
/// the device's staging buffers, streams, events and status words.
std::mutex& device_call_guard(int device);

/// What a launch needs to know about the current device, asked of the runtime once per device:
/// a launch of a few microseconds must not pay several attribute queries each time.
struct DeviceFacts {
    int device;
    int sm_count;
    int shared_optin_limit;  // cudaDevAttrMaxSharedMemoryPerBlockOptin
};
int device_facts(DeviceFacts* out);

}  // namespace fk
