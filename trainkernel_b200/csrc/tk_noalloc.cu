// tk_module_launch_static_workspace: launch a loaded training-step kernel without the caller
// (or this library) allocating anything.
//
// Who needs it: code that must not call cudaMalloc at the point where the step is launched —
// a host thread inside a latency-critical loop where an allocation could stall behind other
// work on the device, a caller that has handed the whole device heap to another allocator, or a
// service whose allocation calls are forbidden after start-up.  tk_module_launch expects such a
// caller to own a workspace buffer; this entry point lends it one instead.
//
// The workspace is the file-scope device array below: TK_STATIC_WORKSPACE_BYTES (4 MiB) per
// device, reserved for as long as this library is loaded in a process that has touched that
// device.  Kernels whose plan needs more are rejected, and so is a `device` that is not the one the
// module was loaded on (the address handed to the kernel would belong to another GPU's array).  Every call on a device uses the same
// array, so two launches that can overlap on the GPU (different streams, or different modules)
// race on it; order them on one stream.  The generated kernels write every workspace region
// before reading it, so nothing has to be cleared between calls; whatever the previous call
// left there is simply overwritten.
//
// In host code the array's name is only a handle for the runtime, not a device address.  The
// address is obtained with cudaGetSymbolAddress the first time a device is used, with that
// device current; that first call may initialise the CUDA runtime for the device, so make it
// before any stream capture begins.  Later calls do no set-up.
#include "trainkernel_rt.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

static __device__ __align__(256) unsigned char tk_static_workspace[TK_STATIC_WORKSPACE_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_address[kMaxDevices] = {};

int report(char* error, size_t capacity, int code, const char* format, const char* detail, unsigned long long a, unsigned long long b) {
    if (error && capacity) snprintf(error, capacity, format, detail, a, b);
    return code;
}

}  // namespace

extern "C" int tk_module_launch_static_workspace(tk_module* module, int device, const void* const* inputs,
                                                 void* const* outputs, size_t workspace_bytes, int grid,
                                                 void* stream, char* error, size_t error_capacity) {
    if (error && error_capacity) error[0] = '\0';
    if (!module || device < 0 || device >= kMaxDevices)
        return report(error, error_capacity, TK_E_ARGUMENT, "trainkernel: invalid argument to %s (device %llu of at most %llu)",
                      "tk_module_launch_static_workspace", (unsigned long long)(device < 0 ? 0 : device), (unsigned long long)kMaxDevices);
    // What the caller says must agree with what the module knows about itself: a wrong ordinal would hand
    // the kernel the address of another GPU's copy of the array, an understated size would let it write
    // past the end.
    int loaded_on = -1;
    size_t planned = 0;
    if (tk_module_device(module, &loaded_on) || tk_module_workspace_bytes(module, &planned))
        return report(error, error_capacity, TK_E_ARGUMENT, "trainkernel: %s: the module handle is not valid (%llu, %llu)",
                      "tk_module_launch_static_workspace", 0ull, 0ull);
    if (loaded_on != device)
        return report(error, error_capacity, TK_E_ARGUMENT,
                      "trainkernel: %s: the module was loaded on device %llu, not on device %llu",
                      "tk_module_launch_static_workspace", (unsigned long long)loaded_on, (unsigned long long)device);
    if (planned > workspace_bytes) workspace_bytes = planned;
    if (workspace_bytes > TK_STATIC_WORKSPACE_BYTES)
        return report(error, error_capacity, TK_E_CAPACITY,
                      "trainkernel: %s: the kernel needs %llu workspace bytes but the built-in workspace holds %llu; use tk_module_launch with a caller-owned buffer",
                      "tk_module_launch_static_workspace", (unsigned long long)workspace_bytes, (unsigned long long)TK_STATIC_WORKSPACE_BYTES);
    void* workspace = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_mutex);
        if (!g_address[device]) {
            // Make the module's device current for the lookup.  The previous device is put back only when
            // it was a different one: selecting a device this process never used would create a context there.
            int previous = device;
            cudaError_t status = cudaGetDevice(&previous);
            if (status == cudaSuccess && previous != device) status = cudaSetDevice(device);
            void* address = nullptr;
            if (status == cudaSuccess) {
                status = cudaGetSymbolAddress(&address, tk_static_workspace);
                if (previous != device) cudaSetDevice(previous);
            }
            if (status != cudaSuccess || !address)
                return report(error, error_capacity, static_cast<int>(status ? status : cudaErrorUnknown),
                              "trainkernel: cudaGetSymbolAddress for the built-in workspace failed: %s (device %llu, code %llu)",
                              cudaGetErrorString(status), (unsigned long long)device, (unsigned long long)status);
            g_address[device] = address;
        }
        workspace = g_address[device];
    }
    const int code = tk_module_launch(module, inputs, outputs, workspace, grid, stream);
    if (code && error && error_capacity) snprintf(error, error_capacity, "%s", tk_last_error());
    return code;
}
