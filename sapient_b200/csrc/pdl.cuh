// Programmatic dependent launch (PDL) helpers.
//
// A decode step is a chain of ~330 short kernels. Launched with the programmatic-stream-serialization
// attribute, kernel N+1 may start while kernel N is still running: everything it does before
// pdl_wait() (for the GEMV: fetching its first weight tiles, which no kernel ever writes) overlaps
// kernel N; pdl_wait() then blocks until kernel N has completed and its writes are visible.
// Every kernel launched through launch_pdl() must call pdl_wait() before it reads or writes anything
// another kernel of the chain touches. pdl_trigger() lets the next kernel begin its own prologue.
// Without the attribute both instructions do nothing.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <utility>

namespace sp {

// Function attributes (the opt-in to large dynamic shared memory) belong to a device: one flag per device of the process.
constexpr int SP_MAX_DEVICES = 64;
inline int current_device_index() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev >= 0 && dev < SP_MAX_DEVICES ? dev : 0;
}


// Multiprocessor count of the device the calling thread has current (cached per device; engines on different devices
// and threads may ask concurrently).
inline int device_sm_count() {
    static std::atomic<int> cache[SP_MAX_DEVICES];
    const int di = current_device_index();
    int v = cache[di].load(std::memory_order_relaxed);
    if (v == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cache[di].store(v, std::memory_order_relaxed);
    }
    return v;
}

// One-time per-device function attributes (the opt-in to large dynamic shared memory): set() runs at least once per
// device before the first launch there; a second thread racing the first may run it again, which is harmless.
struct PerDeviceOnce {
    std::atomic<bool> done[SP_MAX_DEVICES];
    template <typename F>
    cudaError_t run(F&& set) {
        std::atomic<bool>& d = done[current_device_index()];
        if (d.load(std::memory_order_acquire)) return cudaSuccess;
        const cudaError_t e = set();
        if (e == cudaSuccess) d.store(true, std::memory_order_release);
        return e;
    }
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

bool pdl_enabled();            // kernels.cu; default on, SAPIENT_CUDA_PDL=0 turns it off
void pdl_set_enabled(bool on);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace sp
