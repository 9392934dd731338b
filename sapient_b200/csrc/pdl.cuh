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

#include <utility>

namespace sp {

// Function attributes (the opt-in to large dynamic shared memory) belong to a device: one flag per device of the process.
constexpr int SP_MAX_DEVICES = 64;
inline int current_device_index() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev >= 0 && dev < SP_MAX_DEVICES ? dev : 0;
}


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
