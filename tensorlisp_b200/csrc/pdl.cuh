// Programmatic dependent launch for the kernels of a decode step. A kernel launched through
// launch_pdl may start (set up barriers, allocate tensor memory, prefetch WEIGHTS) while the kernel
// before it in the stream is still running; it must execute griddep_wait() before it reads anything
// an earlier kernel wrote or writes anything an earlier kernel may still read. griddep_launch() at
// its top lets the kernel after it do the same. Kernels launched the ordinary way keep the ordinary
// stream order on both sides. TLB_NO_PDL=1 turns the attribute off (the device-side calls are then
// no-ops).
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include <utility>

namespace tlb {

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = [] {
        const char *e = getenv("TLB_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace tlb
