// Programmatic dependent launch for the kernels of a training step.
//
// A step is a chain of short kernels, each a few microseconds long, so the time between the end
// of one kernel and the first instruction of the next is a large part of the step.  Launched with
// the programmatic-serialisation attribute, a kernel's blocks may become resident (parameters
// loaded, shared memory carved, barriers initialised) while the predecessor in the stream still
// runs.  The kernel then calls grid_dependency_sync() before it touches global memory: that waits
// for the predecessor to complete with its writes visible, and then lets this kernel's own
// successor begin to launch, so at most one successor is resident and waiting at any time.
//
// Every kernel launched with the attribute must call grid_dependency_sync() in every block that
// does not return at once: completion of kernel N then implies completion of kernel N-1, which is
// what makes a chain of such launches behave like plain stream order.
#pragma once

#include <cuda_runtime.h>

namespace kge {

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

// Process-wide switch (on by default; KGE_NO_DEPENDENT_LAUNCH=1 in the environment turns it off).
bool dependent_launch_enabled();

// kernel<<<grid, block, smem, stream>>>(args...) with the attribute when enabled.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

}  // namespace kge
