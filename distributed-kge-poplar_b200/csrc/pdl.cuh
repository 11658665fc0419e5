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

// State that CUDA keeps per device (function attributes, occupancy answers) is cached per device:
// the slot of the current device, or -1 when it cannot be cached (then the caller asks CUDA again).
constexpr int kMaxDeviceOrdinals = 64;
inline int current_device_slot() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDeviceOrdinals) return -1;
    return device;
}

// Process-wide switch (on by default; KGE_NO_DEPENDENT_LAUNCH=1 in the environment turns it off).
bool dependent_launch_enabled();

// kernel<<<grid, block, smem, stream>>>(args...) with the attribute when enabled; cluster_z > 1
// also makes every cluster_z blocks that are neighbours in z one thread-block cluster.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            unsigned cluster_z, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    unsigned n = 0;
    if (dependent_launch_enabled()) {
        attribute[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attribute[n].id = cudaLaunchAttributeClusterDimension;
        attribute[n].val.clusterDim.x = 1;
        attribute[n].val.clusterDim.y = 1;
        attribute[n].val.clusterDim.z = cluster_z;
        ++n;
    }
    config.attrs = attribute;
    config.numAttrs = n;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    return launch_dependent_cluster(kernel, grid, block, smem, stream, 1u, static_cast<Args&&>(args)...);
}

}  // namespace kge
