// Programmatic dependent launch: every kernel of this library is launched with the
// programmatic-stream-serialization attribute and brackets its work with the two instructions
// below, so that on a stream (or in a captured Graph) of back-to-back commands the launch
// latency, parameter fetch and prologue of command N + 1 overlap the execution of command N.
//
//   * dependent_launch_release(): first instruction of every kernel.  Once every CTA of the grid
//     has executed it, the next kernel in the stream may begin to launch.
//   * dependent_launch_wait(): executed by every thread before its first access to global
//     memory.  It returns when all earlier work in the stream has completed and its writes are
//     visible, so ordering between commands (append -> decode, partials -> merge, a caller's own
//     kernels -> ours) is exactly stream order.
//
// A kernel that follows something else than a kernel of this library (an event, a copy, a
// caller's kernel without the release instruction) simply starts when that work has finished.
#pragma once

#include <cuda_runtime.h>

namespace lb {
namespace dev {

__device__ __forceinline__ void dependent_launch_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void dependent_launch_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

} // namespace dev

// cudaLaunchKernelEx with the programmatic-stream-serialization attribute set.
template <typename... KernelArgs, typename... Args>
int launch_dependent(void (*kernel)(KernelArgs...), unsigned grid, unsigned block, size_t shared,
                     void *stream, Args &&...args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(block);
    config.dynamicSmemBytes = shared;
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// As launch_dependent, with the grid cut into thread-block clusters of `cluster` consecutive CTAs.
template <typename... KernelArgs, typename... Args>
int launch_dependent_cluster(void (*kernel)(KernelArgs...), unsigned grid, unsigned block,
                             size_t shared, unsigned cluster, void *stream, Args &&...args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(block);
    config.dynamicSmemBytes = shared;
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = cluster;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

} // namespace lb
