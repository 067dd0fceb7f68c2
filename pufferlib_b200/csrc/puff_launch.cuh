// Programmatic dependent launch: the device-side hooks and the host-side launch helper shared by
// every kernel file of the library.
#pragma once
#include <cuda_runtime.h>

#include "../../include/puff_advantage.h"

namespace puff {

// A kernel launched with the programmatic-stream-serialization attribute
// may start while its predecessor in the stream is still running: its CTAs become
// resident as soon as every CTA of the predecessor has executed launch_dependents (or exited) and
// resources allow.  pdl_wait() then blocks until the predecessor grid has completed and its
// memory operations are visible, so everything before it must touch no global memory that an
// earlier kernel may still read or write: only the kernel's own set-up (shared-memory carve-up,
// mbarrier initialisation, fetching the tensor-map descriptors, which are kernel parameters)
// overlaps the predecessor's tail.  Both are no-ops in a launch without the attribute.  A kernel
// launched through launch_kernel() below MUST call pdl_wait() before its first global access:
// with the attribute, nothing else orders it behind the previous kernel of the stream.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

int tune_value(int knob, int fallback);   // puff_advantage_sm100.cu: a PUFF_TUNE_* knob, or the fallback while unset

// Launch with the programmatic-stream-serialization attribute.  PUFF_TUNE_PDL: 1 (default) every
// kernel that comes through here, 2 only the advantage kernels (`core`), 0 none.
template <typename... KArgs, typename... Args>
static cudaError_t launch_with_pdl(bool core, void (*kernel)(KArgs...), int grid, int block, size_t smem,
                                   cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(block));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const int mode = tune_value(PUFF_TUNE_PDL, 1);
    cfg.numAttrs = (mode == 1 || (mode == 2 && core)) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// the advantage kernels
template <typename... KArgs, typename... Args>
static cudaError_t launch_kernel(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st,
                                 Args... args)
{
    return launch_with_pdl(true, kernel, grid, block, smem, st, args...);
}
// The kernels either side of the op (sampler prologue, exchange, minibatch gather).  Used for the
// second and later kernels of an entry point only: the first one is a plain launch, because
// what precedes it in the stream is not this library's to know, and a programmatically launched
// kernel behind an advantage kernel of another stream was measured to slow the pipelined step.
template <typename... KArgs, typename... Args>
static cudaError_t launch_neighbour(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st,
                                    Args... args)
{
    return launch_with_pdl(false, kernel, grid, block, smem, st, args...);
}

}  // namespace puff
