// Launch helper shared by the layer-operator kernels.
//
// Every kernel of the decode step is launched with the programmatic-dependent-launch
// attribute and is written in two parts: what needs nothing from the stream before it
// (index arithmetic, weight prefetch), then `pdl_wait()`, then every read of an
// activation and every global write.  The next kernel's first part therefore overlaps
// this kernel's tail, which matters when a decode step is a chain of a few hundred
// launches of a few microseconds each.
#pragma once
#include <cuda_runtime.h>

#include "common.cuh"

namespace tllm {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
int launch_pdl(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
               Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLLM_ERR_LAUNCH, "%s launch: %s", what, cudaGetErrorString(e));
    }
    return TLLM_OK;
}

}  // namespace tllm
