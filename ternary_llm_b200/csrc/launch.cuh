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

#include <mutex>
#include <unordered_set>

#include "common.cuh"

namespace tllm {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Every kernel of the library asks for the largest shared-memory carve-out.  The streaming
// GEMV needs it (two CTAs of about 90 KB per SM); if its neighbours in a decode step ran
// with another split of the SM's L1/shared memory, each change of kernel would have to wait
// for the SMs to drain and be reconfigured, which defeats the overlap of consecutive launches.
inline void prefer_max_shared(const void* kernel)
{
    static std::mutex mu;
    static std::unordered_set<unsigned long long> done;
    int dev = 0;
    cudaGetDevice(&dev);
    const unsigned long long key = (unsigned long long)reinterpret_cast<uintptr_t>(kernel) * 64ull + (unsigned)dev;
    std::lock_guard<std::mutex> lk(mu);
    if (done.insert(key).second)
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}


template <typename... KArgs, typename... Args>
int launch_pdl(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
               Args... args)
{
    prefer_max_shared(reinterpret_cast<const void*>(kernel));
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
