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

#ifdef TLLM_PROFILE_PHASES
// Timeline probe (never compiled into the shipped library): CTA 0 of every launch appends
// {kernel id, phase, globaltimer} records to a per-translation-unit buffer.
static __device__ unsigned long long g_tl_rec[3 * 8192];
static __device__ unsigned g_tl_n;
__device__ __forceinline__ void tl_mark(int kernel_id, int phase)
{
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const unsigned i = atomicAdd(&g_tl_n, 1u);
        if (i < 8192) {
            g_tl_rec[3 * i] = (unsigned long long)kernel_id;
            g_tl_rec[3 * i + 1] = (unsigned long long)phase;
            g_tl_rec[3 * i + 2] = t;
        }
    }
}
#define TL_MARK(id, ph) tl_mark(id, ph)
#define TL_DUMP(name)                                                                          \
    extern "C" int name(unsigned long long* out, int max_rec)                                  \
    {                                                                                          \
        unsigned n = 0;                                                                        \
        cudaMemcpyFromSymbol(&n, tllm::g_tl_n, sizeof(n));                                           \
        if ((int)n > max_rec) n = (unsigned)max_rec;                                           \
        cudaMemcpyFromSymbol(out, tllm::g_tl_rec, sizeof(unsigned long long) * 3 * n);               \
        const unsigned zero = 0;                                                               \
        cudaMemcpyToSymbol(tllm::g_tl_n, &zero, sizeof(zero));                                       \
        return (int)n;                                                                         \
    }
#else
#define TL_MARK(id, ph)
#define TL_DUMP(name)
#endif

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
