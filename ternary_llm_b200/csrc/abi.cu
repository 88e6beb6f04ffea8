// extern "C" entry points of libtllm_b200: argument checks and dispatch.
// Declarations, argument meaning and the reference interface each entry point
// replaces are in include/tllm_b200.h.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace tllm {

static thread_local char g_err[512] = "";

int fail(int status, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

int check_launch(const char* what)
{
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();   // clear a non-sticky launch error so later calls can proceed
        return fail(TLLM_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    }
    return TLLM_OK;
}

// The kernels are built for sm_100a only; refuse any other device loudly.
int check_device()
{
    static int ok[64] = {};   // 0 unknown, 1 good, -1 bad
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0)
        return fail(TLLM_ERR_DEVICE, "no current CUDA device");
    if (dev < 64 && ok[dev] == 1) return TLLM_OK;
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (dev < 64) ok[dev] = (major == 10) ? 1 : -1;
    if (major != 10)
        return fail(TLLM_ERR_DEVICE, "device %d has compute capability %d.x; this library is sm_100a only", dev, major);
    return TLLM_OK;
}

// Largest token count served by passes of the streaming GEMV (four vectors per pass over the
// weights); above it the tcgen05 kernel, which reads the weights once for the whole batch.
constexpr int kGemvMaxBatch = 8;

static inline bool misaligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

static int check_weights(const void* nz, const void* sg, const void* scales, int rows, int cols, int gs)
{
    if (!nz || !sg || !scales) return fail(TLLM_ERR_NULL, "null weight pointer");
    if (gs != kGroup) return fail(TLLM_ERR_GROUP, "group_size %d unsupported (must be 128)", gs);
    if (rows < 1 || cols < kGroup || cols % kGroup != 0)
        return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d: need rows >= 1 and cols a positive multiple of 128", rows, cols);
    if (misaligned(nz, 16) || misaligned(sg, 16)) return fail(TLLM_ERR_ALIGN, "mask pointers must be 16-byte aligned");
    if (misaligned(scales, 2)) return fail(TLLM_ERR_ALIGN, "scale pointer must be 2-byte aligned");
    return TLLM_OK;
}

}  // namespace tllm

using namespace tllm;

extern "C" {

const char* tllm_b200_status_string(int status)
{
    switch (status) {
        case TLLM_OK: return "ok";
        case TLLM_ERR_NULL: return "null pointer";
        case TLLM_ERR_ALIGN: return "misaligned pointer";
        case TLLM_ERR_SHAPE: return "unsupported shape";
        case TLLM_ERR_GROUP: return "unsupported group size";
        case TLLM_ERR_BATCH: return "batch out of range";
        case TLLM_ERR_LAUNCH: return "CUDA launch or runtime error";
        case TLLM_ERR_DEVICE: return "not an sm_100 device";
        case TLLM_ERR_NONCANON: return "sign bit set without nonzero bit";
        case TLLM_ERR_SIZE: return "buffer too small or size over the stated maximum";
        case TLLM_ERR_TIMEOUT: return "bounded device wait gave up";
        default: return "unknown status";
    }
}

const char* tllm_b200_last_error(void) { return g_err; }

int tllm_b200_version(void) { return 1000; }

int tllm_b200_gemv_batched(const uint32_t* nz, const uint32_t* sg, const void* scales,
                           const void* x, void* y, int batch, int rows, int cols,
                           int group_size, void* stream)
{
    int st = check_weights(nz, sg, scales, rows, cols, group_size);
    if (st) return st;
    if (!x || !y) return fail(TLLM_ERR_NULL, "null activation or output pointer");
    if (batch < 1 || batch > kMaxBatch) return fail(TLLM_ERR_BATCH, "batch %d outside 1..%d", batch, kMaxBatch);
    if (misaligned(x, 16)) return fail(TLLM_ERR_ALIGN, "activation pointer must be 16-byte aligned");
    if (misaligned(y, 2)) return fail(TLLM_ERR_ALIGN, "output pointer must be 2-byte aligned");
    if ((st = check_device())) return st;
    if (const uint8_t* packed = lookup_packed(nz, rows, cols)) {
        // up to eight vectors: the streaming GEMV (four share one weight pass); more: the
        // tensor-core kernel with a 32-token tile reads the weights once for the whole batch
        if (batch > kGemvMaxBatch && gemm_tcgen05_supported(batch, rows, cols))
            return launch_gemm_tcgen05((const half*)x, packed, (half*)y, batch, rows, cols, (cudaStream_t)stream);
        return launch_gemv_packed(packed, (const half*)x, (half*)y, batch, rows, cols, (cudaStream_t)stream);
    }
    return launch_gemv_simt(nz, sg, (const half*)scales, (const half*)x, (half*)y, batch, rows, cols,
                            (cudaStream_t)stream);
}

int tllm_b200_gemv(const uint32_t* nz, const uint32_t* sg, const void* scales, const void* x,
                   void* y, int rows, int cols, int group_size, void* stream)
{
    return tllm_b200_gemv_batched(nz, sg, scales, x, y, 1, rows, cols, group_size, stream);
}

int tllm_b200_gemv_int8(const uint32_t* nz, const uint32_t* sg, const void* weight_scales,
                        const int8_t* input_int8, float input_scale, void* y,
                        int rows, int cols, int group_size, void* stream)
{
    int st = check_weights(nz, sg, weight_scales, rows, cols, group_size);
    if (st) return st;
    if (!input_int8 || !y) return fail(TLLM_ERR_NULL, "null activation or output pointer");
    if (misaligned(input_int8, 16)) return fail(TLLM_ERR_ALIGN, "int8 activation pointer must be 16-byte aligned");
    if (misaligned(y, 2)) return fail(TLLM_ERR_ALIGN, "output pointer must be 2-byte aligned");
    if ((st = check_device())) return st;
    if (const uint8_t* packed = lookup_packed(nz, rows, cols))
        return launch_gemv_int8_packed(packed, input_int8, input_scale, (half*)y, rows, cols, (cudaStream_t)stream);
    return launch_gemv_int8_simt(nz, sg, (const half*)weight_scales, input_int8, input_scale, (half*)y,
                                 rows, cols, (cudaStream_t)stream);
}

int tllm_b200_quantize_absmax_int8(const void* x, int8_t* q, float* scale, int n, void* stream)
{
    if (!x || !q || !scale) return fail(TLLM_ERR_NULL, "null pointer");
    if (n < 1) return fail(TLLM_ERR_SHAPE, "n=%d must be positive", n);
    if (misaligned(x, 2) || misaligned(scale, 4)) return fail(TLLM_ERR_ALIGN, "misaligned input or scale pointer");
    int st = check_device();
    if (st) return st;
    return launch_quantize_absmax_int8((const half*)x, q, scale, n, (cudaStream_t)stream);
}

int tllm_b200_gemm(const void* A, const uint32_t* nz_B, const uint32_t* sign_B, const void* scales_B,
                   void* C, int M, int N, int K, int group_size, void* stream)
{
    int st = check_weights(nz_B, sign_B, scales_B, N, K, group_size);
    if (st) return st;
    if (!A || !C) return fail(TLLM_ERR_NULL, "null A or C pointer");
    if (M < 1) return fail(TLLM_ERR_SHAPE, "M=%d must be positive", M);
    if (misaligned(A, 16)) return fail(TLLM_ERR_ALIGN, "A must be 16-byte aligned");
    if (misaligned(C, 2)) return fail(TLLM_ERR_ALIGN, "C must be 2-byte aligned");
    if ((st = check_device())) return st;
    // Token blocks of at most kMaxBatch rows, each one pass over the weights.
    const uint8_t* packed = lookup_packed(nz_B, N, K);
    if (packed && M > kGemvMaxBatch && gemm_tcgen05_supported(M, N, K))
        return launch_gemm_tcgen05((const half*)A, packed, (half*)C, M, N, K, (cudaStream_t)stream);
    for (int m0 = 0; m0 < M; m0 += kMaxBatch) {
        const int b = (M - m0 < kMaxBatch) ? (M - m0) : kMaxBatch;
        if (packed) {
            st = launch_gemv_packed(packed, (const half*)A + (size_t)m0 * K, (half*)C + (size_t)m0 * N, b, N, K,
                                    (cudaStream_t)stream);
            if (st) return st;
            continue;
        }
        st = launch_gemv_simt(nz_B, sign_B, (const half*)scales_B, (const half*)A + (size_t)m0 * K,
                              (half*)C + (size_t)m0 * N, b, N, K, (cudaStream_t)stream);
        if (st) return st;
    }
    return TLLM_OK;
}

size_t tllm_b200_packed_bytes(int rows, int cols)
{
    if (rows < 1 || cols < kGroup || cols % kGroup) return 0;
    return packed_bytes(rows, cols);
}

int tllm_b200_weight_prepare(const uint32_t* nz, const uint32_t* sg, const void* scales, int rows, int cols,
                             int group_size, void* packed, size_t packed_size, void* stream)
{
    int st = check_weights(nz, sg, scales, rows, cols, group_size);
    if (st) return st;
    if (!packed) return fail(TLLM_ERR_NULL, "null packed buffer");
    if (misaligned(packed, 16)) return fail(TLLM_ERR_ALIGN, "packed buffer must be 16-byte aligned");
    if (packed_size < packed_bytes(rows, cols))
        return fail(TLLM_ERR_SIZE, "packed buffer holds %zu bytes, %zu needed", packed_size, packed_bytes(rows, cols));
    if ((st = check_device())) return st;
    return weight_prepare(nz, sg, (const half*)scales, rows, cols, (uint8_t*)packed, (cudaStream_t)stream);
}

int tllm_b200_weight_unpack(const void* packed, int rows, int cols, int group_size, uint32_t* nz,
                            uint32_t* sg, void* scales, void* stream)
{
    int st = check_weights(nz, sg, scales, rows, cols, group_size);
    if (st) return st;
    if (!packed) return fail(TLLM_ERR_NULL, "null packed buffer");
    if ((st = check_device())) return st;
    return weight_unpack((const uint8_t*)packed, rows, cols, nz, sg, (half*)scales, (cudaStream_t)stream);
}

int tllm_b200_weight_register(const uint32_t* nz, const void* packed, int rows, int cols)
{
    if (!nz || !packed) return fail(TLLM_ERR_NULL, "null pointer");
    if (rows < 1 || cols < kGroup || cols % kGroup) return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d", rows, cols);
    if (misaligned(packed, 16)) return fail(TLLM_ERR_ALIGN, "packed buffer must be 16-byte aligned");
    return weight_register(nz, (const uint8_t*)packed, rows, cols);
}

int tllm_b200_weight_unregister(const uint32_t* nz)
{
    if (!nz) return fail(TLLM_ERR_NULL, "null pointer");
    return weight_unregister(nz);
}

static int check_packed_call(const void* packed, const void* x, const void* y, int rows, int cols)
{
    if (!packed || !x || !y) return fail(TLLM_ERR_NULL, "null pointer");
    if (rows < 1 || cols < kGroup || cols % kGroup)
        return fail(TLLM_ERR_SHAPE, "rows=%d cols=%d: need rows >= 1 and cols a positive multiple of 128", rows, cols);
    if (misaligned(packed, 16) || misaligned(x, 16)) return fail(TLLM_ERR_ALIGN, "packed and activation pointers must be 16-byte aligned");
    if (misaligned(y, 2)) return fail(TLLM_ERR_ALIGN, "output pointer must be 2-byte aligned");
    return check_device();
}

int tllm_b200_gemv_packed(const void* packed, const void* x, void* y, int batch, int rows, int cols, void* stream)
{
    int st = check_packed_call(packed, x, y, rows, cols);
    if (st) return st;
    if (batch < 1 || batch > kMaxBatch) return fail(TLLM_ERR_BATCH, "batch %d outside 1..%d", batch, kMaxBatch);
    if (batch > kGemvMaxBatch && gemm_tcgen05_supported(batch, rows, cols))
        return launch_gemm_tcgen05((const half*)x, (const uint8_t*)packed, (half*)y, batch, rows, cols, (cudaStream_t)stream);
    return launch_gemv_packed((const uint8_t*)packed, (const half*)x, (half*)y, batch, rows, cols, (cudaStream_t)stream);
}

int tllm_b200_gemv_int8_packed(const void* packed, const int8_t* xq, float input_scale, void* y, int rows,
                               int cols, void* stream)
{
    int st = check_packed_call(packed, xq, y, rows, cols);
    if (st) return st;
    return launch_gemv_int8_packed((const uint8_t*)packed, xq, input_scale, (half*)y, rows, cols, (cudaStream_t)stream);
}

int tllm_b200_gemv_packed_multi(int count, const void* const* packed, void* const* y, const int* rows, int cols,
                                const void* x, void* stream)
{
    if (!packed || !y || !rows || !x) return fail(TLLM_ERR_NULL, "null pointer");
    if (count < 1 || count > TLLM_MAX_FUSED) return fail(TLLM_ERR_BATCH, "count %d outside 1..%d", count, TLLM_MAX_FUSED);
    for (int i = 0; i < count; i++) {
        const int st = check_packed_call(packed[i], x, y[i], rows[i], cols);
        if (st) return st;
    }
    return launch_gemv_packed_multi(count, (const uint8_t* const*)packed, (half* const*)y, rows, cols,
                                    (const half*)x, (cudaStream_t)stream);
}

int tllm_b200_gemv_packed_multi_norm(int count, const void* const* packed, void* const* y, const int* rows, int cols,
                                     const void* a, const void* b, const void* norm_weight, void* res_out, float eps,
                                     void* stream)
{
    if (!packed || !y || !rows || !a || !norm_weight) return fail(TLLM_ERR_NULL, "null pointer");
    if (count < 1 || count > TLLM_MAX_FUSED) return fail(TLLM_ERR_BATCH, "count %d outside 1..%d", count, TLLM_MAX_FUSED);
    for (int i = 0; i < count; i++) {
        const int st = check_packed_call(packed[i], a, y[i], rows[i], cols);
        if (st) return st;
    }
    if (misaligned(a, 16) || (b && misaligned(b, 16)) || misaligned(norm_weight, 16) || (res_out && misaligned(res_out, 16)))
        return fail(TLLM_ERR_ALIGN, "gemv_packed_multi_norm: a, b, norm_weight and res_out must be 16-byte aligned");
    if (res_out && (res_out == a || res_out == b))
        return fail(TLLM_ERR_SHAPE, "gemv_packed_multi_norm: res_out must not alias an input (other CTAs still read it)");
    return launch_gemv_packed_multi_norm(count, (const uint8_t* const*)packed, (half* const*)y, rows, cols, (const half*)a,
                                         (const half*)b, (const half*)norm_weight, (half*)res_out, eps, (cudaStream_t)stream);
}

int tllm_b200_gemv_packed_allreduce(const void* packed, const void* x, void* y, int rows, int cols, int rank, int world,
                                    void* const* peer_recv, void* epoch_local, int rows_max, void* stream)
{
    int st = check_packed_call(packed, x, y, rows, cols);
    if (st) return st;
    if (!peer_recv || !epoch_local) return fail(TLLM_ERR_NULL, "null peer buffer table");
    for (int d = 0; d < world && d < TLLM_MAX_PEERS; d++) {
        if (!peer_recv[d]) return fail(TLLM_ERR_NULL, "null receive buffer of rank %d", d);
        if (misaligned(peer_recv[d], 8)) return fail(TLLM_ERR_ALIGN, "receive buffers must be 8-byte aligned");
    }
    return launch_gemv_packed_allreduce((const uint8_t*)packed, (const half*)x, (half*)y, rows, cols, rank, world,
                                        peer_recv, epoch_local, rows_max, (cudaStream_t)stream);
}

int tllm_b200_allreduce_trace(void* buffer, int records)
{
    if (buffer && misaligned(buffer, 8)) return fail(TLLM_ERR_ALIGN, "trace buffer must be 8-byte aligned");
    return allreduce_set_trace(buffer, records);
}

int tllm_b200_gemv_packed_noalloc(const void* packed, const void* x, void* y, int rows, int cols, void* stream)
{
    int st = check_packed_call(packed, x, y, rows, cols);
    if (st) return st;
    return launch_gemv_packed_noalloc((const uint8_t*)packed, (const half*)x, (half*)y, rows, cols,
                                      (cudaStream_t)stream);
}

int tllm_b200_gemv_packed_noalloc_status(void* stream)
{
    int st = check_device();
    if (st) return st;
    return noalloc_error_check((cudaStream_t)stream);
}

int tllm_b200_gemm_packed(const void* A, const void* packed, void* C, int M, int N, int K, void* stream)
{
    if (!A || !packed || !C) return fail(TLLM_ERR_NULL, "null pointer");
    if (M < 1 || N < 1 || K < kGroup || K % kGroup)
        return fail(TLLM_ERR_SHAPE, "M=%d N=%d K=%d: need M,N >= 1 and K a positive multiple of 128", M, N, K);
    if (misaligned(A, 16) || misaligned(packed, 16)) return fail(TLLM_ERR_ALIGN, "A and packed must be 16-byte aligned");
    if (misaligned(C, 2)) return fail(TLLM_ERR_ALIGN, "C must be 2-byte aligned");
    int st = check_device();
    if (st) return st;
    if (M <= kGemvMaxBatch)
        return launch_gemv_packed((const uint8_t*)packed, (const half*)A, (half*)C, M, N, K, (cudaStream_t)stream);
    return launch_gemm_tcgen05((const half*)A, (const uint8_t*)packed, (half*)C, M, N, K, (cudaStream_t)stream);
}

int tllm_b200_check_device_errors(void* stream)
{
    int st = check_device();
    if (st) return st;
    return device_error_check((cudaStream_t)stream);
}

}  // extern "C"
