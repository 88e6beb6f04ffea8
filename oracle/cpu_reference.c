/*
 * CPU restatement of the reference's scalar ternary matvec -- TEST INFRASTRUCTURE.
 *
 * Follows cpu_reference in the reference project, tests/test_ternary_gemv.cu:40-75:
 * per row, per group of `group_size` weights, per weight: test the nonzero bit,
 * then the sign bit, add +x / -x / 0 in float32; multiply the group sum by the
 * group's scale; sum the groups in float32.
 *
 * Nothing in the shipped library links or calls this file.  It is the checker for
 * the GPU kernels and the timed CPU baseline of the benchmark.  It is itself
 * checked against the reference's compiled cpu_reference (oracle/_ref) and the
 * fixtures under tests/golden/.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -shared -fPIC)
 */
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* IEEE binary16 -> binary32, exact (handles subnormals, inf, nan). */
static float half_bits_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp  = (h >> 10) & 0x1fu;
    uint32_t man  = h & 0x3ffu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7f800000u | (man << 13);
    } else {
        out = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* One row, as the reference writes it (tests/test_ternary_gemv.cu:51-73). */
static float row_dot(const uint32_t *nz, const uint32_t *sg, const float *scales,
                     const float *x, int cols, int group_size)
{
    int groups = cols / group_size;
    float sum = 0.0f;
    for (int g = 0; g < groups; g++) {
        float group_sum = 0.0f;
        int c0 = g * group_size;
        for (int j = 0; j < group_size; j++) {
            int col = c0 + j;
            uint32_t a = nz[col >> 5], b = sg[col >> 5];
            int bit = col & 31;
            float w = ((a >> bit) & 1u) ? (((b >> bit) & 1u) ? 1.0f : -1.0f) : 0.0f;
            group_sum += w * x[col];
        }
        sum += scales[g] * group_sum;
    }
    return sum;
}

/* float scales / float input, single thread: the reference's exact signature. */
void oracle_matvec_f32(const uint32_t *nz, const uint32_t *sg, const float *scales,
                       const float *x, float *y, int rows, int cols, int group_size)
{
    int mpr = cols / 32, gpr = cols / group_size;
    for (int r = 0; r < rows; r++)
        y[r] = row_dot(nz + (size_t)r * mpr, sg + (size_t)r * mpr,
                       scales + (size_t)r * gpr, x, cols, group_size);
}

/* Same arithmetic, rows spread over `threads` host threads (0 = all). */
void oracle_matvec_f32_mt(const uint32_t *nz, const uint32_t *sg, const float *scales,
                          const float *x, float *y, int rows, int cols, int group_size,
                          int threads)
{
    int mpr = cols / 32, gpr = cols / group_size;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
    (void)threads;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        y[r] = row_dot(nz + (size_t)r * mpr, sg + (size_t)r * mpr,
                       scales + (size_t)r * gpr, x, cols, group_size);
}

/* Inputs as stored on the device: float16 scales and activations (bit patterns).
 * x is [batch, cols], y is [batch, rows] float32.  scratch-free, threaded. */
void oracle_matvec_f16(const uint32_t *nz, const uint32_t *sg, const uint16_t *scales_h,
                       const uint16_t *x_h, float *y, int batch, int rows, int cols,
                       int group_size, int threads)
{
    int mpr = cols / 32, gpr = cols / group_size;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
    (void)threads;
#pragma omp parallel
    {
        float xf[cols];
        float sf[gpr];
        for (int b = 0; b < batch; b++) {
            for (int k = 0; k < cols; k++) xf[k] = half_bits_to_float(x_h[(size_t)b * cols + k]);
#pragma omp for schedule(static)
            for (int r = 0; r < rows; r++) {
                for (int g = 0; g < gpr; g++) sf[g] = half_bits_to_float(scales_h[(size_t)r * gpr + g]);
                y[(size_t)b * rows + r] = row_dot(nz + (size_t)r * mpr, sg + (size_t)r * mpr,
                                                  sf, xf, cols, group_size);
            }
        }
    }
}

/* INT8-activation form (kernels/ternary_gemv.cu:116-199): exact integer group
 * sums, float32 scale per group, one multiply by input_scale per row. */
void oracle_matvec_i8(const uint32_t *nz, const uint32_t *sg, const uint16_t *scales_h,
                      const int8_t *x, float input_scale, float *y, int rows, int cols,
                      int group_size, int threads)
{
    int mpr = cols / 32, gpr = cols / group_size;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
    (void)threads;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint32_t *a = nz + (size_t)r * mpr, *b = sg + (size_t)r * mpr;
        float acc = 0.0f;
        for (int g = 0; g < gpr; g++) {
            int gsum = 0;
            for (int j = 0; j < group_size; j++) {
                int col = g * group_size + j, bit = col & 31;
                int nzb = (a[col >> 5] >> bit) & 1, sgb = (b[col >> 5] >> bit) & 1;
                gsum += nzb * (2 * sgb - 1) * (int)x[col];
            }
            acc += half_bits_to_float(scales_h[(size_t)r * gpr + g]) * (float)gsum;
        }
        y[r] = acc * input_scale;
    }
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
