/*
 * CPU oracle for the OFT / GEMM hot path.  TEST INFRASTRUCTURE ONLY: nothing in the shipped
 * library links, loads or calls this file; it exists so that the parity tests, the smoke check
 * and the cpu_baseline leg of the benchmark have a checker that is independent of the CUDA path.
 *
 * It restates, as plain C loops, the arithmetic of the reference's scalar CPU routine
 *   cpu_oft_tn            cpu_oft.hpp:22-116   (driver: zero C, loop groups x K-blocks)
 *   ez_gemm               cpu_oft.hpp:9-20     (fp32 accumulate in index order, one fp16 rounding
 *                                               per output element per call)
 * and of the fp64 triple loop the reference's GEMM driver uses as its truth
 *   gemm_sm80_tc.cu:557-568 (C column-major, A/B indexed by the trans flags).
 *
 * Parity status: PINNED.  oft_oracle_cpu_oft_tn is checked bit-for-bit against the unmodified
 * reference header compiled from where it lies (oracle/build_ref.sh -> oracle/_ref/), and against
 * the golden vectors that this comparison produced (tests/golden/).
 *
 * Storage contract (cute_oft_pc.cu:258-262, cpu_oft.hpp:34-93), all row-major, fp16 bit patterns:
 *   A [m][k]            activations
 *   R [n_groups*b][k]   block (g,kb) = rows g*b..g*b+b-1, cols kb*b..kb*b+b-1; the stored block is
 *                       the transpose of the mathematical rotation: XR[i][q] = sum_p A[i][kb*b+p] * R[g*b+q][kb*b+p]
 *   B [n][k]            weight transposed (B[j][kk] = W[kk][j]), n = group_size*n_groups
 *   C [m][n]            output
 *
 * Build: gcc -O3 -mf16c -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: the reference's host build performs a separate multiply and add.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) { f16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f2h(float f) { f16 v = (f16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

int oft_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* One output row of cpu_oft_tn.  Rows of C depend only on the same row of A, so the row loop can be
 * hoisted outside the (g, kb) loops of cpu_oft.hpp:101-115 without changing a single rounding:
 * for each element the sequence of fp32 adds and fp16 roundings is identical. */
static void oft_row(const uint16_t* a_row, const uint16_t* R, const uint16_t* B, uint16_t* c_row,
                    int group_size, int n_groups, int k, int b, float* ar /* b floats of scratch */) {
    const int n = group_size * n_groups;
    const int n_blocks = k / b;
    for (int j = 0; j < n; ++j) c_row[j] = 0;                       /* cpu_oft.hpp:31 */
    for (int g = 0; g < n_groups; ++g) {
        for (int kb = 0; kb < n_blocks; ++kb) {
            /* first ez_gemm (cpu_oft.hpp:104-108): AR = half(0 + sum_p A*R), fp32 accumulate */
            for (int q = 0; q < b; ++q) {
                float acc = 0.0f;
                const uint16_t* r_row = R + (size_t)(g * b + q) * k + (size_t)kb * b;
                const uint16_t* a_blk = a_row + (size_t)kb * b;
                for (int p = 0; p < b; ++p) acc += h2f(a_blk[p]) * h2f(r_row[p]);
                ar[q] = h2f(f2h(acc));
            }
            /* second ez_gemm (cpu_oft.hpp:109-113): C = half(float(C) + sum_q AR*B) */
            for (int j = 0; j < group_size; ++j) {
                float acc = h2f(c_row[g * group_size + j]);
                const uint16_t* b_row = B + (size_t)(g * group_size + j) * k + (size_t)kb * b;
                for (int q = 0; q < b; ++q) acc += ar[q] * h2f(b_row[q]);
                c_row[g * group_size + j] = f2h(acc);
            }
        }
    }
}

/* Restatement of cpu_oft_tn (cpu_oft.hpp:22-116).  threads <= 1 runs on the calling thread like the
 * reference (which has no OpenMP); threads > 1 splits rows across OpenMP threads (bit-identical). */
int oft_oracle_cpu_oft_tn(const uint16_t* A, const uint16_t* R, const uint16_t* B, uint16_t* C,
                          int m, int group_size, int n_groups, int k, int reconn_sz, int threads) {
    if (m < 0 || group_size <= 0 || n_groups <= 0 || k < 0 || reconn_sz <= 0) return 1;
    if (k % reconn_sz != 0) return 2;
    const int n = group_size * n_groups;
    int fail = 0;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
#endif
    {
        float* ar = (float*)malloc(sizeof(float) * (size_t)reconn_sz);
        if (!ar) {
#ifdef _OPENMP
#pragma omp atomic write
#endif
            fail = 1;
        } else {
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 4)
#endif
            for (int i = 0; i < m; ++i)
                oft_row(A + (size_t)i * k, R, B, C + (size_t)i * n, group_size, n_groups, k, reconn_sz, ar);
            free(ar);
        }
    }
    return fail ? 3 : 0;
}

/* Analysis variant (not the parity oracle): same contraction order, fp64 accumulate, no intermediate
 * rounding of C; XR is rounded to fp16 iff round_xr != 0.  Separates the oracle's per-K-block fp16
 * re-rounding of C from real kernel error.  Output in double, row-major [m][n]. */
int oft_oracle_f64(const uint16_t* A, const uint16_t* R, const uint16_t* B, double* C,
                   int m, int group_size, int n_groups, int k, int b, int round_xr, int threads) {
    if (k % b != 0) return 2;
    const int n = group_size * n_groups;
    const int n_blocks = k / b;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 4)
#endif
    for (int i = 0; i < m; ++i) {
        double* c_row = C + (size_t)i * n;
        double* ar = (double*)malloc(sizeof(double) * (size_t)b);
        for (int j = 0; j < n; ++j) c_row[j] = 0.0;
        for (int g = 0; g < n_groups; ++g)
            for (int kb = 0; kb < n_blocks; ++kb) {
                for (int q = 0; q < b; ++q) {
                    double acc = 0.0;
                    const uint16_t* r_row = R + (size_t)(g * b + q) * k + (size_t)kb * b;
                    for (int p = 0; p < b; ++p) acc += (double)h2f(A[(size_t)i * k + kb * b + p]) * (double)h2f(r_row[p]);
                    ar[q] = round_xr ? (double)h2f(f2h((float)acc)) : acc;
                }
                for (int j = 0; j < group_size; ++j) {
                    const uint16_t* b_row = B + (size_t)(g * group_size + j) * k + (size_t)kb * b;
                    double acc = 0.0;
                    for (int q = 0; q < b; ++q) acc += ar[q] * (double)h2f(b_row[q]);
                    c_row[g * group_size + j] += acc;
                }
            }
        free(ar);
    }
    return 0;
}

/* ---- GEMM truth: fp64 triple loop of gemm_sm80_tc.cu:557-568 --------------------------------------
 * a(i,l) = transA in {T,t} ? A[i*ldA + l] : A[i + l*ldA]
 * b(l,j) = transB in {T,t} ? B[l*ldB + j] : B[l + j*ldB]
 * The reference stores ref_C[j*m + i]; here only the sampled rows/columns are produced:
 * out[jj*n_rows + ii] = sum_l a(rows[ii], l) * b(l, cols[jj])     (column-major in the sample).
 * dtype: 0 = fp16 bit patterns, 1 = fp32.  tf32_mode (fp32 only): 0 = use the fp32 values as they
 * are, 1 = drop the low 13 mantissa bits (what a TF32 tensor core consumes), 2 = round-to-nearest
 * to 10 mantissa bits. */
static inline double load_elem(const void* p, size_t idx, int dtype, int tf32_mode) {
    if (dtype == 0) return (double)h2f(((const uint16_t*)p)[idx]);
    uint32_t u; memcpy(&u, (const char*)p + idx * 4, 4);
    if (tf32_mode == 1) u &= 0xFFFFE000u;
    else if (tf32_mode == 2) { if ((u & 0x7F800000u) != 0x7F800000u) { u += 0x00000FFFu + ((u >> 13) & 1u); u &= 0xFFFFE000u; } }
    float f; memcpy(&f, &u, 4);
    return (double)f;
}

int gemm_oracle_f64_sampled(char transA, char transB, int m, int n, int k,
                            const void* A, int ldA, const void* B, int ldB,
                            const int* rows, int n_rows, const int* cols, int n_cols,
                            double* out, int dtype, int tf32_mode, int threads) {
    const int ta = (transA == 'T' || transA == 't');
    const int tb = (transB == 'T' || transB == 't');
    for (int ii = 0; ii < n_rows; ++ii) if (rows[ii] < 0 || rows[ii] >= m) return 1;
    for (int jj = 0; jj < n_cols; ++jj) if (cols[jj] < 0 || cols[jj] >= n) return 1;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1) collapse(2)
#endif
    for (int jj = 0; jj < n_cols; ++jj)
        for (int ii = 0; ii < n_rows; ++ii) {
            const size_t i = (size_t)rows[ii], j = (size_t)cols[jj];
            double sum = 0.0;
            for (size_t l = 0; l < (size_t)k; ++l) {
                double a = ta ? load_elem(A, i * ldA + l, dtype, tf32_mode) : load_elem(A, i + l * ldA, dtype, tf32_mode);
                double b = tb ? load_elem(B, l * ldB + j, dtype, tf32_mode) : load_elem(B, l + j * ldB, dtype, tf32_mode);
                sum += a * b;
            }
            out[(size_t)jj * n_rows + ii] = sum;
        }
    return 0;
}

/* check_result of cute_oft_pc.cu:31-77: count of elements whose relative error exceeds the
 * threshold, and the maximum relative error (fp32 arithmetic, NaN/inf behaviour as the reference:
 * ref == 0 gives inf or NaN, NaN compares false and is not counted). */
uint64_t oft_oracle_check_result(const uint16_t* result, const uint16_t* ref, uint64_t count,
                                 float threshold, float* max_error) {
    uint64_t errors = 0; float mx = 0.0f;
    for (uint64_t i = 0; i < count; ++i) {
        float rv = h2f(ref[i]), xv = h2f(result[i]);
        float e = fabsf((rv - xv) / rv);
        if (e > mx) mx = e;
        if (e > threshold) ++errors;
    }
    *max_error = mx;
    return errors;
}
