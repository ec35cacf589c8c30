/* CPU oracle for the dense GEMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the host-side check that the reference
 * ships next to its Hopper GEMM kernels.  It is the checker the CUDA path is
 * compared with; it is never linked into, called from or used as a fallback by
 * the product library.
 *
 * Parity status: PINNED.  oracle/build.py compiles the reference's own host
 * harness (test/hardware/run_gemm_h100.cu) in place against a fake CUDA
 * driver and checks that (a) the operand bytes the harness uploads and (b) the
 * expected matrix it computes are bit-identical to what the functions below
 * produce for both of its cases (f32/TF32 K=512 and bf16 K=1024).
 *
 * Every function cites the reference lines it follows
 * (paths are relative to the reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OXREF_API __attribute__((visibility("default")))

/* test/hardware/run_gemm_h100.cu:26-30 -- round-to-nearest-even to bf16 bits
 * (the add-0x7fff-plus-lsb form; NaN payloads are not special-cased there
 * either). */
OXREF_API uint16_t oxref_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  uint32_t lsb = (u >> 16) & 1u;
  return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}

/* test/hardware/run_gemm_h100.cu:32-36 -- bf16 bits back to f32 (exact). */
OXREF_API float oxref_of_bf16(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

/* test/hardware/run_gemm_h100.cu:40-44 -- TF32 input rounding: keep sign,
 * exponent and the top 10 mantissa bits (mask 0xffffe000, i.e. truncation). */
OXREF_API float oxref_round_tf32(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  u &= 0xffffe000u;
  memcpy(&f, &u, sizeof f);
  return f;
}

/* test/hardware/run_gemm_h100.cu:129-130 -- the harness's input pattern:
 * A[i] = ((i % 7) + 1) * 0.01f over the M*K row-major elements,
 * B[i] = ((i % 5) + 1) * 0.01f over the K*N row-major elements. */
OXREF_API void oxref_pattern_a(float *a, size_t count) {
  for (size_t i = 0; i < count; i++) a[i] = (float)((i % 7) + 1) * 0.01f;
}
OXREF_API void oxref_pattern_b(float *b, size_t count) {
  for (size_t i = 0; i < count; i++) b[i] = (float)((i % 5) + 1) * 0.01f;
}

/* test/hardware/run_gemm_h100.cu:137-148 -- device operand preparation:
 * A stays row-major M x K, B[K,N] is transposed to B^T[N,K]; both converted
 * to bf16 when `narrow`, otherwise copied as f32.  `out` holds 2- or 4-byte
 * elements accordingly. */
OXREF_API void oxref_prepare_a(const float *a, void *out, int m, int k, int narrow) {
  size_t count = (size_t)m * (size_t)k;
  for (size_t i = 0; i < count; i++) {
    if (narrow) ((uint16_t *)out)[i] = oxref_to_bf16(a[i]);
    else ((float *)out)[i] = a[i];
  }
}
OXREF_API void oxref_prepare_bt(const float *b, void *out, int k, int n, int narrow) {
  for (int kk = 0; kk < k; kk++) {
    for (int nn = 0; nn < n; nn++) {
      float v = b[(size_t)kk * n + nn];
      if (narrow) ((uint16_t *)out)[(size_t)nn * k + kk] = oxref_to_bf16(v);
      else ((float *)out)[(size_t)nn * k + kk] = v;
    }
  }
}

/* Input rounding selector shared by the loops below:
 * 0 = none (plain f32 product), 1 = TF32 truncation, 2 = bf16 RNE
 * (test/hardware/run_gemm_h100.cu:156-157). */
static inline float round_in(float v, int mode) {
  if (mode == 1) return oxref_round_tf32(v);
  if (mode == 2) return oxref_of_bf16(oxref_to_bf16(v));
  return v;
}

/* test/hardware/run_gemm_h100.cu:150-162 -- the host reference GEMM exactly as
 * written there: loops i, j, k in that order, one f32 accumulator per output,
 * `acc += a * b` with both inputs rounded the way the matrix unit rounds them.
 * A is row-major [M,K]; B is row-major [K,N] (B[k*N + j]).  Compiled with
 * -ffp-contract=off so `acc += a*b` is a rounded multiply then a rounded add,
 * which is what the reference's nvcc -O2 host build produces on x86-64. */
OXREF_API void oxref_gemm_rowmajor_b(const float *a, const float *b, float *c,
                                     int m, int n, int k, int mode) {
  for (int i = 0; i < m; i++) {
    for (int j = 0; j < n; j++) {
      float acc = 0.f;
      for (int kk = 0; kk < k; kk++) {
        float av = round_in(a[(size_t)i * k + kk], mode);
        float bv = round_in(b[(size_t)kk * n + j], mode);
        acc += av * bv;
      }
      c[(size_t)i * n + j] = acc;
    }
  }
}

/* Same arithmetic (same i, j, k order, same single f32 accumulator, same
 * rounding), but reading B through the K-major layout B^T[N,K] that the device
 * kernels consume (test/hardware/run_gemm_h100.cu:142-148 builds that layout).
 * Because the per-element operation order is unchanged the result is
 * bit-identical to oxref_gemm_rowmajor_b on the transposed operand.
 *
 * `rows`/`nrows` select a subset of output rows (NULL = all M rows); row r of
 * the subset is written to c + r*ldc.  With threads > 1 the selected rows are
 * split across OpenMP threads; each output element is still produced by one
 * thread with the same sequential k loop, so threading does not change bits. */
OXREF_API void oxref_gemm_kmajor(const float *a, int64_t lda, const float *bt, int64_t ldb,
                                 float *c, int64_t ldc, int m, int n, int k, int mode,
                                 const int *rows, int nrows, int threads) {
  int count = rows ? nrows : m;
#ifdef _OPENMP
  if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
  for (int r = 0; r < count; r++) {
    int i = rows ? rows[r] : r;
    const float *arow = a + (size_t)i * lda;
    for (int j = 0; j < n; j++) {
      const float *brow = bt + (size_t)j * ldb;
      float acc = 0.f;
      for (int kk = 0; kk < k; kk++) {
        acc += round_in(arow[kk], mode) * round_in(brow[kk], mode);
      }
      c[(size_t)r * ldc + j] = acc;
    }
  }
}

/* bf16-bits operands, K-major for both (what the bf16 kernels are fed):
 * widen with of_bf16 (exact) and run the same loop.  Equivalent to
 * oxref_gemm_kmajor with mode 2 on the pre-rounded values. */
OXREF_API void oxref_gemm_kmajor_bf16(const uint16_t *a, int64_t lda, const uint16_t *bt,
                                      int64_t ldb, float *c, int64_t ldc, int m, int n, int k,
                                      const int *rows, int nrows, int threads) {
  int count = rows ? nrows : m;
#ifdef _OPENMP
  if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
  for (int r = 0; r < count; r++) {
    int i = rows ? rows[r] : r;
    const uint16_t *arow = a + (size_t)i * lda;
    for (int j = 0; j < n; j++) {
      const uint16_t *brow = bt + (size_t)j * ldb;
      float acc = 0.f;
      for (int kk = 0; kk < k; kk++) {
        acc += oxref_of_bf16(arow[kk]) * oxref_of_bf16(brow[kk]);
      }
      c[(size_t)r * ldc + j] = acc;
    }
  }
}

/* test/hardware/run_gemm_h100.cu:191-197 -- the reference's acceptance test:
 * every element within an absolute tolerance (5e-2 for f32/TF32 inputs,
 * 2e-1 for bf16).  Returns the index of the first mismatch or -1, and the
 * largest absolute difference through *max_abs. */
OXREF_API int64_t oxref_compare_abs(const float *got, const float *expect, size_t count,
                                    float tol, float *max_abs) {
  int64_t first = -1;
  float worst = 0.f;
  for (size_t i = 0; i < count; i++) {
    float d = fabsf(got[i] - expect[i]);
    if (worst == worst && (d > worst || d != d)) worst = d; /* a NaN sticks */
    if (first < 0 && !(d <= tol)) first = (int64_t)i;
  }
  if (max_abs) *max_abs = worst;
  return first;
}

/* The tolerance this build is graded against for same-rounded inputs:
 * 1e-5 * sqrt(K) * max|A| * max|B|. */
OXREF_API float oxref_tolerance(int k, float max_a, float max_b) {
  return 1e-5f * sqrtf((float)k) * max_a * max_b;
}

OXREF_API int oxref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
