// Kernels around the tcgen05 GEMM: the exact-f32 GEMM, operand re-layout and
// conversion, the split-K reduction and the synthetic-operand generators.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace oxgpu {

// ---- exact f32 GEMM -----------------------------------------------------------
// C[i,j] = sum_k round(A[i,k]) * round(B^T[j,k]) with one f32 accumulator per
// output, k ascending, a rounded multiply followed by a rounded add -- the
// arithmetic of the reference's host loop (test/hardware/run_gemm_h100.cu:
// 150-162), so results are bit-identical to that loop, not merely close.
// IN_MODE: 0 = f32 as is, 1 = f32 truncated to TF32 (mask 0xffffe000,
// run_gemm_h100.cu:40-44), 2 = bf16 bits widened exactly (32-36).
constexpr int kSimtTile = 128;  // C tile edge
constexpr int kSimtBK = 16;     // K slice staged per step
constexpr int kSimtThreads = 256;

template <int IN_MODE>
__device__ __forceinline__ float simt_load(const void *base, int64_t index) {
  if constexpr (IN_MODE == 2) {
    uint32_t bits = ((uint32_t) reinterpret_cast<const uint16_t *>(base)[index]) << 16;
    return __uint_as_float(bits);
  } else {
    float v = reinterpret_cast<const float *>(base)[index];
    if constexpr (IN_MODE == 1) v = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    return v;
  }
}

template <int IN_MODE>
__global__ void __launch_bounds__(kSimtThreads)
simt_gemm_exact_kernel(const void *__restrict__ a, const void *__restrict__ bt, float *__restrict__ c,
                       int m, int n, int k, int64_t lda, int64_t ldb, int64_t ldc) {
  // K-slices stored k-major ([kk][row]) so the inner product reads are
  // conflict-free broadcasts/vectors.
  __shared__ float sa[kSimtBK][kSimtTile + 4];
  __shared__ float sb[kSimtBK][kSimtTile + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 8 x 8 outputs each
  const int row0 = blockIdx.y * kSimtTile, col0 = blockIdx.x * kSimtTile;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < k; k0 += kSimtBK) {
    // 128 rows x 16 k per operand = 2048 elements, 8 per thread
#pragma unroll
    for (int e = 0; e < 8; e++) {
      int idx = tid + e * kSimtThreads;
      int r = idx >> 4, kk = idx & 15;
      int gk = k0 + kk;
      float av = 0.f, bv = 0.f;
      if (gk < k) {
        if (row0 + r < m) av = simt_load<IN_MODE>(a, (int64_t)(row0 + r) * lda + gk);
        if (col0 + r < n) bv = simt_load<IN_MODE>(bt, (int64_t)(col0 + r) * ldb + gk);
      }
      sa[kk][r] = av;
      sb[kk][r] = bv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtBK; kk++) {
      float ar[8], br[8];
#pragma unroll
      for (int i = 0; i < 8; i++) ar[i] = sa[kk][ty * 8 + i];
#pragma unroll
      for (int j = 0; j < 8; j++) br[j] = sb[kk][tx * 8 + j];
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
          acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(ar[i], br[j]));  // never fused
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int r = row0 + ty * 8 + i;
    if (r >= m) continue;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      int cc = col0 + tx * 8 + j;
      if (cc < n) c[(int64_t)r * ldc + cc] = acc[i][j];
    }
  }
}

// ---- B[K,N] -> B^T[N,K] ----------------------------------------------------------
template <typename T>
__global__ void transpose_kernel(const T *__restrict__ src, T *__restrict__ dst, int rows, int cols) {
  __shared__ T tile[32][33];
  int x = blockIdx.x * 32 + threadIdx.x;
  int y0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int y = y0 + j;
    if (x < cols && y < rows) tile[j][threadIdx.x] = src[(int64_t)y * cols + x];
  }
  __syncthreads();
  int tx = blockIdx.y * 32 + threadIdx.x;  // column of dst = row of src
  int ty0 = blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int ty = ty0 + j;  // row of dst = column of src
    if (tx < rows && ty < cols) dst[(int64_t)ty * rows + tx] = tile[threadIdx.x][j];
  }
}

// ---- f32 -> bf16 bits, round to nearest even (run_gemm_h100.cu:26-30) ------------
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  uint32_t lsb = (u >> 16) & 1u;
  return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}

__global__ void f32_to_bf16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst,
                                   size_t count) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) dst[i] = f32_to_bf16_bits(src[i]);
}

// ---- split-K reduction ----------------------------------------------------------
// C[r, :] = sum over slices s (ascending, so the result is deterministic) of
// workspace[s * slice_rows + r, :].  n4 = N / 4 (rows are float4 aligned).
__global__ void splitk_reduce_kernel(const float4 *__restrict__ ws, float *__restrict__ c, int m,
                                     int n, int64_t ldc, int splits, int64_t slice_rows) {
  const int n4 = n >> 2;
  size_t total = (size_t)m * n4;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int r = (int)(i / n4), q = (int)(i - (size_t)r * n4);
    float4 acc = ws[(size_t)r * n4 + q];
    for (int s = 1; s < splits; s++) {
      float4 v = ws[((size_t)s * slice_rows + r) * n4 + q];
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(c + (int64_t)r * ldc + 4 * q) = acc;
  }
}

// ---- synthetic operands -----------------------------------------------------------
// Counter-based: value = f(seed, stream, 64-bit index).  The integer hash and
// the uniform mapping are bit-identical to the host generator in synth.py.
__host__ __device__ __forceinline__ uint32_t synth_hash(uint32_t seed, uint32_t stream, uint64_t index) {
  uint32_t lo = (uint32_t)index, hi = (uint32_t)(index >> 32);
  uint32_t s = seed * 0x9E3779B9u + stream * 0x7F4A7C15u + 0x632BE5ABu;
  uint32_t x = lo ^ s ^ (hi * 0x85EBCA6Bu);
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ float synth_uniform_pm1(uint32_t seed, uint64_t index) {
  uint32_t h = synth_hash(seed, 0, index);
  return __fadd_rn(__fmul_rn((float)(h >> 8), 1.1920928955078125e-07f /* 2^-23 */), -1.0f);
}

__device__ __forceinline__ float synth_normal(uint32_t seed, uint64_t index) {
  uint32_t h1 = synth_hash(seed, 1, index), h2 = synth_hash(seed, 2, index);
  float u1 = ((float)(h1 >> 8) + 1.0f) * 5.9604644775390625e-08f;  // (0, 1]
  float u2 = (float)(h2 >> 8) * 5.9604644775390625e-08f;           // [0, 1)
  return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

// DIST 0 = uniform [-1,1), 1 = normal(0, scale).  OUT16: store bf16 bits.
template <int DIST, bool OUT16>
__global__ void synth_fill_kernel(void *dst, size_t count, uint32_t seed, float scale,
                                  uint64_t index_offset) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) {
    float v = DIST == 0 ? synth_uniform_pm1(seed, index_offset + i)
                        : synth_normal(seed, index_offset + i) * scale;
    if constexpr (OUT16) reinterpret_cast<uint16_t *>(dst)[i] = f32_to_bf16_bits(v);
    else reinterpret_cast<float *>(dst)[i] = v;
  }
}

}  // namespace oxgpu
