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
__global__ void __launch_bounds__(kSimtThreads, 2)
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

// Same re-layout with 16-byte global accesses on both sides, for 16-byte-aligned
// pointers, rows % 64 == 0 and cols % kTransposeCols<T> == 0: tiles of 64 rows x
// 256 bytes (64 f32 or 128 bf16 columns, so every thread has four 16-byte loads
// in flight), transposed through shared memory.  HBM-bound:
// 2 * rows * cols * sizeof(T) bytes.
template <typename T>
constexpr int kTransposeCols = 256 / (int)sizeof(T);

template <typename T>
__global__ void __launch_bounds__(256) transpose64_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                                          int rows, int cols) {
  constexpr int V = 16 / (int)sizeof(T);       // elements per 16-byte access
  constexpr int TC = kTransposeCols<T>;        // tile columns
  constexpr int VPR = TC / V;                  // 16-byte accesses per source tile row (16)
  constexpr int VPO = 64 / V;                  // 16-byte accesses per transposed tile row
  constexpr int PITCH = TC + (sizeof(T) == 4 ? 1 : 2);
  __shared__ T tile[64 * PITCH];
  const int x0 = blockIdx.x * TC, y0 = blockIdx.y * 64;
  for (int v = threadIdx.x; v < 64 * VPR; v += 256) {
    const int r = v / VPR, cv = v % VPR;
    const uint4 q = *reinterpret_cast<const uint4 *>(src + (int64_t)(y0 + r) * cols + x0 + cv * V);
    const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
    for (int i = 0; i < V; i++) tile[r * PITCH + cv * V + i] = e[i];
  }
  __syncthreads();
  for (int v = threadIdx.x; v < TC * VPO; v += 256) {
    const int r = v / VPO, cv = v % VPO;       // row r of the transposed tile = column r of the source tile
    uint4 q;
    T *e = reinterpret_cast<T *>(&q);
#pragma unroll
    for (int i = 0; i < V; i++) e[i] = tile[(cv * V + i) * PITCH + r];
    *reinterpret_cast<uint4 *>(dst + (int64_t)(x0 + r) * rows + y0 + cv * V) = q;
  }
}

// The 2-byte case of the above with half the shared-memory instructions: the
// tile is kept as 32-bit pairs of neighbouring columns, and a thread of the
// store phase reads eight pairs (eight source rows, two source columns) and
// writes 16 bytes of each of the two transposed rows.
__global__ void __launch_bounds__(256) transpose64_pairs_kernel(const uint16_t *__restrict__ src,
                                                                uint16_t *__restrict__ dst, int rows, int cols) {
  constexpr int PITCH = 65;                     // 64 pairs per tile row + 1
  __shared__ uint32_t tile[64 * PITCH];
  const int x0 = blockIdx.x * 128, y0 = blockIdx.y * 64;
  for (int v = threadIdx.x; v < 64 * 16; v += 256) {
    const int r = v >> 4, cv = v & 15;
    const uint4 q = *reinterpret_cast<const uint4 *>(src + (int64_t)(y0 + r) * cols + x0 + cv * 8);
    uint32_t *t = tile + r * PITCH + cv * 4;
    t[0] = q.x, t[1] = q.y, t[2] = q.z, t[3] = q.w;
  }
  __syncthreads();
  for (int v = threadIdx.x; v < 64 * 8; v += 256) {
    const int pair = v >> 3, cv = v & 7;        // source columns 2*pair, 2*pair+1; source rows 8*cv .. 8*cv+7
    uint32_t w[8];
#pragma unroll
    for (int e = 0; e < 8; e++) w[e] = tile[(cv * 8 + e) * PITCH + pair];
    uint4 even, odd;                            // transposed rows 2*pair and 2*pair+1
    even.x = __byte_perm(w[0], w[1], 0x5410), odd.x = __byte_perm(w[0], w[1], 0x7632);
    even.y = __byte_perm(w[2], w[3], 0x5410), odd.y = __byte_perm(w[2], w[3], 0x7632);
    even.z = __byte_perm(w[4], w[5], 0x5410), odd.z = __byte_perm(w[4], w[5], 0x7632);
    even.w = __byte_perm(w[6], w[7], 0x5410), odd.w = __byte_perm(w[6], w[7], 0x7632);
    uint16_t *o = dst + (int64_t)(x0 + 2 * pair) * rows + y0 + cv * 8;
    *reinterpret_cast<uint4 *>(o) = even;
    *reinterpret_cast<uint4 *>(o + rows) = odd;
  }
}

// ---- f32 -> bf16 bits, round to nearest even (run_gemm_h100.cu:26-30) ------------
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  uint32_t lsb = (u >> 16) & 1u;
  return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}

// B[K,N] f32 -> B^T[N,K] bf16 in one pass (the two steps a caller with a
// row-major f32 B needs before the bf16 GEMM, bench/bench.py:255-271): the
// rounding of f32_to_bf16_bits, the tiling of transpose64_kernel.  HBM-bound:
// 6 bytes per element instead of 6 + 4 for the two kernels in a row.
__global__ void __launch_bounds__(256) transpose64_f32_to_bf16_kernel(const float *__restrict__ src,
                                                                      uint16_t *__restrict__ dst, int rows,
                                                                      int cols) {
  constexpr int PITCH = 66;
  __shared__ uint16_t tile[64 * PITCH];
  const int x0 = blockIdx.x * 64, y0 = blockIdx.y * 64;
  for (int v = threadIdx.x; v < 64 * 16; v += 256) {  // 16 four-element loads per tile row
    const int r = v >> 4, cv = v & 15;
    const float4 q = *reinterpret_cast<const float4 *>(src + (int64_t)(y0 + r) * cols + x0 + cv * 4);
    uint16_t *t = tile + r * PITCH + cv * 4;
    t[0] = f32_to_bf16_bits(q.x);
    t[1] = f32_to_bf16_bits(q.y);
    t[2] = f32_to_bf16_bits(q.z);
    t[3] = f32_to_bf16_bits(q.w);
  }
  __syncthreads();
  for (int v = threadIdx.x; v < 64 * 8; v += 256) {   // 8 eight-element stores per transposed row
    const int r = v >> 3, cv = v & 7;
    uint4 q;
    uint16_t *e = reinterpret_cast<uint16_t *>(&q);
#pragma unroll
    for (int i = 0; i < 8; i++) e[i] = tile[(cv * 8 + i) * PITCH + r];
    *reinterpret_cast<uint4 *>(dst + (int64_t)(x0 + r) * rows + y0 + cv * 8) = q;
  }
}

// Eight elements per thread and step (two 16-byte loads, one 16-byte store) when
// both pointers are 16-byte aligned, element by element otherwise and for the
// tail.  HBM-bound: 6 bytes per element.
__global__ void f32_to_bf16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst,
                                   size_t count, int vector_ok) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t groups = vector_ok ? count / 8 : 0;
  for (size_t g = tid; g < groups; g += stride) {
    const float4 lo = reinterpret_cast<const float4 *>(src)[2 * g];
    const float4 hi = reinterpret_cast<const float4 *>(src)[2 * g + 1];
    uint4 out;
    out.x = (uint32_t)f32_to_bf16_bits(lo.x) | ((uint32_t)f32_to_bf16_bits(lo.y) << 16);
    out.y = (uint32_t)f32_to_bf16_bits(lo.z) | ((uint32_t)f32_to_bf16_bits(lo.w) << 16);
    out.z = (uint32_t)f32_to_bf16_bits(hi.x) | ((uint32_t)f32_to_bf16_bits(hi.y) << 16);
    out.w = (uint32_t)f32_to_bf16_bits(hi.z) | ((uint32_t)f32_to_bf16_bits(hi.w) << 16);
    reinterpret_cast<uint4 *>(dst)[g] = out;
  }
  for (size_t i = groups * 8 + tid; i < count; i += stride) dst[i] = f32_to_bf16_bits(src[i]);
}

// ---- f32 operands split into TF32 pieces ------------------------------------------
// x = hi + lo with hi = x truncated to TF32 (what the matrix unit would keep,
// run_gemm_h100.cu:40-44) and lo = x - hi (exact in f32; the unit truncates it
// again).  Row r of dst holds three K-long pieces: [hi | lo | hi] (order 0, for A)
// or [lo | hi | hi] (order 1, for B^T), so that one TF32 GEMM over 3K computes
// hi*lo + lo*hi + hi*hi -- the f32 product up to a 2^-20 relative term -- with f32
// accumulation.  The small cross terms come first: the matrix unit's adder drops
// bits relative to the running sum, so they are summed while it is still small.
// k % 4 == 0, 16-byte aligned rows.
__global__ void split_tf32_kernel(const float *__restrict__ src, float *__restrict__ dst, int rows, int k,
                                  int64_t ld_src, int order) {
  const int k4 = k >> 2;
  const size_t total = (size_t)rows * k4;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int r = (int)(i / k4), q = (int)(i - (size_t)r * k4);
    const float4 x = *reinterpret_cast<const float4 *>(src + (int64_t)r * ld_src + 4 * q);
    float4 hi, lo;
    hi.x = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u);
    hi.y = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u);
    hi.z = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u);
    hi.w = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u);
    lo.x = __fsub_rn(x.x, hi.x);
    lo.y = __fsub_rn(x.y, hi.y);
    lo.z = __fsub_rn(x.z, hi.z);
    lo.w = __fsub_rn(x.w, hi.w);
    float *row = dst + (size_t)r * 3 * k + 4 * q;
    *reinterpret_cast<float4 *>(row) = order == 0 ? hi : lo;
    *reinterpret_cast<float4 *>(row + k) = order == 0 ? lo : hi;
    *reinterpret_cast<float4 *>(row + 2 * k) = hi;
  }
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

// DIST 0 = uniform [-1,1), 1 = normal(0, scale).  OUT16: store bf16 bits.  Each
// thread produces four consecutive elements per step and stores them as one 16-
// or 8-byte vector when `dst` is 16-byte aligned (vector_ok).
template <int DIST, bool OUT16>
__global__ void synth_fill_kernel(void *dst, size_t count, uint32_t seed, float scale,
                                  uint64_t index_offset, int vector_ok) {
  auto value = [&](size_t i) {
    return DIST == 0 ? synth_uniform_pm1(seed, index_offset + i) : synth_normal(seed, index_offset + i) * scale;
  };
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t groups = vector_ok ? count / 4 : 0;
  for (size_t g = tid; g < groups; g += stride) {
    const float v0 = value(4 * g), v1 = value(4 * g + 1), v2 = value(4 * g + 2), v3 = value(4 * g + 3);
    if constexpr (OUT16) {
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(v0) | ((uint32_t)f32_to_bf16_bits(v1) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(v2) | ((uint32_t)f32_to_bf16_bits(v3) << 16);
      reinterpret_cast<uint2 *>(dst)[g] = o;
    } else {
      reinterpret_cast<float4 *>(dst)[g] = make_float4(v0, v1, v2, v3);
    }
  }
  for (size_t i = groups * 4 + tid; i < count; i += stride) {
    const float v = value(i);
    if constexpr (OUT16) reinterpret_cast<uint16_t *>(dst)[i] = f32_to_bf16_bits(v);
    else reinterpret_cast<float *>(dst)[i] = v;
  }
}

}  // namespace oxgpu
