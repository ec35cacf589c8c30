// Declarations shared by the host-only catalog and the CUDA launch layer.
#pragma once

#include <cstdint>
#include <string>

#include "../../include/oxgpu_b200.h"

#define OXGPU_STRINGIFY_(x) #x
#define OXGPU_STRINGIFY(x) OXGPU_STRINGIFY_(x)

#if defined(__CUDACC__)
#define OXGPU_HD __host__ __device__
#else
#define OXGPU_HD
#endif

namespace oxgpu {

// B200 kernel variants (values match OXGPU_VARIANT_* in the public header).
enum Variant {
  VARIANT_AUTO = 0,
  VARIANT_1CTA_128x256 = 1,
  VARIANT_1CTA_128x128 = 2,
  VARIANT_1CTA_256x128 = 3,
  VARIANT_2CTA_256x256 = 4,
  VARIANT_2CTA_256x128 = 5,
  VARIANT_SPLITK = 6,
  VARIANT_2CTA_512x256 = 7,
  VARIANT_1CTA_256x256 = 8,
  VARIANT_CLUSTER_SPLITK_128x256 = 9,   // K slices across a cluster, reduced through DSMEM
  VARIANT_CLUSTER_SPLITK_128x128 = 10,
  VARIANT_2CTA_256x512 = 11,            // two 256-column blocks per pair tile; each CTA stages 256 contiguous B^T rows
};

// Every tcgen05 GEMM kernel here runs 10 warps: TMA producer, MMA issuer (also
// owns the TMEM allocation), and eight epilogue warps (two per TMEM lane
// quadrant).
constexpr int kThreadsPerCta = 320;
// Largest dynamic shared window a CTA may opt into on sm_100 (227 KiB).
constexpr int kMaxDynamicSmem = 232448;
// Per-warp epilogue staging: one 32x32 f32 sub-tile (4 KiB) x 8 warps.
constexpr int kEpilogueStagingBytes = 8 * 4096;
// Barriers + TMEM base slot, padded.
constexpr int kBarrierRegionBytes = 1024;
// Stage bases must be 1024-byte aligned for the 128-byte swizzle atoms; the
// dynamic window itself is only guaranteed 16-byte alignment, so the kernel
// rounds its base up and the host requests this much slack.
constexpr int kSmemAlignSlack = 1024;
constexpr int kMaxStages = 8;
// A CTA that asks for more than half of an SM's shared memory never shares the
// SM, which the kernels rely on for their TMEM allocation (up to all 512
// columns per CTA).  Every launch requests at least this much.
constexpr int kMinSmemRequest = 118784;

struct VariantShape {
  int cta_group;   // 1 or 2
  int tile_m;      // rows of C per scheduled tile (per CTA pair when cta_group == 2)
  int tile_n;      // columns of C per scheduled tile
  int cta_a_rows;  // rows of A one CTA stages per K block
  int cta_b_rows;  // rows of B^T one CTA stages per K block
};

inline VariantShape variant_shape(int variant) {
  switch (variant) {
    case VARIANT_1CTA_128x256: return {1, 128, 256, 128, 256};
    case VARIANT_1CTA_128x128: return {1, 128, 128, 128, 128};
    case VARIANT_1CTA_256x128: return {1, 256, 128, 256, 128};
    case VARIANT_2CTA_256x256: return {2, 256, 256, 128, 128};
    case VARIANT_2CTA_256x128: return {2, 256, 128, 128, 64};
    case VARIANT_2CTA_512x256: return {2, 512, 256, 256, 128};
    case VARIANT_1CTA_256x256: return {1, 256, 256, 256, 256};
    case VARIANT_2CTA_256x512: return {2, 256, 512, 128, 256};
    default: return {0, 0, 0, 0, 0};
  }
}

// One K block is one 128-byte swizzle row: 64 bf16 or 32 f32 elements.
inline int variant_stage_bytes(int variant) {
  VariantShape s = variant_shape(variant);
  return (s.cta_a_rows + s.cta_b_rows) * 128;
}

inline int variant_max_stages(int variant) {
  int avail = kMaxDynamicSmem - kEpilogueStagingBytes - kBarrierRegionBytes - kSmemAlignSlack;
  int s = avail / variant_stage_bytes(variant);
  return s > kMaxStages ? kMaxStages : s;
}

// Dynamic shared bytes a launch of `variant` with `stages` ring slots requests
// (stages <= 0 or too deep: the deepest ring that fits).
inline int variant_smem_bytes(int variant, int stages) {
  int most = variant_max_stages(variant);
  if (stages <= 0 || stages > most) stages = most;
  int bytes = stages * variant_stage_bytes(variant) + kEpilogueStagingBytes + kBarrierRegionBytes +
              kSmemAlignSlack;
  return bytes < kMinSmemRequest ? kMinSmemRequest : bytes;
}

struct CatalogEntry {
  const char *name;
  oxgpu_tile_config tile;
  int element_bytes;  // 4 = f32 inputs (TF32 math), 2 = bf16
  int variant;
};

const CatalogEntry *find_entry(const char *name);

int fail(int status, const std::string &message);

// Grouped CTA order (tools/exporter/export_prims_index.ml:52-58): walk `group`
// tile-rows before advancing along N, so the tiles in flight share a few row
// blocks of A and a few column blocks of B.
OXGPU_HD inline void grouped_tile(int pid, int group, int tiles_m, int tiles_n, int *tile_m,
                                  int *tile_n) {
  int per_group = group * tiles_n;
  int first = (pid / per_group) * group;
  int rows = tiles_m - first < group ? tiles_m - first : group;
  *tile_m = first + pid % rows;
  *tile_n = (pid % per_group) / rows;
}

// Division by a number that is fixed for a whole launch, for the kernels' tile
// arithmetic: an integer division costs one thread about 200 clocks, and the
// producer lane does several in a row before its first load.  magic =
// floor(2^40 / d) + 1 gives floor(a / d) = (a * magic) >> 40 exactly whenever
// a * d < 2^40 (the excess over a / d is below 1 / d); make_fast_divisor returns
// magic = 0, meaning "divide", when the largest dividend does not allow that.
struct FastDivisor {
  unsigned long long magic;
  int d;
  int pad;
};
OXGPU_HD inline FastDivisor make_fast_divisor(int d, long long max_dividend) {
  FastDivisor f{0ull, d, 0};
  if (d > 0 && max_dividend >= 0 && max_dividend < (1ll << 22) && (long long)d < (1ll << 18))
    f.magic = (1ull << 40) / (unsigned long long)d + 1ull;
  return f;
}
OXGPU_HD inline int fast_div(int a, const FastDivisor &f) {
  return f.magic ? (int)(((unsigned long long)(unsigned)a * f.magic) >> 40) : a / f.d;
}

// grouped_tile with the launch's divisors prepared (per_group = group * tiles_n),
// plus the index of the group of tile rows the tile lies in.  Same results as
// grouped_tile for every pid in [0, tiles_m * tiles_n).
OXGPU_HD inline void grouped_tile_fast(int pid, const FastDivisor &per_group, const FastDivisor &group, int tiles_m,
                                       int *tile_m, int *tile_n, int *group_index) {
  const int q = fast_div(pid, per_group);
  const int r = pid - q * per_group.d;
  const int first = q * group.d;
  *group_index = q;
  if (tiles_m - first >= group.d) {  // a full group: pid % rows == r % group
    const int col = fast_div(r, group);
    *tile_n = col;
    *tile_m = first + (r - col * group.d);
  } else {  // the last, shorter group of tile rows
    const int rows = tiles_m - first;
    *tile_m = first + pid % rows;
    *tile_n = r / rows;
  }
}

}  // namespace oxgpu
