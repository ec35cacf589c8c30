// The dense GEMM hot path on sm_100a: C[M,N] f32 = A[M,K] * B^T[N,K]^T with
// bf16 or TF32 inputs.
//
// What it replaces: the reference's Hopper schedule hopper_gemm /
// hopper_gemm_bf16 (examples/kernels/gemm.ml:47-163, gemm_bf16.ml:33-128),
// i.e. a TMA producer filling a ring of 128-byte-swizzled K-major stages
// guarded by full/empty mbarriers, warpgroup WGMMA consumers, grouped CTA
// order and a vector-store epilogue.  WGMMA does not exist on Blackwell, so
// the schedule is rebuilt around tcgen05:
//
//   warp 0      TMA producer      one lane issues cp.async.bulk.tensor loads
//   warp 1      UMMA issuer       one lane issues tcgen05.mma; the warp owns the
//                                 TMEM allocation
//   warps 2-9   epilogue          tcgen05.ld TMEM -> registers -> swizzled
//                                 shared staging -> TMA store to C (two groups
//                                 of four warps, one warp per TMEM lane quadrant)
//
// The kernel is persistent: each CTA (or CTA pair) walks tiles
// first, first+stride, ... in the grouped order, or, on problems of many tiles,
// takes the next tile of that order from a queue (TileFeed).  Where the tile's accumulator
// takes at most half of TMEM, two accumulator sets alternate so the epilogue of
// tile i overlaps the main loop of tile i+1; the largest tile (256 rows x 256
// columns per CTA) fills TMEM and trades that overlap for a quarter less
// operand traffic per flop.  In the CTA-pair variants (cta_group::2) each CTA
// stages its own rows of A and its own half of the B^T rows, the leader CTA
// issues UMMAs that read both CTAs' shared memory, and no load is multicast.
//
// Every mbarrier wait is bounded: when a wait outlives its budget the waiter
// records where it gave up in the device status block, raises the CTA's abort
// flag and all roles leave through the common teardown (pending loads/stores
// drained, TMEM released).  The reference's waits spin forever
// (lib/backend/ptx.ml:174-181).  The hardware barriers (CTA, named, cluster)
// are placed where every thread they count reaches them whatever its waits
// returned, and `griddepcontrol.wait` ends when the kernel before this one in
// the stream does.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "common.hpp"
#include "ptx.cuh"

namespace oxgpu {

// Device status block: words[0] = code (0 = healthy), [1] = blockIdx.x,
// [2] = role-specific detail (stage / tile), [3] = parity, [4] = barrier kind.
__device__ uint32_t g_device_status[8];

// Tile queues of the dynamic schedule: slot s holds {next tile to hand out,
// clusters that have finished}.  A launch that uses the dynamic schedule is
// given a slot by the host (round robin); the last cluster to finish puts both
// words back to zero, so a slot is clean again when its launch has completed.
constexpr int kSchedSlots = 1024;
__device__ unsigned int g_tile_queue[2 * kSchedSlots];

enum WaitKind : uint32_t {
  WAIT_EMPTY = 1,       // producer waiting for a free ring slot
  WAIT_FULL = 2,        // issuer waiting for operand bytes
  WAIT_TMEM_EMPTY = 3,  // issuer waiting for the epilogue to drain an accumulator
  WAIT_TMEM_FULL = 4,   // epilogue waiting for an accumulator
  WAIT_DRAIN = 5,       // teardown waiting for in-flight work
  WAIT_SELFTEST = 6,    // the bounded-wait self test
  WAIT_TILE = 7,        // a role waiting for the producer to announce the next tile
};

struct GemmParams {
  // Tensor maps passed by value (buffer entry points).  a_map_ptr / b_map_ptr,
  // when non-null, point at caller-owned maps in device memory instead (the
  // catalog entry points take device pointers to maps, lib/backend/ptx.ml:6-18).
  CUtensorMap map_a, map_b, map_c;
  const void *a_map_ptr, *b_map_ptr;
  int tiles_m, tiles_n, num_k_blocks;
  int stages;
  int group_m;
  int a_box_rows, b_box_rows;  // rows one TMA load brings (the caller's box)
  int k_block_elems;           // elements per 128-byte K block (64 bf16 / 32 f32)
  // Split-K: each tile is cut into `splits` K slices of `kb_per_split` blocks;
  // slice s stores its partial tile `split_row_stride` rows further down the C
  // map (a [splits * rows, N] workspace).  splits == 1: plain GEMM.
  int splits, kb_per_split, split_row_stride;
  // Tiles with two row blocks per CTA: how many K blocks at either end of a tile
  // are issued block-major (see the issuer); 0 = always interleaved.
  int reorder_kb;
  // L2 eviction priority of the A loads, the B^T loads and the C stores:
  // 0 = normal, 1 = evict first, 2 = evict last.
  int hint_a, hint_b, hint_c;
  // Split-K inside a thread-block cluster (one-CTA 128-row tiles only): the
  // `splits` CTAs of a cluster take the K slices of one tile, leave their
  // partial tiles in their own shared memory, and each CTA then sums one column
  // range of the tile across the cluster through distributed shared memory and
  // writes it to C.  No workspace, no second kernel, fixed summation order.
  // (cluster_reduce == 1.)  With two slices there is a shorter way, cluster_reduce
  // == 2: the tile of C is zeroed while the main loop runs, and each CTA then adds
  // its partial tile to it with TMA reductions (the L2 does the additions; with two
  // addends the order cannot change the sum).  The epilogue is then the ordinary
  // one -- no parking, no cross-CTA reads, no cluster barrier on the way out.
  int cluster_reduce;
  float *c_ptr;
  long long c_ld;
  int c_rows, c_cols;
  unsigned long long wait_budget_ns;
  // Affine epilogue (AFFINE kernels only): C = alpha * (A B) + beta * C_in + bias,
  // bias[N] broadcast over rows (null: none); C_in is read only when beta != 0 and
  // may be C itself.
  float alpha, beta;
  const float *bias;
  const float *c_in;
  long long c_in_ld;
  // Tile schedule.  0: static -- cluster c takes tiles c, c + clusters, ...  s + 1:
  // dynamic -- after its first tile a cluster takes the next tile nobody has
  // started from queue slot s of g_tile_queue (see TileFeed).
  int sched_slot_plus1;
  // splits, group_m * tiles_n and group_m with their reciprocals (see FastDivisor)
  FastDivisor div_splits, div_per_group, div_group;
};

// Parameters of the fan-out kernels: the epilogue writes every staged 32x32
// sub-tile of C to `n_dests` destinations instead of one.  A destination is a
// row-major f32 matrix with this GEMM's rows and a column window of its own;
// it may live in this GPU's memory or in a peer's (mapped into this process),
// which turns "GEMM, then all-gather of the column shards" into one kernel: a
// rank's tiles leave over NVLink as they are produced, already interleaved
// into the replicated row-major C.  The stores are ordinary (non-multicast)
// TMA tile stores; map_c of the base struct is unused.
constexpr int kMaxFanout = 8;
struct GemmParamsFanout : GemmParams {
  CUtensorMap dest_maps[kMaxFanout];
  int n_dests;
};

// Tile t of the walk -> (tile row, tile column): the reference's grouped order
// (common.hpp grouped_tile), with the columns of every other group of tile rows
// walked in reverse.  At the turn from one group to the next the B^T panels that
// were used last are used first, while they are still in L2 (16384 x 16384 x
// 8192 with a cold L2: 3.13 -> 2.97 ms; no effect at 8192^3, where a group is
// a third of the problem).  Which SM computes a tile does not change its value.
__device__ __forceinline__ void tile_coords(const GemmParams &p, int t, int *tm, int *tn) {
  int group_index;
  grouped_tile_fast(t, p.div_per_group, p.div_group, p.tiles_m, tm, tn, &group_index);
  if (group_index & 1) *tn = p.tiles_n - 1 - *tn;
}
// work item -> (tile, K slice)
__device__ __forceinline__ void split_work(const GemmParams &p, int w, int *t, int *sp) {
  *t = fast_div(w, p.div_splits);
  *sp = w - *t * p.splits;
}

struct WaitCtx {
  unsigned long long budget_ns;
  volatile uint32_t *abort_flag;  // shared memory, one per CTA
};

constexpr int kTileRing = 8;  // announced-tile slots per CTA

// Bounded mbarrier wait.  Returns false if the budget ran out (or another
// role of this CTA already gave up).  The waiter is parked by the hardware
// (try_wait with a suspend-time hint) and resumed when the phase completes, so
// a wait that lasts a whole main loop costs a few instructions per park, not a
// polling loop; the abort flag and the budget are looked at between parks.
constexpr uint32_t kParkNs = 4000;
template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const WaitCtx &ctx,
                                             uint32_t kind, uint32_t detail) {
  if constexpr (!CLUSTER_ACQUIRE) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = ptx::globaltimer_ns();
  while (true) {
    if constexpr (CLUSTER_ACQUIRE) {
      if (ptx::mbar_try_wait_parked_cluster(bar, parity, kParkNs)) return true;
    } else {
      if (ptx::mbar_try_wait_parked(bar, parity, kParkNs)) return true;
    }
    if (*ctx.abort_flag) return false;
    if (ptx::globaltimer_ns() - t0 > ctx.budget_ns) {
      if (atomicCAS(&g_device_status[0], 0u, kind) == 0u) {
        g_device_status[1] = blockIdx.x;
        g_device_status[2] = detail;
        g_device_status[3] = parity;
        g_device_status[4] = kind;
        __threadfence();
      }
      *ctx.abort_flag = 1;
      return false;
    }
  }
}

// Which tile a role works on next.  Static schedule: cluster c walks c, c + C,
// c + 2C, ... (C clusters).  Dynamic schedule: the producer of the leader CTA
// takes tile indices from a global queue (its own first tile is c, so the queue
// starts at C) and announces them, one tile ahead, in a ring of kTileRing slots
// in the shared memory of every CTA of the cluster; the other roles read the
// ring.  Tiles are then handed out in walk order to whichever cluster is free,
// so the tiles in flight stay a compact window of the walk however long the
// launch runs: clusters that share an operand panel stay at nearly the same K
// offset and the panel is fetched from HBM once.  With the static walk the
// clusters drift apart over tens of waves (measured at 16384 x 32768 x 8192:
// 9.9 GB of DRAM reads against 6.9 GB for the vendor library's kernel of the
// same tile shape, and a lower SM clock under the power cap as a result).
// No announced slot is reused before every reader is done with it: the
// producer runs at most the ring depth of the operand ring plus one accumulator
// ahead of the slowest role, far fewer than kTileRing tiles.
template <bool PAIR>
struct TileFeed {
  bool dynamic;
  int first, stride, total;
  uint32_t ring_bar, ring_tile;  // shared-memory addresses in this CTA
  int local = 0;

  // next tile for a reading role; returns total (or more) when there is none, -1 if the wait gave up
  __device__ __forceinline__ int take(const WaitCtx &ctx) {
    int w;
    if (!dynamic) {
      w = first + local * stride;
    } else {
      const uint32_t slot = (uint32_t)local & (kTileRing - 1);
      if (!bounded_wait<PAIR>(ring_bar + 8u * slot, ((uint32_t)local / kTileRing) & 1u, ctx, WAIT_TILE,
                              (uint32_t)local))
        return -1;
      w = (int)ptx::ld_shared_u32(ring_tile + 4u * slot);
    }
    local++;
    return w;
  }
  // the announcing side (leader CTA's producer lane): publish tile `w` as tile number `n` of this cluster
  __device__ __forceinline__ void announce(int n, int w) const {
    const uint32_t slot = (uint32_t)n & (kTileRing - 1);
    ptx::st_shared_u32(ring_tile + 4u * slot, (uint32_t)w);
    ptx::mbar_arrive(ring_bar + 8u * slot);
    if constexpr (PAIR) {
      ptx::st_shared_cluster_u32(ptx::map_to_cta(ring_tile + 4u * slot, 1), (uint32_t)w);
      ptx::mbar_arrive_cluster(ptx::map_to_cta(ring_bar + 8u * slot, 1));
    }
  }
};

// Shared-memory matrix descriptor of a K-major operand tile whose rows are one
// 128-byte swizzle span: 8-row atoms 1024 bytes apart (stride byte offset),
// leading byte offset unused for swizzled K-major, descriptor version 1
// (sm_100), layout type 2 = 128-byte swizzle.  The reference packs the Hopper
// form of the same facts (lib/frontend/kernel_frontend.ml:34-51,
// lib/backend/ptx.ml:182-199); the bit layout differs on Blackwell.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// 32-bit UMMA instruction descriptor: f32 accumulate, both operands K-major.
template <int KIND>
__host__ __device__ constexpr uint32_t instr_desc(int umma_m, int umma_n) {
  uint32_t fmt = KIND == 0 ? 1u /* bf16 */ : 2u /* tf32 */;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(umma_n >> 3) << 17) |
         ((uint32_t)(umma_m >> 4) << 24);
}

// Split-K inside a cluster, reduction step: sum one column range of the S
// partial tiles parked in the S CTAs' shared memory (row r at r * row_bytes,
// 16-byte pieces XOR-swizzled by r % 8) and write it to C.  Remote loads have a
// long latency, so each thread keeps 16 of them in flight: UNROLL pieces x S
// slices, summed in ascending slice order (deterministic).
struct CrossSliceSum {
  uint32_t smem_base;       // this CTA's shared-memory address of the parked tile
  int row_bytes;            // bytes per row of a parked tile
  int piece0, pieces;       // first 16-byte piece of this CTA's column range, pieces per row (a power of two)
  int row0, col0;           // tile origin in C
  float *c;
  long long ldc;
  int c_rows, c_cols;

  template <int S>
  __device__ __forceinline__ void run(int tid, int nthreads) const {
    constexpr int UNROLL = 16 / S;
    uint32_t peer[S];
#pragma unroll
    for (int s = 0; s < S; s++) peer[s] = ptx::map_to_cta(smem_base, (uint32_t)s);
    const int total = 128 * pieces, lg = 31 - __clz(pieces);
    for (int i0 = tid; i0 < total; i0 += nthreads * UNROLL) {
      float4 v[UNROLL][S];
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const int i = i0 + u * nthreads;
        const int r = i >> lg, pc = piece0 + (i & (pieces - 1));
        const uint32_t off = (uint32_t)r * (uint32_t)row_bytes + (((uint32_t)pc ^ (uint32_t)(r & 7)) << 4);
#pragma unroll
        for (int s = 0; s < S; s++)
          if (i < total) v[u][s] = ptx::ld_shared_cluster_v4(peer[s] + off);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const int i = i0 + u * nthreads;
        if (i >= total) break;
        const int r = i >> lg, pc = piece0 + (i & (pieces - 1));
        float4 acc = v[u][0];
#pragma unroll
        for (int s = 1; s < S; s++) {
          acc.x += v[u][s].x;
          acc.y += v[u][s].y;
          acc.z += v[u][s].z;
          acc.w += v[u][s].w;
        }
        const int row = row0 + r, col = col0 + pc * 4;
        if (row < c_rows) {
          float *dst = c + (long long)row * ldc + col;
          if (col + 4 <= c_cols) {
            *reinterpret_cast<float4 *>(dst) = acc;
          } else {
            const float e[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int q = 0; q < 4; q++)
              if (col + q < c_cols) dst[q] = e[q];
          }
        }
      }
    }
  }
};

// The affine epilogue: v = (alpha * acc + beta * c_in) + bias, every step rounded
// on its own (no fused multiply-add), so a host that applies the same three
// operations in f32 to the plain GEMM's output gets the same bits.  It is
// applied to a 32x32 f32 sub-tile that already sits in the warp's swizzled
// staging buffer, not to the accumulator's own register layout (lane = row):
// there a lane would read its own row of C_in, 32 different 128-byte lines per
// warp instruction, and the load/store unit was busy with that for a quarter of
// a tile's time (4096^3: 151 us against 102 us plain).
// In the staged layout a warp instruction covers 4 rows x 128 bytes (lane -> row
// 4i + lane / 8, 16-byte piece lane % 8), so the reads of C_in are whole
// 128-byte lines, 4 per instruction, and they are issued one chunk ahead
// (affine_fetch_rows) so their latency hides behind the previous chunk's store.
struct AffineRows {
  float4 ci[8];
};

__device__ __forceinline__ void affine_fetch_rows(AffineRows &t, const GemmParams &p, int row0, int col0, int lane) {
  const int piece_col = col0 + 4 * (lane & 7);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = row0 + 4 * i + (lane >> 3);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.beta != 0.0f && row < p.c_rows) {
      const float *src = p.c_in + (long long)row * p.c_in_ld + piece_col;
      if (piece_col + 4 <= p.c_cols) {
        v = *reinterpret_cast<const float4 *>(src);
      } else {
        if (piece_col < p.c_cols) v.x = src[0];
        if (piece_col + 1 < p.c_cols) v.y = src[1];
        if (piece_col + 2 < p.c_cols) v.z = src[2];
      }
    }
    t.ci[i] = v;
  }
}

__device__ __forceinline__ void affine_apply_staged(uint32_t buf, const AffineRows &t, const GemmParams &p, int col0,
                                                    int lane) {
  const int piece = lane & 7, piece_col = col0 + 4 * piece;
  float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.bias) {
    if (piece_col + 4 <= p.c_cols) {
      b = __ldg(reinterpret_cast<const float4 *>(p.bias + piece_col));
    } else {
      if (piece_col < p.c_cols) b.x = __ldg(p.bias + piece_col);
      if (piece_col + 1 < p.c_cols) b.y = __ldg(p.bias + piece_col + 1);
      if (piece_col + 2 < p.c_cols) b.z = __ldg(p.bias + piece_col + 2);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int r = 4 * i + (lane >> 3);
    const uint32_t addr = buf + (uint32_t)r * 128u + (uint32_t)((piece ^ (r & 7)) << 4);
    float4 a = ptx::ld_shared_v4(addr);
    const float4 c = t.ci[i];
    a.x = __fadd_rn(__fadd_rn(__fmul_rn(p.alpha, a.x), __fmul_rn(p.beta, c.x)), b.x);
    a.y = __fadd_rn(__fadd_rn(__fmul_rn(p.alpha, a.y), __fmul_rn(p.beta, c.y)), b.y);
    a.z = __fadd_rn(__fadd_rn(__fmul_rn(p.alpha, a.z), __fmul_rn(p.beta, c.z)), b.z);
    a.w = __fadd_rn(__fadd_rn(__fmul_rn(p.alpha, a.w), __fmul_rn(p.beta, c.w)), b.w);
    ptx::st_shared_v4(addr, __float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w));
  }
}

// OUT16: C is stored as bf16 (round to nearest even) instead of f32 -- the
// narrow-output epilogue the reference lists as future work
// (docs/roadmap.md:67-71); the C map is then a bf16 map with 64-column boxes.
// NI: column blocks of BN per tile (tile width NI * BN).  NI == 2 exists for
// CTA pairs whose CTAs each stage 2 * BN / 2 CONTIGUOUS rows of B^T in one box
// (the reference's 256-row B^T box): UMMA `ni` of a K step reads rows
// [ni * BN/2, (ni + 1) * BN/2) of both CTAs' stages, so accumulator column j of
// block ni is tile column (j / (BN/2)) * BN + ni * BN/2 + j % (BN/2).
// AFFINE: the epilogue applies alpha, beta * C_in and a bias row (affine_apply_staged) in
// f32, before the rounding to bf16 when OUT16 is set as well.
template <int KIND, int BM_CTA, int BN, int CTA_GROUP, bool OUT16 = false, bool FANOUT = false, int NI = 1,
          bool AFFINE = false>
__global__ void __launch_bounds__(kThreadsPerCta, 1)
umma_gemm_kernel(const __grid_constant__ typename std::conditional<FANOUT, GemmParamsFanout, GemmParams>::type p) {
  static_assert(!(FANOUT && OUT16), "the fan-out epilogue writes f32");
  // A CTA owns BM_CTA rows of the tile as MI blocks of 128 rows (one UMMA each
  // per K step, all sharing the staged B^T rows).  Block `mi` of accumulator
  // set `set` is one hand-off unit between the issuer and the epilogue.
  constexpr int MI = BM_CTA / 128;
  constexpr int U = MI * NI;                      // hand-off units (UMMA blocks) per accumulator set
  constexpr int UMMA_M = 128 * CTA_GROUP;         // rows one instruction produces (per pair)
  constexpr int B_ROWS = BN / CTA_GROUP;          // rows of B^T this CTA stages per column block
  constexpr int ACC_COLS = U * BN;                // TMEM columns of one accumulator set
  constexpr int SETS = (2 * ACC_COLS <= 512) ? 2 : 1;  // two sets: epilogue overlaps next main loop
  constexpr int TMEM_COLS = SETS * ACC_COLS;
  constexpr int CHUNKS = BN / 32;                 // 32-column epilogue chunks per unit
  // 8 epilogue warps form two groups; with two units group g drains unit g,
  // with one unit the groups split its columns.
  constexpr int CHUNKS_PER_GROUP = U == 2 ? CHUNKS : CHUNKS / 2;
  constexpr int EMPTY_ARRIVALS = (U == 2 ? 4 : 8) * CTA_GROUP;
  constexpr uint32_t A_BYTES = BM_CTA * 128;
  constexpr uint32_t B_BYTES = NI * B_ROWS * 128;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t IDESC = instr_desc<KIND>(UMMA_M, BN);
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM allocation must be a power of two");
  static_assert(BM_CTA == 128 || BM_CTA == 256, "unsupported tile");
  static_assert(NI == 1 || (NI == 2 && MI == 1 && CTA_GROUP == 2 && !OUT16), "unsupported column blocking");
  static_assert(CHUNKS_PER_GROUP >= 1 && CHUNKS % 2 == 0, "unsupported tile width");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const int stages = p.stages;
  const uint32_t staging_base = smem_base + (uint32_t)stages * STAGE_BYTES;
  const uint32_t bar_base = staging_base + kEpilogueStagingBytes;
  // barrier region: full[8], empty[8], tmem_full[4], tmem_empty[4], drain,
  // the TMEM base slot and the abort flag, then the announced-tile ring
  // (barriers, then tile indices).
  const uint32_t full_bar = bar_base;
  const uint32_t empty_bar = bar_base + 8u * kMaxStages;
  const uint32_t tmem_full_bar = bar_base + 16u * kMaxStages;
  const uint32_t tmem_empty_bar = tmem_full_bar + 32u;
  const uint32_t drain_bar = tmem_empty_bar + 32u;
  const uint32_t tmem_slot = drain_bar + 8u;
  const uint32_t abort_slot = tmem_slot + 4u;
  const uint32_t ring_bar = abort_slot + 4u;
  const uint32_t ring_tile = ring_bar + 8u * kTileRing;
  static_assert(16 * kMaxStages + 32 + 32 + 8 + 4 + 4 + 12 * kTileRing <= kBarrierRegionBytes, "barrier region");
  uint8_t *const generic_base = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  volatile uint32_t *const tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t *>(generic_base + (tmem_slot - smem_base));
  volatile uint32_t *const abort_ptr =
      reinterpret_cast<volatile uint32_t *>(generic_base + (abort_slot - smem_base));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = CTA_GROUP == 2 ? ptx::cluster_ctarank() : 0u;
  const bool is_leader = cta_rank == 0;
  const int cluster_id = CTA_GROUP == 2 ? (int)ptx::cluster_id_x() : (int)blockIdx.x;
  const int num_clusters = CTA_GROUP == 2 ? (int)ptx::num_clusters_x() : (int)gridDim.x;

  const void *map_a = p.a_map_ptr ? p.a_map_ptr : (const void *)&p.map_a;
  const void *map_b = p.b_map_ptr ? p.b_map_ptr : (const void *)&p.map_b;
  const void *map_c = (const void *)&p.map_c;

  const WaitCtx wctx{p.wait_budget_ns, abort_ptr};
  const int total_work = p.tiles_m * p.tiles_n * p.splits;
  const bool dynamic = p.sched_slot_plus1 > 0;
  TileFeed<CTA_GROUP == 2> feed{dynamic, cluster_id, num_clusters, total_work, ring_bar, ring_tile};

  // ---- set-up ---------------------------------------------------------------
  // The kernel's parameters sit in the constant bank, cold at every launch, and a
  // miss costs a few hundred clocks.  The producer lane would take those misses one
  // after the other on its way to the first load (hints, split geometry, queue
  // slot: different lines); warps that have nothing to do yet touch one line each
  // now, in parallel, so the lines are there when the roles need them.
  if (lane == 0 && warp >= 2) {
    // one field in every 32 bytes of the scalar part of the parameter block
    const int touched = warp == 2   ? p.tiles_m
                        : warp == 3 ? p.splits
                        : warp == 4 ? p.c_rows
                        : warp == 5 ? __float_as_int(p.alpha)
                        : warp == 6 ? p.sched_slot_plus1
                        : warp == 7 ? p.div_per_group.d
                        : warp == 8 ? p.div_group.d
                                    : p.hint_a;
    asm volatile("" ::"r"(touched));
  }
  if (threadIdx.x == 0) {
    *abort_ptr = 0;
    for (int s = 0; s < stages; s++) {
      ptx::mbar_init(full_bar + 8u * s, 1);
      ptx::mbar_init(empty_bar + 8u * s, 1);
    }
    for (int u = 0; u < SETS * U; u++) {
      ptx::mbar_init(tmem_full_bar + 8u * u, 1);
      // one arrival per epilogue warp (of every CTA feeding this issuer) that reads the unit
      ptx::mbar_init(tmem_empty_bar + 8u * u, EMPTY_ARRIVALS);
    }
    ptx::mbar_init(drain_bar, 1);
    for (int i = 0; i < kTileRing; i++) ptx::mbar_init(ring_bar + 8u * i, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(map_a);
    ptx::prefetch_tensormap(map_b);
    if constexpr (FANOUT) {
      for (int d = 0; d < p.n_dests; d++) ptx::prefetch_tensormap(&p.dest_maps[d]);
    } else {
      ptx::prefetch_tensormap(map_c);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc<CTA_GROUP>(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish<CTA_GROUP>();
  }
  // What the producer lane needs before its first load and can work out from the
  // kernel's parameters alone: the cache policies and where its first tile lies
  // (a chain of integer divisions, about a microsecond for one thread).
  struct ProducerTile {
    int a_row0, b_row0, kb_begin, kb_end;
  };
  auto producer_tile = [&](int w) {
    int t, sp, tm, tn;
    split_work(p, w, &t, &sp);
    tile_coords(p, t, &tm, &tn);
    ProducerTile r;
    r.kb_begin = sp * p.kb_per_split;
    r.kb_end = min(p.num_k_blocks, r.kb_begin + p.kb_per_split);
    r.a_row0 = tm * (BM_CTA * CTA_GROUP) + (int)cta_rank * BM_CTA;
    r.b_row0 = tn * (NI * BN) + (int)cta_rank * (NI * B_ROWS);
    return r;
  };
  uint64_t pol_a = 0, pol_b = 0;
  ProducerTile first_tile{0, 0, 0, 0};
  auto producer_preamble = [&]() {  // producer lane only
    auto policy = [](int h) {
      return h == 1 ? ptx::l2_policy_evict_first() : h == 2 ? ptx::l2_policy_evict_last()
                                                             : ptx::l2_policy_evict_normal();
    };
    // (the empty asm statements pin the arithmetic between the barrier arrival
    // before this call and the wait after it: both are volatile asm too)
    int first = cluster_id;
    asm volatile("" : "+r"(first));
    if (first < total_work) first_tile = producer_tile(first);
    pol_a = policy(p.hint_a);
    pol_b = policy(p.hint_b);
    asm volatile("" : "+r"(first_tile.a_row0), "+r"(first_tile.b_row0), "+r"(first_tile.kb_begin), "+r"(first_tile.kb_end));
  };
  ptx::tc_fence_before_sync();
  if constexpr (CTA_GROUP == 2) {
    __syncthreads();
    // The peer's barriers must exist before anything arrives on them remotely.
    // The two CTAs of a pair do not start at the same instant: the producer lane
    // does its arithmetic between its arrival and the wait, under that skew.
    ptx::cluster_arrive_relaxed();
    if (warp == 0) {
      if (lane == 0) producer_preamble();
      __syncwarp();
    }
    ptx::cluster_wait();
  } else {
    // The producer warp needs nothing the other warps set up (its lane initialised
    // the barriers itself, and it never touches TMEM): it arrives and goes straight
    // to its first loads, which are then in flight while the TMEM allocation and
    // this hand-off complete -- about a microsecond earlier, which a problem that
    // lasts tens of microseconds notices.
    if (warp == 0) {
      ptx::named_barrier_arrive(3u, kThreadsPerCta);
      if (lane == 0) producer_preamble();
      __syncwarp();
    } else {
      ptx::named_barrier_sync(3u, kThreadsPerCta);
    }
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Everything above touched only this CTA's shared memory, TMEM and the kernel's
  // own parameters, so under a programmatic dependent launch it has overlapped the
  // tail of the kernel before this one in the stream.  The roles that touch global
  // memory (the producer: operands and the tile queue; the epilogue: C, C_in, bias)
  // wait for that kernel themselves, as late as they can; the issuer works on
  // shared memory and TMEM only and needs no wait of its own.

  // ---- roles ------------------------------------------------------------------
  // cluster_reduce == 2: one cluster barrier phase separates the zeroing of the C
  // tile (every epilogue warp of both CTAs, before it waits for its accumulator)
  // from the first addition into it.  Every thread arrives exactly once; the
  // producer and issuer warps arrive at once and collect the phase when their
  // role is over.
  bool reduce_add = false;
  // (only the plain one-CTA 128-row kernels are ever launched as split-K clusters)
  constexpr bool CLUSTER_SPLIT_CAPABLE = CTA_GROUP == 1 && MI == 1 && !OUT16 && !FANOUT && !AFFINE;
  if constexpr (CLUSTER_SPLIT_CAPABLE) reduce_add = p.cluster_reduce == 2;
  if (reduce_add && warp < 2) ptx::cluster_arrive();
  if (warp == 0) {
    // ===== TMA producer (examples/kernels/gemm.ml:92-98 `prefetch`) =====
    if (lane == 0) {
      const uint32_t full_remote0 =
          CTA_GROUP == 2 ? ptx::map_to_cta(full_bar, 0) : full_bar;  // leader's full[0]
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      // The leader's lane owns the dynamic schedule: it announces this cluster's
      // tile n + 1 (taken from the queue) before it loads tile n, so the other
      // roles never wait for an index.  The peer CTA's lane reads the ring.
      const bool announcer = dynamic && is_leader;
      unsigned int *const queue = g_tile_queue + 2 * (dynamic ? p.sched_slot_plus1 - 1 : 0);
      if (announcer) feed.announce(0, cluster_id);
      int w = announcer ? cluster_id : feed.take(wctx);
      // The first tile of every CTA is tile `cluster_id` (static walk, or the one the
      // leader announced first); its coordinates come from the set-up.  Those of each
      // later tile are worked out right after the loads of the tile before it have
      // been issued, while they are in flight.
      ProducerTile pt = first_tile;
      if (w >= 0 && w < total_work && w != cluster_id) pt = producer_tile(w);
      for (int n_local = 0; ok && w >= 0 && w < total_work; n_local++) {
        const int kb_begin = pt.kb_begin, kb_end = pt.kb_end, a_row0 = pt.a_row0, b_row0 = pt.b_row0;
        if (n_local == 0) {
          // first access to global memory (the queue, then the operands)
          ptx::grid_dependency_wait();
          ptx::grid_launch_dependents();
        }
        int w_next = 0;
        if (announcer) {
          w_next = num_clusters + (int)atomicAdd(queue, 1u);
          feed.announce(n_local + 1, w_next);
        }
        for (int kb = kb_begin; kb < kb_end; kb++) {
          if (!bounded_wait(empty_bar + 8u * stage, phase ^ 1u, wctx, WAIT_EMPTY, (uint32_t)stage)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + (uint32_t)stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          const int kc = kb * p.k_block_elems;
          if constexpr (CTA_GROUP == 1) {
            const uint32_t bar = full_bar + 8u * stage;
            ptx::mbar_arrive_expect_tx(bar, STAGE_BYTES);
            for (int r = 0; r < BM_CTA; r += p.a_box_rows)
              ptx::tma_load_2d_hint(a_dst + (uint32_t)r * 128u, map_a, kc, a_row0 + r, bar, pol_a);
            for (int r = 0; r < NI * B_ROWS; r += p.b_box_rows)
              ptx::tma_load_2d_hint(b_dst + (uint32_t)r * 128u, map_b, kc, b_row0 + r, bar, pol_b);
          } else {
            // Both CTAs credit the leader's barrier; the leader expects the
            // bytes of the whole pair.
            if (is_leader) ptx::mbar_arrive_expect_tx(full_bar + 8u * stage, 2u * STAGE_BYTES);
            const uint32_t bar = full_remote0 + 8u * stage;
            for (int r = 0; r < BM_CTA; r += p.a_box_rows)
              ptx::tma_load_2d_pair_hint(a_dst + (uint32_t)r * 128u, map_a, kc, a_row0 + r, bar, pol_a);
            for (int r = 0; r < NI * B_ROWS; r += p.b_box_rows)
              ptx::tma_load_2d_pair_hint(b_dst + (uint32_t)r * 128u, map_b, kc, b_row0 + r, bar, pol_b);
          }
          issued++;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        w = announcer ? w_next : feed.take(wctx);
        if (w >= 0 && w < total_work) pt = producer_tile(w);
      }
      if (w < 0) ok = false;
      if (!ok || *abort_ptr) {
        // Abort path: let the loads already issued land before shared memory
        // is given up (the leader's full barriers count both CTAs' bytes).
        if (CTA_GROUP == 1 || is_leader) {
          long long n = issued < stages ? issued : stages;
          for (long long i = 0; i < n; i++) {
            int s = (int)((issued - 1 - i) % stages);
            uint32_t ph = (uint32_t)(((issued - 1 - i) / stages) & 1);
            const uint64_t t0 = ptx::globaltimer_ns();
            while (!ptx::mbar_try_wait(full_bar + 8u * s, ph)) {
              if (ptx::globaltimer_ns() - t0 > 50ull * 1000 * 1000) break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===== UMMA issuer (examples/kernels/gemm.ml:107-141, the K loop) =====
    if (lane == 0 && is_leader) {
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      // Four UMMAs (32 bytes of K each: 16 bf16 / 8 tf32) of K block `kb` for
      // row block `mi`, reading ring slot `slot`.  The start address advances
      // inside the swizzle span, as the reference does with its `+8*ki` /
      // `+16*ki` element offsets (gemm.ml:121-125).
      auto issue = [&](int slot, int u, uint32_t d_tmem, bool first_block) {
        const uint32_t a_addr = smem_base + (uint32_t)slot * STAGE_BYTES;
        const uint64_t a_desc = smem_desc_sw128(a_addr) + (uint64_t)(((MI == 2 ? u : 0) * 128 * 128) >> 4);
        const uint64_t b_desc = smem_desc_sw128(a_addr + A_BYTES) + (uint64_t)(((NI == 2 ? u : 0) * B_ROWS * 128) >> 4);
#pragma unroll
        for (int ki = 0; ki < 4; ki++)
          ptx::umma<KIND, CTA_GROUP>(d_tmem + (uint32_t)(u * BN), a_desc + (uint64_t)(ki * 2),
                                     b_desc + (uint64_t)(ki * 2), IDESC, (!first_block || ki > 0) ? 1u : 0u);
      };
      auto release_slot = [&](int slot) {  // frees the ring slot once the UMMAs issued so far have read it
        if constexpr (CTA_GROUP == 1) ptx::umma_commit(empty_bar + 8u * slot);
        else ptx::umma_commit_pair(empty_bar + 8u * slot, 3);
      };
      auto publish = [&](int unit) {  // wakes the epilogue of every CTA holding rows of this unit
        if constexpr (CTA_GROUP == 1) ptx::umma_commit(tmem_full_bar + 8u * unit);
        else ptx::umma_commit_pair(tmem_full_bar + 8u * unit, 3);
      };
      // slot / parity of the i-th upcoming K block (i < stages)
      auto slot_of = [&](int i) { return stage + i >= stages ? stage + i - stages : stage + i; };
      auto phase_of = [&](int i) { return stage + i >= stages ? phase ^ 1u : phase; };
      auto advance = [&]() {
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      };
      for (int w = feed.take(wctx); ok && w < total_work; w = feed.take(wctx), local_tile++) {
        if (w < 0) {
          ok = false;
          break;
        }
        int t_of_w, sp;
        split_work(p, w, &t_of_w, &sp);
        const int kb_begin = sp * p.kb_per_split;
        const int kb_end = min(p.num_k_blocks, kb_begin + p.kb_per_split);
        const int set = local_tile % SETS;
        const uint32_t set_phase = (uint32_t)(local_tile / SETS) & 1u;
        const uint32_t d_tmem = tmem_base + (uint32_t)(set * ACC_COLS);
        // With two row blocks per CTA the first and last G K blocks of a tile
        // are issued block-major (all of row block 0, then all of row block 1)
        // instead of interleaved: at the end of a tile row block 0 is complete G
        // block-times before row block 1, so its epilogue starts early, and at
        // the start of the next tile row block 0 can accumulate again while row
        // block 1 is still being drained.  The G slots involved stay occupied
        // until the second pass has read them.
        int G = 0;
        if constexpr (U == 2) {
          G = p.reorder_kb;
          if (G > stages - 1) G = stages - 1;
          if (G > (kb_end - kb_begin) / 2) G = (kb_end - kb_begin) / 2;
        }
        int kb = kb_begin;
        if (G > 0) {
          // ---- head, row block 0 then row block 1 ----
          ok = bounded_wait(tmem_empty_bar + 8u * (set * U), set_phase ^ 1u, wctx, WAIT_TMEM_EMPTY, (uint32_t)w);
          for (int i = 0; ok && i < G; i++) {
            ok = bounded_wait(full_bar + 8u * slot_of(i), phase_of(i), wctx, WAIT_FULL, (uint32_t)slot_of(i));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            issue(slot_of(i), 0, d_tmem, i == 0);
          }
          if (ok) ok = bounded_wait(tmem_empty_bar + 8u * (set * U + 1), set_phase ^ 1u, wctx, WAIT_TMEM_EMPTY, (uint32_t)w);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          for (int i = 0; i < G; i++) {
            issue(stage, 1, d_tmem, i == 0);
            release_slot(stage);
            advance();
          }
          kb += G;
        } else {
          for (int mi = 0; ok && mi < U; mi++)
            ok = bounded_wait(tmem_empty_bar + 8u * (set * U + mi), set_phase ^ 1u, wctx,
                              WAIT_TMEM_EMPTY, (uint32_t)w);
          if (!ok) break;
          ptx::tc_fence_after_sync();
        }
        // ---- body: row blocks interleaved per K block ----
        for (; kb < kb_end - G; kb++) {
          if (!bounded_wait(full_bar + 8u * stage, phase, wctx, WAIT_FULL, (uint32_t)stage)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int mi = 0; mi < U; mi++) issue(stage, mi, d_tmem, kb == kb_begin);
          release_slot(stage);
          advance();
        }
        if (!ok) break;
        if (G > 0) {
          // ---- tail, row block 0 then row block 1 ----
          for (int i = 0; ok && i < G; i++) {
            ok = bounded_wait(full_bar + 8u * slot_of(i), phase_of(i), wctx, WAIT_FULL, (uint32_t)slot_of(i));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            issue(slot_of(i), 0, d_tmem, false);
          }
          if (!ok) break;
          publish(set * U);
          for (int i = 0; i < G; i++) {
            issue(stage, 1, d_tmem, false);
            release_slot(stage);
            advance();
          }
          publish(set * U + 1);
        } else {
          for (int mi = 0; mi < U; mi++) publish(set * U + mi);
        }
      }
      if (!ok || *abort_ptr) {
        // let every UMMA in flight retire before TMEM is released
        ptx::umma_commit(drain_bar);
        const uint64_t t0 = ptx::globaltimer_ns();
        while (!ptx::mbar_try_wait(drain_bar, 0)) {
          if (ptx::globaltimer_ns() - t0 > 50ull * 1000 * 1000) break;
        }
      }
    }
  } else {
    // ===== epilogue (examples/kernels/gemm.ml:143-161) =====
    const int quad = warp & 3;         // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    const int ew = warp - 2;           // 0..7, staging slot
    const int group = ew >> 2;         // 0 or 1
    const int mi = U == 2 ? group : 0;  // the unit this warp drains
    const int ch_begin = U == 2 ? 0 : group * CHUNKS_PER_GROUP;
    const uint32_t buf = staging_base + (uint32_t)ew * 4096u;  // one 32x32 f32 sub-tile
    const uint32_t row_addr = buf + (uint32_t)lane * 128u;
    const uint32_t tmem_empty_remote =
        CTA_GROUP == 2 ? ptx::map_to_cta(tmem_empty_bar, 0) : tmem_empty_bar;
    int local_tile = 0;
    const uint64_t pol_c = p.hint_c == 1 ? ptx::l2_policy_evict_first()
                           : p.hint_c == 2 ? ptx::l2_policy_evict_last() : ptx::l2_policy_evict_normal();
    ptx::grid_dependency_wait();  // before anything of C, C_in or the bias is touched
    for (;; local_tile++) {
      // Every pass ends in the group's named barrier below, the last one
      // included: the four warps of a group leave the loop together or not at
      // all, whatever each of them saw (a warp that gave up on a wait while its
      // neighbours went on would leave them in a hardware barrier for good).
      const int w = feed.take(wctx);
      const bool valid = w >= 0 && w < total_work;
      const int set = local_tile % SETS;
      const uint32_t set_phase = (uint32_t)(local_tile / SETS) & 1u;
      const int unit = set * U + mi;
      // where the tile goes: worked out before the wait, not between the
      // accumulator becoming ready and the first TMEM load
      int tm = 0, tn = 0, sp = 0;
      if (valid) {
        int t;
        split_work(p, w, &t, &sp);
        tile_coords(p, t, &tm, &tn);
      }
      const int c_row = sp * p.split_row_stride + tm * (BM_CTA * CTA_GROUP) + (int)cta_rank * BM_CTA +
                        (MI == 2 ? mi * 128 : 0) + quad * 32;
      if (reduce_add && local_tile == 0) {
        // Zero this warp's part of the C tile (its 32 rows): K slice 0 takes the even
        // 32-column chunks, slice 1 the odd ones.  Ordinary stores, four whole
        // 128-byte rows per instruction; the proxy fence orders them before the TMA
        // reductions that follow the barrier.
        if (valid) {
          for (int c = 0; c < CHUNKS_PER_GROUP; c++) {
            if (((ch_begin + c) & 1) != (sp & 1)) continue;
            const int col = tn * BN + (ch_begin + c) * 32 + 4 * (lane & 7);
            if (col >= p.c_cols) continue;
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int row = c_row + 4 * j + (lane >> 3);
              if (row < p.c_rows) ptx::st_global_v4_zero(p.c_ptr + (size_t)row * (size_t)p.c_ld + col);
            }
          }
          ptx::fence_proxy_async_global();
          __syncwarp();
        }
        ptx::cluster_arrive();
      }
      bool stop = !valid;
      if (valid && (ew & 3) == 0 && lane == 0)
        stop = !bounded_wait(tmem_full_bar + 8u * unit, set_phase, wctx, WAIT_TMEM_FULL, (uint32_t)w);
      __syncwarp();
      // One lane of each group of four warps waits on the accumulator's barrier
      // (the wait can last a whole main loop); everyone else sleeps in the named
      // barrier, which issues nothing, and its OR hands all 128 threads the same
      // verdict.
      if (ptx::named_barrier_or(1u + (uint32_t)group, 128u, stop)) break;
      if (reduce_add) ptx::cluster_wait();  // the whole tile of C is zero, in both CTAs' view
      // The last tile of this CTA (static walk), single accumulator unit: its UMMAs
      // are all complete, no load is in flight or will be issued, so the operand
      // ring is free.  Each 32-column chunk then gets a staging buffer of its own
      // there (at most four per warp with these tiles) and no chunk waits for the
      // TMA store before it to have read its source: what a problem of one tile per
      // CTA sees of the epilogue is a chain of store latencies otherwise.
      bool spread = false;
      if constexpr (U == 1 && CHUNKS_PER_GROUP <= 4)
        spread = !dynamic && w + num_clusters >= total_work && (uint32_t)stages * STAGE_BYTES >= 8u * 3u * 4096u;
      auto chunk_buf = [&](int c) {  // staging buffer of the c-th chunk this warp handles
        return spread && c > 0 ? smem_base + (uint32_t)(ew * 3 + (c - 1)) * 4096u : buf;
      };
      // first column in C of this warp's chunk c (32 accumulator columns)
      auto chunk_col = [&](int c) {
        const int j = (ch_begin + c) * 32;
        if constexpr (NI == 1) return tn * BN + j;
        else return tn * (NI * BN) + (j / B_ROWS) * (NI * B_ROWS) + mi * B_ROWS + j % B_ROWS;
      };
      ptx::tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) +
                              (uint32_t)(set * ACC_COLS + mi * BN + ch_begin * 32);
      if constexpr (CLUSTER_SPLIT_CAPABLE) {
        if (p.cluster_reduce == 1) {
          // Leave this CTA's partial tile in its own shared memory, in the (now
          // idle) operand ring: row r at r * BN * 4 bytes, 16-byte pieces
          // XOR-swizzled by r % 8 inside each 128-byte group.
          const uint32_t row_base = smem_base + (uint32_t)(quad * 32 + lane) * (uint32_t)(BN * 4);
#pragma unroll 1
          for (int c = 0; c < CHUNKS_PER_GROUP; c++) {
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32(t_addr + (uint32_t)(c * 32), v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const uint32_t piece = (uint32_t)((ch_begin + c) * 8 + j) ^ (uint32_t)(lane & 7);
              ptx::st_shared_v4(row_base + (piece << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
          }
          continue;  // exactly one work item per CTA in this mode
        }
      }
      auto release_unit = [&]() {
        // the unit is in registers everywhere in this warp: hand it back to
        // the issuer before finishing the stores
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTA_GROUP == 1) ptx::mbar_arrive(tmem_empty_bar + 8u * unit);
          else ptx::mbar_arrive_cluster(tmem_empty_remote + 8u * unit);
        }
      };
      if constexpr (!OUT16) {
        // Software-pipelined over 32-column chunks: the TMEM load of chunk c+1 is
        // in flight while chunk c goes through shared memory to the TMA store.
        uint32_t va[32], vb[32];
        AffineRows cin_a, cin_b;  // C_in of the current / the next chunk (AFFINE only)
        ptx::tmem_ld_32x32b_x32(t_addr, va);
        if constexpr (AFFINE) affine_fetch_rows(cin_a, p, c_row, chunk_col(0), lane);
#pragma unroll
        for (int c = 0; c < CHUNKS_PER_GROUP; c++) {
          uint32_t(&cur)[32] = (c & 1) ? vb : va;
          uint32_t(&nxt)[32] = (c & 1) ? va : vb;
          ptx::tmem_ld_wait();
          if (c + 1 < CHUNKS_PER_GROUP) ptx::tmem_ld_32x32b_x32(t_addr + (uint32_t)((c + 1) * 32), nxt);
          else release_unit();
          if constexpr (AFFINE) {
            if (c + 1 < CHUNKS_PER_GROUP) affine_fetch_rows((c & 1) ? cin_a : cin_b, p, c_row, chunk_col(c + 1), lane);
          }
          // the previous store must be done reading the staging buffer
          const uint32_t cbuf = chunk_buf(c), crow = cbuf + (uint32_t)lane * 128u;
          if (!spread || c == 0) {
            if (lane == 0) ptx::tma_store_wait_read<0>();
            __syncwarp();
          }
          // row `lane` of the 32x32 sub-tile, 16-byte chunks XOR-swizzled by
          // (row % 8) as the 128-byte-swizzle store map expects
#pragma unroll
          for (int j = 0; j < 8; j++) {
            ptx::st_shared_v4(crow + (uint32_t)((j ^ (lane & 7)) << 4), cur[4 * j], cur[4 * j + 1],
                              cur[4 * j + 2], cur[4 * j + 3]);
          }
          if constexpr (AFFINE) {
            __syncwarp();  // the whole sub-tile is staged: transform it in place, four rows per instruction
            affine_apply_staged(cbuf, (c & 1) ? cin_b : cin_a, p, chunk_col(c), lane);
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if constexpr (FANOUT) {
              // one bulk group per sub-tile: the staging buffer is reused once
              // every destination's store has read it
              for (int d = 0; d < p.n_dests; d++)
                ptx::tma_store_2d_hint(&p.dest_maps[d], chunk_col(c), c_row, cbuf, pol_c);
            } else if (reduce_add) {
              ptx::tma_reduce_add_2d(map_c, chunk_col(c), c_row, cbuf);
            } else {
              ptx::tma_store_2d_hint(map_c, chunk_col(c), c_row, cbuf, pol_c);
            }
            ptx::tma_store_commit();
          }
        }
      } else {
        // bf16 C: two 32-column chunks make one 128-byte row of 64 bf16.
        static_assert(CHUNKS_PER_GROUP % 2 == 0, "bf16 output needs column chunks in pairs");
#pragma unroll 1
        for (int c2 = 0; c2 < CHUNKS_PER_GROUP / 2; c2++) {
          uint32_t va[32], vb[32];
          ptx::tmem_ld_32x32b_x32(t_addr + (uint32_t)(c2 * 64), va);
          ptx::tmem_ld_32x32b_x32(t_addr + (uint32_t)(c2 * 64 + 32), vb);
          AffineRows cin_a, cin_b;
          if constexpr (AFFINE) {  // in flight while the accumulator chunks arrive
            affine_fetch_rows(cin_a, p, c_row, chunk_col(2 * c2), lane);
            affine_fetch_rows(cin_b, p, c_row, chunk_col(2 * c2) + 32, lane);
          }
          ptx::tmem_ld_wait();
          if (c2 + 1 == CHUNKS_PER_GROUP / 2) release_unit();
          if (lane == 0) ptx::tma_store_wait_read<0>();
          __syncwarp();
          if constexpr (AFFINE) {
            // In f32, before the one rounding to bf16: each 32-column half goes through
            // the staging buffer as f32, is transformed there four rows per instruction
            // (coalesced C_in, see affine_apply_staged) and comes back to its row's lane.
#pragma unroll
            for (int h = 0; h < 2; h++) {
              uint32_t(&v)[32] = h == 0 ? va : vb;
#pragma unroll
              for (int j = 0; j < 8; j++)
                ptx::st_shared_v4(row_addr + (uint32_t)((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2],
                                  v[4 * j + 3]);
              __syncwarp();
              affine_apply_staged(buf, h == 0 ? cin_a : cin_b, p, chunk_col(2 * c2) + 32 * h, lane);
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 t = ptx::ld_shared_v4(row_addr + (uint32_t)((j ^ (lane & 7)) << 4));
                v[4 * j] = __float_as_uint(t.x), v[4 * j + 1] = __float_as_uint(t.y);
                v[4 * j + 2] = __float_as_uint(t.z), v[4 * j + 3] = __float_as_uint(t.w);
              }
              __syncwarp();
            }
          }
#pragma unroll
          for (int j = 0; j < 8; j++) {
            uint32_t(&src)[32] = j < 4 ? va : vb;
            const int o = (j & 3) * 8;
            ptx::st_shared_v4(row_addr + (uint32_t)((j ^ (lane & 7)) << 4),
                              ptx::pack_bf16x2(src[o], src[o + 1]), ptx::pack_bf16x2(src[o + 2], src[o + 3]),
                              ptx::pack_bf16x2(src[o + 4], src[o + 5]), ptx::pack_bf16x2(src[o + 6], src[o + 7]));
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            ptx::tma_store_2d_hint(map_c, chunk_col(2 * c2), c_row, buf, pol_c);
            ptx::tma_store_commit();
          }
        }
      }
    }
    if (lane == 0) ptx::tma_store_wait_all<0>();
    __syncwarp();
  }
  if (reduce_add && warp < 2) {
    __syncwarp();
    ptx::cluster_wait();
  }

  // ---- split-K reduction across the cluster --------------------------------------
  if constexpr (CLUSTER_SPLIT_CAPABLE) {
    if (p.cluster_reduce == 1) {
      // Every thread of every CTA passes both cluster barriers, whatever
      // happened in its role (a timed-out wait included), so nobody is left
      // waiting; the data is only meaningful if no wait timed out, which the
      // status block tells the host.
      __syncthreads();
      ptx::cluster_arrive();
      ptx::cluster_wait();  // all partial tiles of the cluster are in place
      if (warp >= 2 && blockIdx.x < (unsigned)total_work) {
        const int S = p.splits;
        const int rank = (int)(blockIdx.x % (unsigned)S);
        const int t = (int)(blockIdx.x / (unsigned)S);
        int tm, tn;
        tile_coords(p, t, &tm, &tn);
        const int pieces_per_row = (BN / 4) / S;  // this CTA's column range, in 16-byte pieces
        const int row0 = tm * 128, col0 = tn * BN;
        const CrossSliceSum job{smem_base, BN * 4, rank * pieces_per_row, pieces_per_row, row0, col0,
                                p.c_ptr, p.c_ld, p.c_rows, p.c_cols};
        if (S == 2) job.template run<2>((int)threadIdx.x - 64, kThreadsPerCta - 64);
        else if (S == 4) job.template run<4>((int)threadIdx.x - 64, kThreadsPerCta - 64);
        else job.template run<8>((int)threadIdx.x - 64, kThreadsPerCta - 64);
      }
      ptx::cluster_arrive();
      ptx::cluster_wait();  // nobody retires while a peer may still read its shared memory
    }
  }

  // ---- teardown -----------------------------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (CTA_GROUP == 2) {
    // the leader's UMMAs read the peer's shared memory and arrive on its
    // barriers: neither CTA may retire before both are done
    __syncwarp();
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<CTA_GROUP>(tmem_base, TMEM_COLS);
  }
  if (dynamic && is_leader && threadIdx.x == 0) {
    // This cluster takes no more tiles.  The last cluster to get here leaves the
    // queue as it found it, ready for the slot's next launch.
    unsigned int *const queue = g_tile_queue + 2 * (p.sched_slot_plus1 - 1);
    __threadfence();
    if (atomicAdd(queue + 1, 1u) == (unsigned)num_clusters - 1u) {
      queue[0] = 0u;
      queue[1] = 0u;
      __threadfence();
    }
  }
}

// The bounded-wait self test: one CTA waits on a barrier nothing arrives on.
// The wait must give up after `budget_ns`, record WAIT_SELFTEST in the status
// block and return normally.
__global__ void bounded_wait_selftest_kernel(unsigned long long budget_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_mbar_init();
    WaitCtx ctx{budget_ns, &abort_flag};
    bounded_wait(ptx::smem_u32(&bar), 0, ctx, WAIT_SELFTEST, 0);
  }
}

}  // namespace oxgpu
