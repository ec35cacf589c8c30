// C-ABI launch layer: argument contracts, tensor-map encoding, variant choice
// and kernel launches.  Host-side counterpart of the reference's launcher
// (test/hardware/run_gemm_h100.cu:46-72,119-122,164-186; bench/bench.py:
// 126-156,266-292).  There is no CPU fallback anywhere in this file: every
// compute entry point either launches a CUDA kernel or returns an error.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "common.hpp"
#include "umma_gemm.cuh"
#include "util_kernels.cuh"

namespace oxgpu {

namespace {

constexpr int kMaxDevices = 64;
constexpr int kKinds = 8;     // 0 = bf16, 1 = tf32, 2 = bf16 with bf16 C, 3 / 4 = bf16 / tf32 fan-out, 5 / 6 = affine, 7 = affine with bf16 C
constexpr int kVariants = 12;  // index by Variant value

std::atomic<uint64_t> g_launches{0};
std::atomic<unsigned> g_sched_seq{0};  // next queue slot of the dynamic tile schedule (round robin)

// OXGPU_TILE_SCHEDULE=static keeps every launch on the static walk (cluster c
// takes tiles c, c + clusters, ...); anything else leaves the choice to the
// library.  Read at every launch so a process can switch.
bool static_schedule_forced() {
  const char *e = std::getenv("OXGPU_TILE_SCHEDULE");
  return e && std::strcmp(e, "static") == 0;
}

// OXGPU_DEPENDENT_LAUNCH=0 launches the GEMM kernels as ordinary stream-ordered
// kernels; anything else lets each one start its set-up (barriers, TMEM
// allocation, descriptor prefetch) under the tail of the kernel before it.
bool dependent_launch_enabled() {
  const char *e = std::getenv("OXGPU_DEPENDENT_LAUNCH");
  return !(e && std::strcmp(e, "0") == 0);
}

// OXGPU_CLUSTER_REDUCE=dsmem keeps the two-slice in-cluster split-K on the
// distributed-shared-memory reduction that four and eight slices use.
bool cluster_reduce_through_dsmem() {
  const char *e = std::getenv("OXGPU_CLUSTER_REDUCE");
  return e && std::strcmp(e, "dsmem") == 0;
}

struct Staging {
  void *a = nullptr, *bt = nullptr, *c = nullptr;
  size_t a_bytes = 0, bt_bytes = 0, c_bytes = 0;
  cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
  cudaEvent_t a_ready[64] = {}, c_ready[64] = {};  // upload-landed / block-computed, one slot per step
  bool events = false;
};

// Lazily filled per-device facts.  Host threads may race to fill them (the
// values written are the same whoever wins), so every field that is read
// outside g_mutex is an atomic; `ready` is published with release ordering
// after sm_count.
struct DeviceState {
  std::atomic<bool> ready{false};
  std::atomic<int> sm_count{0};
  std::atomic<bool> attr_set[kKinds][kVariants] = {};
  std::atomic<int> max_clusters[kKinds][kVariants] = {};
  Staging staging;
};

DeviceState g_dev[kMaxDevices];
std::mutex g_mutex;          // lazy per-device and driver-entry set-up
std::mutex g_staging_mutex;  // host-buffer entry points (one at a time)

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::atomic<EncodeTiledFn> g_encode{nullptr};

int cuda_fail(cudaError_t e, const char *what) {
  return fail((int)e, std::string(what) + ": " + cudaGetErrorName(e) + ": " + cudaGetErrorString(e));
}

#define OX_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call); \
  } while (0)

int resolve_driver() {
  if (g_encode.load(std::memory_order_acquire)) return OXGPU_OK;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_encode.load(std::memory_order_acquire)) return OXGPU_OK;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000,
                                                   cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return fail(OXGPU_E_NO_DRIVER, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  }
  g_encode.store((EncodeTiledFn)fn, std::memory_order_release);
  return OXGPU_OK;
}

int current_device(int *dev, DeviceState **state) {
  OX_CUDA(cudaGetDevice(dev));
  if (*dev < 0 || *dev >= kMaxDevices) return fail(OXGPU_E_INVALID_ARG, "device index out of range");
  DeviceState &s = g_dev[*dev];
  if (!s.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!s.ready.load(std::memory_order_acquire)) {
      int sms = 0;
      OX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, *dev));
      s.sm_count.store(sms, std::memory_order_relaxed);
      int major = 0;
      OX_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, *dev));
      if (major != 10)
        return fail(OXGPU_E_INVALID_ARG,
                    "this library is built for sm_100a only; the current device is not a B200-class GPU");
      s.ready.store(true, std::memory_order_release);
    }
  }
  *state = &s;
  return OXGPU_OK;
}

int encode_2d(CUtensorMap *map, const void *ptr, int element_bytes, uint64_t dim0, uint64_t dim1,
              uint64_t stride1_bytes, uint32_t box0, uint32_t box1,
              CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
  int st = resolve_driver();
  if (st) return st;
  CUtensorMapDataType dt;
  if (element_bytes == 4) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  else if (element_bytes == 2) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else return fail(OXGPU_E_INVALID_ARG, "element_bytes must be 2 (bf16) or 4 (f32)");
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {stride1_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode.load(std::memory_order_acquire)(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promotion,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char text[200];
    std::snprintf(text, sizeof text,
                  "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, stride %llu, box %u x %u)",
                  (int)r, (unsigned long long)dim0, (unsigned long long)dim1,
                  (unsigned long long)stride1_bytes, box0, box1);
    return fail((int)r, text);
  }
  return OXGPU_OK;
}

const void *kernel_for(int kind, int variant, bool out16 = false) {
#define OX_K(K, BM, BN, CG) ((const void *)umma_gemm_kernel<K, BM, BN, CG>)
  if (out16) {  // bf16 inputs, bf16 C
    switch (variant) {
      case VARIANT_1CTA_128x256: return (const void *)umma_gemm_kernel<0, 128, 256, 1, true>;
      case VARIANT_1CTA_128x128: return (const void *)umma_gemm_kernel<0, 128, 128, 1, true>;
      case VARIANT_2CTA_256x256: return (const void *)umma_gemm_kernel<0, 128, 256, 2, true>;
      case VARIANT_2CTA_512x256: return (const void *)umma_gemm_kernel<0, 256, 256, 2, true>;
    }
    return nullptr;
  }
  if (kind == 0) {
    switch (variant) {
      case VARIANT_1CTA_128x256: return OX_K(0, 128, 256, 1);
      case VARIANT_1CTA_128x128: return OX_K(0, 128, 128, 1);
      case VARIANT_1CTA_256x128: return OX_K(0, 256, 128, 1);
      case VARIANT_2CTA_256x256: return OX_K(0, 128, 256, 2);
      case VARIANT_2CTA_256x128: return OX_K(0, 128, 128, 2);
      case VARIANT_2CTA_512x256: return OX_K(0, 256, 256, 2);
      case VARIANT_1CTA_256x256: return OX_K(0, 256, 256, 1);
      case VARIANT_2CTA_256x512: return (const void *)umma_gemm_kernel<0, 128, 256, 2, false, false, 2>;
    }
  } else {
    switch (variant) {
      case VARIANT_1CTA_128x256: return OX_K(1, 128, 256, 1);
      case VARIANT_1CTA_128x128: return OX_K(1, 128, 128, 1);
      case VARIANT_1CTA_256x128: return OX_K(1, 256, 128, 1);
      case VARIANT_2CTA_256x256: return OX_K(1, 128, 256, 2);
      case VARIANT_2CTA_256x128: return OX_K(1, 128, 128, 2);
      case VARIANT_2CTA_512x256: return OX_K(1, 256, 256, 2);
      case VARIANT_1CTA_256x256: return OX_K(1, 256, 256, 1);
      case VARIANT_2CTA_256x512: return (const void *)umma_gemm_kernel<1, 128, 256, 2, false, false, 2>;
    }
  }
#undef OX_K
  return nullptr;
}

// Fan-out kernels (several destinations per C tile).
const void *fanout_kernel_for(int kind, int variant) {
#define OX_F(K, BM, BN, CG) ((const void *)umma_gemm_kernel<K, BM, BN, CG, false, true>)
  if (kind == 0) {
    switch (variant) {
      case VARIANT_1CTA_128x128: return OX_F(0, 128, 128, 1);
      case VARIANT_2CTA_256x256: return OX_F(0, 128, 256, 2);
      case VARIANT_2CTA_512x256: return OX_F(0, 256, 256, 2);
    }
  } else {
    switch (variant) {
      case VARIANT_1CTA_128x128: return OX_F(1, 128, 128, 1);
      case VARIANT_2CTA_256x256: return OX_F(1, 128, 256, 2);
      case VARIANT_2CTA_512x256: return OX_F(1, 256, 256, 2);
    }
  }
#undef OX_F
  return nullptr;
}

// Kernels with the affine epilogue (alpha, beta, bias).
const void *affine_kernel_for(int kind, int variant) {
#define OX_A(K, BM, BN, CG) ((const void *)umma_gemm_kernel<K, BM, BN, CG, false, false, 1, true>)
  if (kind == 0) {
    switch (variant) {
      case VARIANT_1CTA_128x128: return OX_A(0, 128, 128, 1);
      case VARIANT_2CTA_256x256: return OX_A(0, 128, 256, 2);
      case VARIANT_2CTA_512x256: return OX_A(0, 256, 256, 2);
    }
  } else {
    switch (variant) {
      case VARIANT_1CTA_128x128: return OX_A(1, 128, 128, 1);
      case VARIANT_2CTA_256x256: return OX_A(1, 128, 256, 2);
      case VARIANT_2CTA_512x256: return OX_A(1, 256, 256, 2);
    }
  }
#undef OX_A
  return nullptr;
}

// bf16 inputs, affine epilogue, bf16 C.
const void *affine_out16_kernel_for(int variant) {
  switch (variant) {
    case VARIANT_1CTA_128x128: return (const void *)umma_gemm_kernel<0, 128, 128, 1, true, false, 1, true>;
    case VARIANT_2CTA_256x256: return (const void *)umma_gemm_kernel<0, 128, 256, 2, true, false, 1, true>;
    case VARIANT_2CTA_512x256: return (const void *)umma_gemm_kernel<0, 256, 256, 2, true, false, 1, true>;
  }
  return nullptr;
}

unsigned long long wait_budget_ns() {
  static unsigned long long v = [] {
    const char *e = std::getenv("OXGPU_WAIT_BUDGET_MS");
    double ms = e ? std::atof(e) : 5000.0;
    if (!(ms > 0)) ms = 5000.0;
    return (unsigned long long)(ms * 1e6);
  }();
  return v;
}

struct LaunchPlan {
  int kind, variant, stages, group_m;
  int splits, kb_per_split, split_row_stride;
  int reorder_kb = -1;  // -1: library default
  bool out16 = false;   // bf16 C
  int cluster_splits = 0;  // > 1: split-K across a cluster of that many CTAs (one-CTA 128-row tiles)
  bool fanout = false;     // `p` is a GemmParamsFanout and the fan-out kernel is launched
  bool affine = false;     // the kernel with the affine epilogue is launched
};

// K blocks issued block-major at either end of a tile (two-row-block tiles).
constexpr int kDefaultReorderKb = 3;

// Launch one tcgen05 GEMM.  Maps are either inside `p` (by value) or behind
// p.a_map_ptr / p.b_map_ptr.
int launch_umma(DeviceState &dev, const LaunchPlan &plan, GemmParams &p, int m, int n, int k,
                cudaStream_t stream) {
  const VariantShape shape = variant_shape(plan.variant);
  const void *fn = plan.fanout   ? fanout_kernel_for(plan.kind, plan.variant)
                   : plan.affine && plan.out16 ? affine_out16_kernel_for(plan.variant)
                   : plan.affine ? affine_kernel_for(plan.kind, plan.variant)
                                 : kernel_for(plan.kind, plan.variant, plan.out16);
  if (!fn || shape.cta_group == 0) return fail(OXGPU_E_INVALID_ARG, "unknown kernel variant");
  const int attr_kind = plan.fanout ? 3 + plan.kind : plan.affine ? (plan.out16 ? 7 : 5 + plan.kind) : (plan.out16 ? 2 : plan.kind);
  int stages = plan.stages;
  const int most = variant_max_stages(plan.variant);
  if (stages <= 0 || stages > most) stages = most;
  if (stages < 2) stages = 2;
  if (plan.cluster_splits > 1 && (plan.affine || plan.fanout || plan.out16))
    return fail(OXGPU_E_INVALID_ARG, "in-cluster split-K exists for the plain f32-output kernels only");
  if (plan.cluster_splits > 1) {
    // the partial tile (128 rows x tile_n f32) is parked in the operand ring
    const int need = 128 * shape.tile_n * 4, per = variant_stage_bytes(plan.variant);
    if (stages * per < need) stages = (need + per - 1) / per;
  }
  const int smem = variant_smem_bytes(plan.variant, stages);

  const int kbe = plan.kind == 0 ? 64 : 32;
  p.tiles_m = (m + shape.tile_m - 1) / shape.tile_m;
  p.tiles_n = (n + shape.tile_n - 1) / shape.tile_n;
  p.num_k_blocks = (k + kbe - 1) / kbe;
  p.stages = stages;
  // Group height of the tile order.  The reference uses 16 tile-rows of 128 =
  // 2048 rows of A; the same 2048 rows are 8 tile-rows of 256 and 4 of 512.  The
  // A panels of a group are what the next tiles of the walk reuse, so they should
  // survive in L2 beside the B^T panels streaming past: with K = 8192 that is
  // 32 MiB of A.  Measured with the queue-driven schedule, 512-row tiles, sustained
  // clocks, fraction of the vendor library doing the same work: M=32768 N=65536
  // K=8192 0.985 / 0.999 / 0.982 / 0.958 with 3 / 4 / 6 / 8 tile-rows (0.825 with
  // 16); 8192 x 8192 x 28672 0.993 / 0.987 / 0.954 with 4 / 6 / 8.
  p.group_m = plan.group_m > 0 ? plan.group_m : (shape.tile_m >= 512 ? 4 : shape.tile_m >= 256 ? 8 : 16);
  p.k_block_elems = kbe;
  p.splits = plan.splits > 0 ? plan.splits : 1;
  p.kb_per_split = plan.splits > 1 ? plan.kb_per_split : p.num_k_blocks;
  p.split_row_stride = plan.split_row_stride;
  p.reorder_kb = plan.reorder_kb >= 0 ? plan.reorder_kb : kDefaultReorderKb;
  // C is written once and never read by this kernel: its stores are marked
  // evict-first so the output stream does not push operand tiles out of L2
  // (worth 6 points on 32768^2-sized outputs, nothing at 8192^3).
  // (Operands are kept with evict-last priority when both fit a few times over
  // in L2-sized waves: +1 point up to 576 MiB of A + B^T, -3 points at 1 GiB.)
  const double operand_bytes = ((double)m * k + (double)n * k) * (plan.kind == 0 ? 2 : 4);
  p.hint_a = p.hint_b = operand_bytes <= 768.0 * 1024 * 1024 ? 2 : 0;
  p.hint_c = 1;
  // An operand whose every row feeds one or two tiles only (B^T when M is a tile
  // row or two, A when N is) is streamed, not reused: its loads are marked
  // evict-first, so they recycle their own lines instead of pushing out the other
  // operand -- or whatever dirty lines L2 holds, whose write-back would then share
  // HBM with the stream -- and the operand that every tile re-reads is kept with
  // evict-last.  With L2 full of dirty lines (the bench's flush), 128 x 8192 x 8192:
  // 43.0 -> 36.9 us (the vendor library: 36.9), 128 x 28672 x 8192: 112.7 -> 104.4
  // (106.6), 128 x 8192 x 28672: 104.4 -> 94.3 (92.3).
  const int rows_of_tiles = (m + shape.tile_m - 1) / shape.tile_m, cols_of_tiles = (n + shape.tile_n - 1) / shape.tile_n;
  if (rows_of_tiles <= 2 && cols_of_tiles > 2) {
    p.hint_a = 2;
    p.hint_b = 1;
  } else if (cols_of_tiles <= 2 && rows_of_tiles > 2) {
    p.hint_a = 1;
    p.hint_b = 2;
  }
  p.wait_budget_ns = wait_budget_ns();

  std::atomic<bool> &attr = dev.attr_set[attr_kind][plan.variant];
  if (!attr.load(std::memory_order_acquire)) {
    OX_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem));
    attr.store(true, std::memory_order_release);
  }

  const long long work = (long long)p.tiles_m * p.tiles_n * p.splits;
  if (work <= 0 || work > 0x7fffffffLL) return fail(OXGPU_E_TOO_LARGE, "too many tiles");
  if ((long long)p.group_m * p.tiles_n > 0x7fffffffLL) return fail(OXGPU_E_TOO_LARGE, "too many tiles in a group of tile rows");
  p.div_splits = make_fast_divisor(p.splits, work);
  p.div_per_group = make_fast_divisor(p.group_m * p.tiles_n, work);
  p.div_group = make_fast_divisor(p.group_m, work);

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreadsPerCta, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  // attrs[0]: the kernel may start while the kernel before it in the stream is
  // still running (its set-up touches no global memory and it waits for that
  // kernel before anything else); attrs[1]: the cluster shape, when there is one.
  cudaLaunchAttribute attrs[2];
  const unsigned base_attrs = dependent_launch_enabled() ? 1u : 0u;
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchAttribute *const cluster_attr = attrs + base_attrs;
  cfg.attrs = attrs;
  cfg.numAttrs = base_attrs;
  if (shape.cta_group == 2) {
    cluster_attr->id = cudaLaunchAttributeClusterDimension;
    cluster_attr->val.clusterDim.x = 2;
    cluster_attr->val.clusterDim.y = 1;
    cluster_attr->val.clusterDim.z = 1;
    cfg.numAttrs = base_attrs + 1;
    std::atomic<int> &cached = dev.max_clusters[attr_kind][plan.variant];
    int maxc = cached.load(std::memory_order_relaxed);
    if (maxc == 0) {
      cfg.gridDim = dim3(2 * (dev.sm_count / 2), 1, 1);
      int nc = 0;
      OX_CUDA(cudaOccupancyMaxActiveClusters(&nc, fn, &cfg));
      if (nc <= 0) return fail(OXGPU_E_INVALID_ARG, "no CTA pair of this variant fits on the device");
      maxc = nc;
      cached.store(nc, std::memory_order_relaxed);
    }
    long long clusters = work < maxc ? work : maxc;
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  } else if (plan.cluster_splits > 1) {
    // one work item per CTA: cluster c = tile c, CTA rank = K slice
    cluster_attr->id = cudaLaunchAttributeClusterDimension;
    cluster_attr->val.clusterDim.x = (unsigned)plan.cluster_splits;
    cluster_attr->val.clusterDim.y = 1;
    cluster_attr->val.clusterDim.z = 1;
    cfg.numAttrs = base_attrs + 1;
    cfg.gridDim = dim3((unsigned)work, 1, 1);
    // Two slices: the tile of C is zeroed during the main loop and both CTAs add
    // their partial tiles to it with TMA reductions (C then stays in L2 between the
    // zeroing and the additions, so it is not marked evict-first).  More slices: the
    // partial tiles are summed in a fixed order through distributed shared memory.
    p.cluster_reduce = plan.cluster_splits == 2 && !cluster_reduce_through_dsmem() ? 2 : 1;
    if (p.cluster_reduce == 2) p.hint_c = 0;
  } else {
    const int sms = dev.sm_count;
    long long ctas = work < sms ? work : sms;
    cfg.gridDim = dim3((unsigned)ctas, 1, 1);
  }
  // One wave (every tile has its own CTA or CTA pair, in-cluster split-K included):
  // each operand byte is wanted by all its readers at about the same time and
  // never again, so both operands are loaded evict-first.  Their lines then
  // recycle among themselves instead of displacing what L2 held before the launch;
  // when that is dirty (another kernel's output, or the bench's flush) its
  // write-back would share HBM with the loads.  L2 flushed, 512 x 4096 x 4096: 26.0
  // -> 23.0 us, 1024 x 1024 x 8192: 27.0 -> 24.8; no change on the other one-wave
  // shapes measured (128 / 256 / 384 / 512 x 8192 x 8192, 2048^3, 128 x 4096 x 4096).
  if (work <= (long long)cfg.gridDim.x / (plan.cluster_splits > 1 ? 1 : shape.cta_group)) p.hint_a = p.hint_b = 1;
  // Problems that keep every cluster busy for several tiles take their tiles
  // from a queue in walk order instead of a fixed stride, so the tiles in flight
  // stay a compact window of the walk (see TileFeed).  Split-K keeps the static
  // walk: its work items are tied to cluster ranks or to workspace slices.
  p.sched_slot_plus1 = 0;
  if (p.splits == 1 && plan.cluster_splits <= 1 && work >= 2LL * cfg.gridDim.x / shape.cta_group &&
      !static_schedule_forced())
    p.sched_slot_plus1 = 1 + (int)(g_sched_seq.fetch_add(1, std::memory_order_relaxed) % (unsigned)kSchedSlots);
  void *args[1] = {(void *)&p};
  OX_CUDA(cudaLaunchKernelExC(&cfg, fn, args));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_buffers(const void *a, const void *bt, const float *c, int m, int n, int k, int64_t lda,
                  int64_t ldb, int64_t ldc, int esize) {
  if (!a || !bt || !c) return fail(OXGPU_E_INVALID_ARG, "null operand pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(OXGPU_E_INVALID_ARG, "M, N and K must be positive");
  if (lda < k || ldb < k || ldc < n)
    return fail(OXGPU_E_INVALID_ARG, "leading dimension smaller than the row length");
  if (!aligned16(a) || !aligned16(bt) || !aligned16(c))
    return fail(OXGPU_E_ALIGN, "operand pointers must be 16-byte aligned");
  if ((lda * esize) % 16 || (ldb * esize) % 16 || (ldc * 4) % 16)
    return fail(OXGPU_E_ALIGN, "leading dimensions must be multiples of 16 bytes");
  if (((int64_t)k * esize) % 16)
    return fail(OXGPU_E_SHAPE, "K must make a row a multiple of 16 bytes (8 bf16 / 4 f32)");
  return OXGPU_OK;
}

// Slices of the in-cluster split-K when the caller names the variant but not
// the slice count: as many as fill the GPU once, a power of two, at most 8, each
// at least 32 K blocks long.
int auto_cluster_slices(int sm_count, long long tiles, int num_kb) {
  int s = 8;
  while (s > 1 && (tiles * s > sm_count || num_kb / s < 32)) s >>= 1;
  return s;
}

// Variant choice for the buffer entry points.  Large problems take the CTA-pair
// 512x256 tile (least shared-memory and L2 traffic per flop).  Everything smaller
// is decided by an estimate of each candidate's time in SM clocks at boost:
// waves of tiles x (K blocks x clocks per K block + a fixed cost per tile), never
// less than the problem's bytes at the HBM rate, plus the reduction tail of an
// in-cluster split.  The clocks per K block are measured ones (one wave of each
// tile at K = 8192, L2 flushed): what a CTA sustains is set by how fast it takes
// its operand bytes from L2, 40-70 bytes per clock depending on the tile.  The
// tall pair tiles need M to fill at least three quarters of them (with M = 128 a
// 512-row pair tile would do four times the work: 174 us instead of 111 us at
// 128 x 28672 x 8192).  What the estimate changed against a fixed cascade
// (measured, L2 flushed, us): 384 x 8192 x 8192 88 -> 55 (one wave of 256x256
// pair tiles), 512 x 8192 x 8192 88 -> 55, 2048^3 32 -> 25, 256 x 8192 x 8192
// 50 -> 47 (128x256 tiles, two slices), 128 x 4096 x 4096 23.5 -> 21.4 (four
// slices).
int choose_variant(const DeviceState &dev, int m, int n, int k, int kbe, int esize, int *cluster_slices) {
  auto tiles = [&](int tm, int tn) { return (long long)((m + tm - 1) / tm) * ((n + tn - 1) / tn); };
  const int sms = dev.sm_count, pairs = sms / 2;
  auto fills = [&](int tm) { return 4LL * m >= 3LL * (long long)((m + tm - 1) / tm) * tm; };
  *cluster_slices = 0;
  // The 512x256 pair tile moves a quarter less operand data per flop than
  // 256x256 (48 instead of 64 bytes per clock per SM at full tensor rate), which
  // is what limits the kernel at boost clocks: 95 % against 91.5 % of cuBLAS at
  // bf16 8192^3, even though it cannot double-buffer its accumulator.
  if (fills(512) && tiles(512, 256) >= pairs) return VARIANT_2CTA_512x256;

  const int num_kb = (k + kbe - 1) / kbe;
  const double hbm_bytes_per_clk = 3282.0;  // 6.45 TB/s at 1.965 GHz, all SMs together
  const double floor_clk = (((double)m + n) * k * esize + (double)m * n * 4.0) / hbm_bytes_per_clk;
  const double tile_clk = 8000.0;           // fill latency + accumulator drain of one tile
  const double slice_tail_clk = 3000.0;     // per slice of an in-cluster split: barrier + cross-CTA sum
  struct Candidate {
    int variant, tile_m, tile_n, ctas_per_tile;
    double kb_clk;  // clocks per K block of one tile
    bool cluster_split;
  };
  const Candidate candidates[] = {
      {VARIANT_2CTA_512x256, 512, 256, 2, 1340, false}, {VARIANT_2CTA_256x256, 256, 256, 2, 700, false},
      {VARIANT_2CTA_256x128, 256, 128, 2, 620, false},  {VARIANT_1CTA_128x256, 128, 256, 1, 820, false},
      {VARIANT_1CTA_128x128, 128, 128, 1, 600, false},  {VARIANT_CLUSTER_SPLITK_128x128, 128, 128, 1, 600, true},
      {VARIANT_CLUSTER_SPLITK_128x256, 128, 256, 1, 820, true},
  };
  int best = VARIANT_1CTA_128x128;
  double best_clk = 0;
  auto consider = [&](int variant, double clk, int slices) {
    if (best_clk == 0 || clk < best_clk) {
      best_clk = clk;
      best = variant;
      *cluster_slices = slices;
    }
  };
  for (const Candidate &c : candidates) {
    if (c.tile_m > 128 && !fills(c.tile_m)) continue;
    const long long t = tiles(c.tile_m, c.tile_n);
    if (c.cluster_split) {
      if (k < 2048) continue;
      for (int s = 2; s <= 8; s *= 2) {  // one wave, every slice at least 16 K blocks
        if (t * s > sms || num_kb / s < 16) break;
        consider(c.variant, std::max((double)((num_kb + s - 1) / s) * c.kb_clk + tile_clk, floor_clk) + slice_tail_clk * s, s);
      }
    } else {
      const long long units = sms / c.ctas_per_tile;
      const long long waves = (t + units - 1) / units;
      consider(c.variant, std::max((double)waves * (num_kb * c.kb_clk + tile_clk), floor_clk), 0);
    }
  }
  return best;
}

int gemm_buffers(int kind, const void *a, const void *bt, float *c, int m, int n, int k, int64_t lda,
                 int64_t ldb, int64_t ldc, unsigned flags, void *workspace, size_t workspace_bytes,
                 cudaStream_t stream, bool out16 = false) {
  const int esize = kind == 0 ? 2 : 4;
  int st = check_buffers(a, bt, c, m, n, k, lda, ldb, ldc, esize);
  if (st) return st;
  if (out16 && (ldc * 2) % 16) return fail(OXGPU_E_ALIGN, "bf16 C needs ldc to be a multiple of 8");
  int dev_index;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;

  int variant = (int)(flags & 0xffu);
  const int stages = (int)((flags >> 8) & 0xfu);
  const int group_m = (int)((flags >> 12) & 0xffu);
  int splits = (int)((flags >> 20) & 0xffu);
  const bool splitk = variant == VARIANT_SPLITK;
  const bool was_auto = variant == VARIANT_AUTO;
  if (was_auto) {
    int model_slices = 0;
    variant = choose_variant(*dev, m, n, k, kind == 0 ? 64 : 32, esize, &model_slices);
    if (model_slices > 0 && splits <= 0) splits = model_slices;
    if (out16 && (variant == VARIANT_CLUSTER_SPLITK_128x256 || variant == VARIANT_CLUSTER_SPLITK_128x128))
      variant = VARIANT_1CTA_128x128;  // the cluster reduction writes f32 only
  }
  if (splitk) variant = VARIANT_1CTA_128x128;
  int cluster_splits = 0;
  if (variant == VARIANT_CLUSTER_SPLITK_128x256 || variant == VARIANT_CLUSTER_SPLITK_128x128) {
    if (out16) return fail(OXGPU_E_INVALID_ARG, "cluster split-K writes f32 C only");
    const int tile_n = variant == VARIANT_CLUSTER_SPLITK_128x256 ? 256 : 128;
    variant = tile_n == 256 ? VARIANT_1CTA_128x256 : VARIANT_1CTA_128x128;
    const int num_kb = (k + (kind == 0 ? 64 : 32) - 1) / (kind == 0 ? 64 : 32);
    const long long tiles = (long long)((m + 127) / 128) * ((n + tile_n - 1) / tile_n);
    int s = splits;
    if (s <= 0) s = auto_cluster_slices(dev->sm_count, tiles, num_kb);
    while (s > 1 && (num_kb + s - 1) / s * (s - 1) >= num_kb) s >>= 1;  // every slice gets a K block
    if (s != 1 && s != 2 && s != 4 && s != 8)
      return fail(OXGPU_E_INVALID_ARG, "cluster split-K takes 2, 4 or 8 slices");
    cluster_splits = s;  // 1: nothing to split, plain kernel
  }
  if (out16 && !splitk && !kernel_for(0, variant, true)) {
    if (!was_auto) return fail(OXGPU_E_INVALID_ARG, "this variant has no bf16-output kernel");
    variant = VARIANT_1CTA_128x128;
  }
  if (variant_shape(variant).cta_group == 0)
    return fail(OXGPU_E_INVALID_ARG, "unknown variant in flags");
  const VariantShape shape = variant_shape(variant);
  const int kbe = kind == 0 ? 64 : 32;

  LaunchPlan plan{kind, variant, stages, group_m, 1, 0, 0};
  if (cluster_splits > 1) {
    const int num_kb = (k + kbe - 1) / kbe;
    plan.cluster_splits = cluster_splits;
    plan.splits = cluster_splits;
    plan.kb_per_split = (num_kb + cluster_splits - 1) / cluster_splits;
  }
  const int reorder_field = (int)((flags >> 28) & 0xfu);  // 0 default, 15 off, else that many K blocks
  plan.reorder_kb = reorder_field == 0 ? -1 : (reorder_field == 15 ? 0 : reorder_field);
  GemmParams p;
  std::memset(&p, 0, sizeof p);
  const int a_box = shape.cta_a_rows, b_box = shape.cta_b_rows;
  p.a_box_rows = a_box;
  p.b_box_rows = b_box;
  if ((st = encode_2d(&p.map_a, a, esize, (uint64_t)k, (uint64_t)m, (uint64_t)lda * esize, kbe, a_box)))
    return st;
  if ((st = encode_2d(&p.map_b, bt, esize, (uint64_t)k, (uint64_t)n, (uint64_t)ldb * esize, kbe, b_box)))
    return st;

  if (out16) {
    if (splitk) return fail(OXGPU_E_INVALID_ARG, "split-K writes f32 partial tiles; no bf16 output");
    plan.out16 = true;
    if ((st = encode_2d(&p.map_c, c, 2, (uint64_t)n, (uint64_t)m, (uint64_t)ldc * 2, 64, 32)))
      return st;
    return launch_umma(*dev, plan, p, m, n, k, stream);
  }
  if (!splitk) {
    if ((st = encode_2d(&p.map_c, c, 4, (uint64_t)n, (uint64_t)m, (uint64_t)ldc * 4, 32, 32)))
      return st;
    p.c_ptr = c;
    p.c_ld = ldc;
    p.c_rows = m;
    p.c_cols = n;
    return launch_umma(*dev, plan, p, m, n, k, stream);
  }

  // split-K: partial tiles go to the workspace [splits][m_pad][n4*4], then a
  // deterministic reduction writes C.
  if (n % 4) return fail(OXGPU_E_SHAPE, "split-K needs N to be a multiple of 4");
  const int num_kb = (k + kbe - 1) / kbe;
  if (splits <= 0) {
    long long tiles = (long long)((m + 127) / 128) * ((n + 127) / 128);
    splits = (int)((2LL * dev->sm_count + tiles - 1) / tiles);
    if (splits > 16) splits = 16;
  }
  if (splits > num_kb) splits = num_kb;
  if (splits < 1) splits = 1;
  const int kb_per = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per - 1) / kb_per;  // every slice gets at least one K block
  const int m_pad = ((m + 127) / 128) * 128;
  const size_t need = (size_t)splits * m_pad * (size_t)n * sizeof(float);
  if (!workspace || workspace_bytes < need || !aligned16(workspace))
    return fail(OXGPU_E_INVALID_ARG, "split-K workspace missing, misaligned or too small");
  if ((st = encode_2d(&p.map_c, workspace, 4, (uint64_t)n, (uint64_t)splits * m_pad, (uint64_t)n * 4,
                      32, 32)))
    return st;
  plan.splits = splits;
  plan.kb_per_split = kb_per;
  plan.split_row_stride = m_pad;
  if ((st = launch_umma(*dev, plan, p, m, n, k, stream))) return st;
  const size_t total = (size_t)m * (n / 4);
  int blocks = (int)((total + 255) / 256);
  if (blocks > dev->sm_count * 8) blocks = dev->sm_count * 8;
  splitk_reduce_kernel<<<blocks, 256, 0, stream>>>((const float4 *)workspace, c, m, n, ldc, splits,
                                                   (int64_t)m_pad);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

// The three tile shapes the fan-out and affine kernels exist for.
int choose_large_tile_variant(const DeviceState &dev, int m, int n) {
  auto tiles = [&](int tm, int tn) { return (long long)((m + tm - 1) / tm) * ((n + tn - 1) / tn); };
  const int pairs = dev.sm_count / 2;
  return tiles(512, 256) >= pairs   ? VARIANT_2CTA_512x256
         : tiles(256, 256) >= pairs ? VARIANT_2CTA_256x256
                                    : VARIANT_1CTA_128x128;
}

// GEMM whose C tiles go to several destinations (see GemmParamsFanout).
int gemm_fanout(int kind, const void *a, const void *bt, float *const *dests, int n_dests, int m, int n,
                int k, int64_t lda, int64_t ldb, int64_t ldc, unsigned flags, cudaStream_t stream) {
  const int esize = kind == 0 ? 2 : 4;
  if (!dests || n_dests < 1 || n_dests > kMaxFanout)
    return fail(OXGPU_E_INVALID_ARG, "the number of destinations must be between 1 and 8");
  int st;
  for (int d = 0; d < n_dests; d++)
    if ((st = check_buffers(a, bt, dests[d], m, n, k, lda, ldb, ldc, esize))) return st;
  int dev_index;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;

  int variant = (int)(flags & 0xffu);
  if (variant == VARIANT_AUTO) variant = choose_large_tile_variant(*dev, m, n);
  if (!fanout_kernel_for(kind, variant))
    return fail(OXGPU_E_INVALID_ARG, "this variant has no fan-out kernel (use 1cta_128x128, 2cta_256x256 or 2cta_512x256)");
  const VariantShape shape = variant_shape(variant);
  const int kbe = kind == 0 ? 64 : 32;

  LaunchPlan plan{kind, variant, (int)((flags >> 8) & 0xfu), (int)((flags >> 12) & 0xffu), 1, 0, 0};
  const int reorder_field = (int)((flags >> 28) & 0xfu);
  plan.reorder_kb = reorder_field == 0 ? -1 : (reorder_field == 15 ? 0 : reorder_field);
  plan.fanout = true;
  GemmParamsFanout p;
  std::memset((void *)&p, 0, sizeof p);
  p.a_box_rows = shape.cta_a_rows;
  p.b_box_rows = shape.cta_b_rows;
  if ((st = encode_2d(&p.map_a, a, esize, (uint64_t)k, (uint64_t)m, (uint64_t)lda * esize, kbe, p.a_box_rows)))
    return st;
  if ((st = encode_2d(&p.map_b, bt, esize, (uint64_t)k, (uint64_t)n, (uint64_t)ldb * esize, kbe, p.b_box_rows)))
    return st;
  for (int d = 0; d < n_dests; d++)
    if ((st = encode_2d(&p.dest_maps[d], dests[d], 4, (uint64_t)n, (uint64_t)m, (uint64_t)ldc * 4, 32, 32)))
      return st;
  p.n_dests = n_dests;
  return launch_umma(*dev, plan, p, m, n, k, stream);
}

// C = alpha * (A B) + beta * C_in + bias in the GEMM's own epilogue.
int gemm_affine(int kind, const void *a, const void *bt, float *c, int m, int n, int k, int64_t lda,
                int64_t ldb, int64_t ldc, const oxgpu_epilogue *ep, unsigned flags, cudaStream_t stream,
                bool out16 = false) {
  const int esize = kind == 0 ? 2 : 4;
  if (!ep) return fail(OXGPU_E_INVALID_ARG, "null epilogue description");
  int st = check_buffers(a, bt, c, m, n, k, lda, ldb, ldc, esize);
  if (st) return st;
  if (out16 && (ldc * 2) % 16) return fail(OXGPU_E_ALIGN, "bf16 C needs ldc to be a multiple of 8");
  if (ep->bias && !aligned16(ep->bias)) return fail(OXGPU_E_ALIGN, "bias must be 16-byte aligned");
  if (ep->beta != 0.0f) {
    if (!ep->c_in) return fail(OXGPU_E_INVALID_ARG, "beta != 0 needs c_in");
    if (!aligned16(ep->c_in) || (ep->ldc_in * 4) % 16 || ep->ldc_in < n)
      return fail(OXGPU_E_ALIGN, "c_in must be 16-byte aligned with a leading dimension that is a multiple of 4 and at least N");
  }
  int dev_index;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  int variant = (int)(flags & 0xffu);
  if (variant == VARIANT_AUTO) variant = choose_large_tile_variant(*dev, m, n);
  if (out16 ? !affine_out16_kernel_for(variant) : !affine_kernel_for(kind, variant))
    return fail(OXGPU_E_INVALID_ARG, "this variant has no affine-epilogue kernel (use 1cta_128x128, 2cta_256x256 or 2cta_512x256)");
  const VariantShape shape = variant_shape(variant);
  const int kbe = kind == 0 ? 64 : 32;
  LaunchPlan plan{kind, variant, (int)((flags >> 8) & 0xfu), (int)((flags >> 12) & 0xffu), 1, 0, 0};
  const int reorder_field = (int)((flags >> 28) & 0xfu);
  plan.reorder_kb = reorder_field == 0 ? -1 : (reorder_field == 15 ? 0 : reorder_field);
  plan.affine = true;
  plan.out16 = out16;
  GemmParams p;
  std::memset(&p, 0, sizeof p);
  p.a_box_rows = shape.cta_a_rows;
  p.b_box_rows = shape.cta_b_rows;
  if ((st = encode_2d(&p.map_a, a, esize, (uint64_t)k, (uint64_t)m, (uint64_t)lda * esize, kbe, p.a_box_rows)))
    return st;
  if ((st = encode_2d(&p.map_b, bt, esize, (uint64_t)k, (uint64_t)n, (uint64_t)ldb * esize, kbe, p.b_box_rows)))
    return st;
  if (out16) st = encode_2d(&p.map_c, c, 2, (uint64_t)n, (uint64_t)m, (uint64_t)ldc * 2, 64, 32);
  else st = encode_2d(&p.map_c, c, 4, (uint64_t)n, (uint64_t)m, (uint64_t)ldc * 4, 32, 32);
  if (st) return st;
  p.c_ptr = c;
  p.c_ld = ldc;
  p.c_rows = m;
  p.c_cols = n;
  p.alpha = ep->alpha;
  p.beta = ep->beta;
  p.bias = ep->bias;
  p.c_in = ep->beta != 0.0f ? ep->c_in : nullptr;
  p.c_in_ld = ep->ldc_in;
  return launch_umma(*dev, plan, p, m, n, k, stream);
}

int ensure_staging(Staging &s, size_t a_bytes, size_t bt_bytes, size_t c_bytes) {
  if (!s.in) {
    OX_CUDA(cudaStreamCreateWithFlags(&s.in, cudaStreamNonBlocking));
    OX_CUDA(cudaStreamCreateWithFlags(&s.compute, cudaStreamNonBlocking));
    OX_CUDA(cudaStreamCreateWithFlags(&s.out, cudaStreamNonBlocking));
  }
  if (!s.events) {
    for (int i = 0; i < 64; i++) {
      OX_CUDA(cudaEventCreateWithFlags(&s.a_ready[i], cudaEventDisableTiming));
      OX_CUDA(cudaEventCreateWithFlags(&s.c_ready[i], cudaEventDisableTiming));
    }
    s.events = true;
  }
  auto grow = [](void **ptr, size_t *have, size_t want) -> cudaError_t {
    if (*have >= want) return cudaSuccess;
    if (*ptr) {
      cudaError_t e = cudaFree(*ptr);
      if (e != cudaSuccess) return e;
      *ptr = nullptr;
      *have = 0;
    }
    cudaError_t e = cudaMalloc(ptr, want);
    if (e == cudaSuccess) *have = want;
    return e;
  };
  OX_CUDA(grow(&s.a, &s.a_bytes, a_bytes));
  OX_CUDA(grow(&s.bt, &s.bt_bytes, bt_bytes));
  OX_CUDA(grow(&s.c, &s.c_bytes, c_bytes));
  return OXGPU_OK;
}

// Host-buffer GEMM.  PCIe is the limit (operands up, C down), so the schedule
// keeps both directions busy: A and B^T go up in row blocks, alternating
// A0 B0 A1 B1 ..., and as soon as a block lands the library computes every part
// of C that has just become computable (a new block row of C against the B^T
// blocks already present, or a new block column against the A blocks already
// present) and starts its download.  Uploads, GEMMs and downloads run on three
// streams chained by events.
int gemm_host(int kind, const void *a_host, const void *bt_host, void *c_host, int m, int n, int k,
              unsigned flags, bool out16 = false) {
  const int esize = kind == 0 ? 2 : 4;
  const size_t csize = out16 ? 2 : 4;  // bytes per element of C
  if (!a_host || !bt_host || !c_host) return fail(OXGPU_E_INVALID_ARG, "null host pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(OXGPU_E_INVALID_ARG, "M, N and K must be positive");
  if (((int64_t)k * esize) % 16 || n % 4)
    return fail(OXGPU_E_SHAPE, "rows of A/B^T must be multiples of 16 bytes and N a multiple of 4");
  if (out16 && n % 8) return fail(OXGPU_E_SHAPE, "bf16 C needs N to be a multiple of 8");
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  Staging &s = dev->staging;
  std::lock_guard<std::mutex> lock(g_staging_mutex);
  const size_t a_bytes = (size_t)m * k * esize, bt_bytes = (size_t)n * k * esize;
  const size_t c_bytes = (size_t)m * n * csize;
  if ((st = ensure_staging(s, a_bytes, bt_bytes, c_bytes))) return st;

  // Row blocks: multiples of 256 rows, about 6 per operand (at most 16).  The
  // part of C that can be computed grows with the square of the fraction of the
  // operands that has landed, so the download trails the upload by design; smaller
  // blocks shorten what is left to compute and send after the last upload, but
  // every copy costs a start-up gap on its stream (8192^3, blocks per operand ->
  // ms: 3 -> 7.43, 4 -> 7.19, 6 -> 6.99, 8 -> 7.28, 12 -> 7.19, 16 -> 7.63).
  auto block_rows_of = [](int rows) {
    int b = ((rows / 6 + 255) / 256) * 256;
    if (b < 256) b = 256;
    while ((rows + b - 1) / b > 16) b *= 2;
    return b;
  };
  const int a_rows = block_rows_of(m), b_rows = block_rows_of(n);
  const int na = (m + a_rows - 1) / a_rows, nb = (n + b_rows - 1) / b_rows;
  const size_t row_bytes = (size_t)k * esize;
  int a_up = 0, b_up = 0, ev = 0;  // blocks uploaded so far; next event slot
  // On any error the copies and kernels already queued are waited for before the
  // call returns: they read the caller's A and B^T and write the caller's C, and
  // the staging buffers must be idle before the next call reuses them.
  struct Drain {
    Staging &s;
    bool armed = true;
    ~Drain() {
      if (!armed) return;
      cudaStreamSynchronize(s.in);
      cudaStreamSynchronize(s.compute);
      cudaStreamSynchronize(s.out);
      cudaGetLastError();
    }
  } drain{s};

  // compute C[r0:r0+rows, c0:c0+cols] on the device and send it down
  auto emit = [&](int r0, int rows, int c0, int cols, cudaEvent_t ready) -> int {
    OX_CUDA(cudaStreamWaitEvent(s.compute, ready, 0));
    const char *a_dev = (const char *)s.a + (size_t)r0 * row_bytes;
    const char *b_dev = (const char *)s.bt + (size_t)c0 * row_bytes;
    char *c_dev = (char *)s.c + ((size_t)r0 * n + c0) * csize;
    int st2 = gemm_buffers(kind, a_dev, b_dev, (float *)c_dev, rows, cols, k, k, k, n, flags, nullptr, 0, s.compute,
                           out16);
    if (st2) return st2;
    cudaEvent_t done = s.c_ready[ev % 64];
    OX_CUDA(cudaEventRecord(done, s.compute));
    OX_CUDA(cudaStreamWaitEvent(s.out, done, 0));
    OX_CUDA(cudaMemcpy2DAsync((char *)c_host + ((size_t)r0 * n + c0) * csize, (size_t)n * csize, c_dev,
                              (size_t)n * csize, (size_t)cols * csize, (size_t)rows, cudaMemcpyDeviceToHost,
                              s.out));
    return OXGPU_OK;
  };

  // Two passes over the same sequence of steps: first every upload is queued (with
  // its event), then every product and download.  Queued that way the upload
  // stream never waits for the host thread, which needs tens of microseconds per
  // step for the tensor maps, the launch and the event calls of a product.
  for (int pass = 0; pass < 2; pass++) {
    a_up = b_up = ev = 0;
    while (a_up < na || b_up < nb) {
      // next upload: keep the two operands' progress balanced (as fractions)
      const bool take_a = b_up >= nb || (a_up < na && (long long)a_up * nb <= (long long)b_up * na);
      cudaEvent_t up = s.a_ready[ev % 64];
      if (take_a) {
        const int r0 = a_up * a_rows, rows = m - r0 < a_rows ? m - r0 : a_rows;
        if (pass == 0) {
          OX_CUDA(cudaMemcpyAsync((char *)s.a + (size_t)r0 * row_bytes, (const char *)a_host + (size_t)r0 * row_bytes,
                                  (size_t)rows * row_bytes, cudaMemcpyHostToDevice, s.in));
          OX_CUDA(cudaEventRecord(up, s.in));
        }
        a_up++;
        if (pass == 1 && b_up > 0) {  // new block row of C against every B^T block present
          const int cols = b_up * b_rows < n ? b_up * b_rows : n;
          if ((st = emit(r0, rows, 0, cols, up))) return st;
        }
      } else {
        const int c0 = b_up * b_rows, cols = n - c0 < b_rows ? n - c0 : b_rows;
        if (pass == 0) {
          OX_CUDA(cudaMemcpyAsync((char *)s.bt + (size_t)c0 * row_bytes, (const char *)bt_host + (size_t)c0 * row_bytes,
                                  (size_t)cols * row_bytes, cudaMemcpyHostToDevice, s.in));
          OX_CUDA(cudaEventRecord(up, s.in));
        }
        b_up++;
        if (pass == 1 && a_up > 0) {  // new block column of C against every A block present
          const int rows = a_up * a_rows < m ? a_up * a_rows : m;
          if ((st = emit(0, rows, c0, cols, up))) return st;
        }
      }
      ev++;
    }
  }
  OX_CUDA(cudaStreamSynchronize(s.out));
  OX_CUDA(cudaStreamSynchronize(s.in));
  drain.armed = false;
  return OXGPU_OK;
}

}  // namespace
}  // namespace oxgpu

using namespace oxgpu;

extern "C" {

int oxgpu_b200_encode_tmap_2d(void *map_out, const void *device_ptr, int element_bytes,
                              uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes, uint32_t box0,
                              uint32_t box1) {
  if (!map_out || !device_ptr) return fail(OXGPU_E_INVALID_ARG, "null argument");
  if ((reinterpret_cast<uintptr_t>(map_out) & 63u) != 0)
    return fail(OXGPU_E_ALIGN, "a CUtensorMap must be 64-byte aligned");
  return encode_2d((CUtensorMap *)map_out, device_ptr, element_bytes, dim0, dim1, stride1_bytes, box0,
                   box1);
}

int oxgpu_b200_gemm_tmap(const char *name, uint64_t a_tmap, uint64_t b_tmap, uint64_t c, int m,
                         int n, int k, void *stream) {
  const CatalogEntry *e = find_entry(name);
  if (!e) return fail(OXGPU_E_UNKNOWN_KERNEL, std::string("no kernel named ") + (name ? name : "(null)"));
  if (!a_tmap || !b_tmap || !c) return fail(OXGPU_E_INVALID_ARG, "null device pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(OXGPU_E_INVALID_ARG, "M, N and K must be positive");
  if ((a_tmap & 63u) || (b_tmap & 63u))
    return fail(OXGPU_E_ALIGN, "tensor maps must be 64-byte aligned in device memory");
  if (c & 15u) return fail(OXGPU_E_ALIGN, "C must be 16-byte aligned");
  const oxgpu_tile_config &t = e->tile;
  // The reference refuses these sizes before launching (bench/bench.py:247-250).
  if (m % t.bm || n % t.bn || k % t.bk) {
    char text[160];
    std::snprintf(text, sizeof text,
                  "matmul size %dx%dx%d must be divisible by CTA %dx%d and BK %d", m, n, k, t.bm,
                  t.bn, t.bk);
    return fail(OXGPU_E_SHAPE, text);
  }
  // The caller's maps fix the rows one load brings (the entry's bm rows of A,
  // bn rows of B^T); any tile whose per-CTA rows are multiples of those boxes
  // can serve the entry.  In order of operand traffic per flop:
  //  * 64/128-row A box: the CTA pair with two 256-column blocks (256 x 512 per
  //    pair): each CTA stages 128 rows of A and 256 CONTIGUOUS rows of B^T, which
  //    the reference's 256-row B^T box delivers in one load (48 bytes of operand
  //    per clock per SM at full rate, as the library's own 512 x 256 tile);
  //  * 256-row A box with a 128-row B^T box: the 512 x 256 pair tile as is;
  //  * otherwise the one-CTA 256 x 256 tile (64 bytes per clock), and the
  //    entry's own tile shape when M or N is not a multiple of 256.
  // A larger tile is only taken when it still gives every SM (or SM pair) a
  // tile; small problems keep the entry's own shape so more SMs have work.
  // (A bm=64 entry is served by a 128-row tile fed by two of the caller's 64-row
  // boxes; when M is an odd multiple of 64 the second box of the last tile row
  // lies past the end of A, TMA fills it with zeros and still credits its bytes,
  // and the C map, encoded with M rows, clips the store.)
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  const long long pairs = dev->sm_count / 2;
  auto tiles = [&](int tm, int tn) { return (long long)(m / tm) * (n / tn); };
  int variant = e->variant;
  if (t.bm <= 128 && m % 256 == 0 && n % 512 == 0 && tiles(256, 512) >= pairs)
    variant = VARIANT_2CTA_256x512;
  else if (t.bm == 256 && t.bn == 128 && m % 512 == 0 && n % 256 == 0 && tiles(512, 256) >= pairs)
    variant = VARIANT_2CTA_512x256;
  else if (m % 256 == 0 && n % 256 == 0 && tiles(256, 256) >= dev->sm_count)
    variant = VARIANT_1CTA_256x256;
  GemmParams p;
  std::memset(&p, 0, sizeof p);
  p.a_map_ptr = (const void *)(uintptr_t)a_tmap;
  p.b_map_ptr = (const void *)(uintptr_t)b_tmap;
  p.a_box_rows = t.bm;
  p.b_box_rows = t.bn;
  // C's row stride is (n / bn) * bn = n (examples/kernels/gemm.ml:61-66).
  if ((st = encode_2d(&p.map_c, (const void *)(uintptr_t)c, 4, (uint64_t)n, (uint64_t)m,
                      (uint64_t)n * 4, 32, 32)))
    return st;
  // The entry's stage count is a request; the ring is as deep as it asks for or
  // as deep as fits, whichever is smaller.
  LaunchPlan plan{e->element_bytes == 2 ? 0 : 1, variant, t.stages, 16, 1, 0, 0};
  return launch_umma(*dev, plan, p, m, n, k, (cudaStream_t)stream);
}

int oxgpu_b200_gemm_tf32(const float *a, const float *bt, float *c, int m, int n, int k, int64_t lda,
                         int64_t ldb, int64_t ldc, unsigned flags, void *stream) {
  if ((flags & 0xffu) == VARIANT_SPLITK)
    return fail(OXGPU_E_INVALID_ARG, "split-K needs a workspace: use the _ws entry point");
  return gemm_buffers(1, a, bt, c, m, n, k, lda, ldb, ldc, flags, nullptr, 0, (cudaStream_t)stream);
}

int oxgpu_b200_gemm_bf16(const uint16_t *a, const uint16_t *bt, float *c, int m, int n, int k,
                         int64_t lda, int64_t ldb, int64_t ldc, unsigned flags, void *stream) {
  if ((flags & 0xffu) == VARIANT_SPLITK)
    return fail(OXGPU_E_INVALID_ARG, "split-K needs a workspace: use the _ws entry point");
  return gemm_buffers(0, a, bt, c, m, n, k, lda, ldb, ldc, flags, nullptr, 0, (cudaStream_t)stream);
}

int oxgpu_b200_gemm_bf16_out16(const uint16_t *a, const uint16_t *bt, uint16_t *c, int m, int n, int k,
                               int64_t lda, int64_t ldb, int64_t ldc, unsigned flags, void *stream) {
  // check_buffers treats C as 4-byte elements for alignment; bf16 C is checked inside
  unsigned v = flags & 0xffu;
  if (v == VARIANT_1CTA_256x128 || v == VARIANT_2CTA_256x128 || v == VARIANT_SPLITK)
    return fail(OXGPU_E_INVALID_ARG, "this variant has no bf16-output kernel");
  return gemm_buffers(0, a, bt, (float *)c, m, n, k, lda, ldb, ldc, flags, nullptr, 0, (cudaStream_t)stream,
                      true);
}

size_t oxgpu_b200_splitk_workspace_bytes(int m, int n, int splits) {
  if (m <= 0 || n <= 0) return 0;
  if (splits <= 0) splits = 16;
  const size_t m_pad = (size_t)((m + 127) / 128) * 128;
  return (size_t)splits * m_pad * (size_t)n * sizeof(float);
}

int oxgpu_b200_gemm_bf16_ws(const uint16_t *a, const uint16_t *bt, float *c, int m, int n, int k,
                            int64_t lda, int64_t ldb, int64_t ldc, unsigned flags, void *workspace,
                            size_t workspace_bytes, void *stream) {
  return gemm_buffers(0, a, bt, c, m, n, k, lda, ldb, ldc, flags, workspace, workspace_bytes,
                      (cudaStream_t)stream);
}

int oxgpu_b200_gemm_bf16_fanout(const uint16_t *a, const uint16_t *bt, float *const *c_dests, int n_dests,
                                int m, int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                                unsigned flags, void *stream) {
  return oxgpu::gemm_fanout(0, a, bt, c_dests, n_dests, m, n, k, lda, ldb, ldc, flags, (cudaStream_t)stream);
}

int oxgpu_b200_gemm_tf32_fanout(const float *a, const float *bt, float *const *c_dests, int n_dests, int m,
                                int n, int k, int64_t lda, int64_t ldb, int64_t ldc, unsigned flags,
                                void *stream) {
  return oxgpu::gemm_fanout(1, a, bt, c_dests, n_dests, m, n, k, lda, ldb, ldc, flags, (cudaStream_t)stream);
}

size_t oxgpu_b200_f32_split_workspace_bytes(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  return 3 * (size_t)k * ((size_t)m + (size_t)n) * sizeof(float);
}

int oxgpu_b200_gemm_f32_split(const float *a, const float *bt, float *c, int m, int n, int k, int64_t lda,
                              int64_t ldb, int64_t ldc, unsigned flags, void *workspace,
                              size_t workspace_bytes, void *stream) {
  using namespace oxgpu;
  int st = check_buffers(a, bt, c, m, n, k, lda, ldb, ldc, 4);
  if (st) return st;
  if ((long long)k * 3 > 0x7fffffffLL) return fail(OXGPU_E_TOO_LARGE, "K too large for the three-piece split");
  const size_t need = oxgpu_b200_f32_split_workspace_bytes(m, n, k);
  if (!workspace || workspace_bytes < need || !aligned16(workspace))
    return fail(OXGPU_E_INVALID_ARG, "split workspace missing, misaligned or too small");
  int dev_index;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  cudaStream_t s = (cudaStream_t)stream;
  float *a3 = (float *)workspace;
  float *b3 = a3 + 3 * (size_t)k * m;
  auto blocks_for = [&](int rows) {
    size_t b = ((size_t)rows * (k / 4) + 255) / 256;
    const size_t most = (size_t)dev->sm_count * 16;
    return (unsigned)(b > most ? most : (b ? b : 1));
  };
  split_tf32_kernel<<<blocks_for(m), 256, 0, s>>>(a, a3, m, k, lda, 0);
  OX_CUDA(cudaGetLastError());
  split_tf32_kernel<<<blocks_for(n), 256, 0, s>>>(bt, b3, n, k, ldb, 1);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(2, std::memory_order_relaxed);
  return gemm_buffers(1, a3, b3, c, m, n, 3 * k, 3 * (int64_t)k, 3 * (int64_t)k, ldc, flags, nullptr, 0, s);
}

int oxgpu_b200_gemm_bf16_affine(const uint16_t *a, const uint16_t *bt, float *c, int m, int n, int k,
                                int64_t lda, int64_t ldb, int64_t ldc, const oxgpu_epilogue *epilogue,
                                unsigned flags, void *stream) {
  return oxgpu::gemm_affine(0, a, bt, c, m, n, k, lda, ldb, ldc, epilogue, flags, (cudaStream_t)stream);
}

int oxgpu_b200_gemm_bf16_out16_affine(const uint16_t *a, const uint16_t *bt, uint16_t *c, int m, int n, int k,
                                      int64_t lda, int64_t ldb, int64_t ldc, const oxgpu_epilogue *epilogue,
                                      unsigned flags, void *stream) {
  // (check_buffers only looks at the pointer and the leading dimension of C)
  return oxgpu::gemm_affine(0, a, bt, reinterpret_cast<float *>(c), m, n, k, lda, ldb, ldc, epilogue, flags,
                            (cudaStream_t)stream, true);
}

int oxgpu_b200_gemm_tf32_affine(const float *a, const float *bt, float *c, int m, int n, int k, int64_t lda,
                                int64_t ldb, int64_t ldc, const oxgpu_epilogue *epilogue, unsigned flags,
                                void *stream) {
  return oxgpu::gemm_affine(1, a, bt, c, m, n, k, lda, ldb, ldc, epilogue, flags, (cudaStream_t)stream);
}

int oxgpu_b200_shared_alloc(size_t bytes, void **ptr, unsigned char handle[64]) {
  using namespace oxgpu;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes in the C ABI");
  if (!ptr || !handle || bytes == 0) return fail(OXGPU_E_INVALID_ARG, "null argument or zero size");
  void *q = nullptr;
  OX_CUDA(cudaMalloc(&q, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, q);
  if (e != cudaSuccess) {
    cudaFree(q);
    return cuda_fail(e, "cudaIpcGetMemHandle");
  }
  std::memcpy(handle, &h, 64);
  *ptr = q;
  return OXGPU_OK;
}

int oxgpu_b200_shared_open(const unsigned char handle[64], void **ptr) {
  using namespace oxgpu;
  if (!ptr || !handle) return fail(OXGPU_E_INVALID_ARG, "null argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  OX_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return OXGPU_OK;
}

int oxgpu_b200_shared_close(void *ptr) {
  using namespace oxgpu;
  if (!ptr) return OXGPU_OK;
  OX_CUDA(cudaIpcCloseMemHandle(ptr));
  return OXGPU_OK;
}

int oxgpu_b200_shared_free(void *ptr) {
  using namespace oxgpu;
  if (!ptr) return OXGPU_OK;
  OX_CUDA(cudaFree(ptr));
  return OXGPU_OK;
}

// ---- split-K without any allocation ------------------------------------------------
// The partial tiles live in this file-scope device array.  In host code the
// array's name is only a stand-in, not a device address, so its address is
// looked up once per device with cudaGetSymbolAddress and that pointer is what
// the kernels receive (through the workspace tensor map and the reduction's
// argument).
static __device__ __align__(256) float g_static_splitk_scratch[OXGPU_STATIC_SCRATCH_BYTES / sizeof(float)];
static std::atomic<float *> g_static_scratch_addr[64];  // per device; filled on the first call there

int oxgpu_b200_gemm_bf16_splitk_static(const uint16_t *a, const uint16_t *bt, float *c, int m, int n,
                                       int k, int64_t lda, int64_t ldb, int64_t ldc, int splits,
                                       void *stream) {
  int st = check_buffers(a, bt, c, m, n, k, lda, ldb, ldc, 2);
  if (st) return st;
  if (splits < 0 || splits > 255) return fail(OXGPU_E_INVALID_ARG, "splits must be in [0, 255]");
  if (n % 4) return fail(OXGPU_E_SHAPE, "split-K needs N to be a multiple of 4");
  int dev_index;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  // the slice count the split-K path will settle on (same rule as the
  // workspace entry point), so the size can be refused before anything runs
  const int num_kb = (k + 63) / 64;
  if (splits == 0) {
    long long tiles = (long long)((m + 127) / 128) * ((n + 127) / 128);
    splits = (int)((2LL * dev->sm_count + tiles - 1) / tiles);
    if (splits > 16) splits = 16;
  }
  if (splits > num_kb) splits = num_kb;
  if (splits < 1) splits = 1;
  const int kb_per = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per - 1) / kb_per;
  const size_t m_pad = (size_t)((m + 127) / 128) * 128;
  const size_t need = (size_t)splits * m_pad * (size_t)n * sizeof(float);
  if (need > (size_t)OXGPU_STATIC_SCRATCH_BYTES) {
    char text[200];
    std::snprintf(text, sizeof text,
                  "split-K partial tiles need %zu bytes (%d slices x %zu rows x %d columns), the "
                  "built-in scratch holds %u: use fewer slices or the workspace entry point",
                  need, splits, m_pad, n, (unsigned)OXGPU_STATIC_SCRATCH_BYTES);
    return fail(OXGPU_E_TOO_LARGE, text);
  }
  if (!g_static_scratch_addr[dev_index].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_static_scratch_addr[dev_index].load(std::memory_order_acquire)) {
      float *addr = nullptr;
      OX_CUDA(cudaGetSymbolAddress((void **)&addr, g_static_splitk_scratch));
      if (!addr) return fail(OXGPU_E_INVALID_ARG, "cudaGetSymbolAddress returned a null address");
      g_static_scratch_addr[dev_index].store(addr, std::memory_order_release);
    }
  }
  const unsigned flags = OXGPU_FLAG_VARIANT(OXGPU_VARIANT_SPLITK) | OXGPU_FLAG_SPLITS(splits);
  return gemm_buffers(0, a, bt, c, m, n, k, lda, ldb, ldc, flags, g_static_scratch_addr[dev_index].load(std::memory_order_acquire),
                      (size_t)OXGPU_STATIC_SCRATCH_BYTES, (cudaStream_t)stream);
}

int oxgpu_b200_gemm_exact(const void *a, const void *bt, float *c, int m, int n, int k, int64_t lda,
                          int64_t ldb, int64_t ldc, int input_mode, void *stream) {
  if (!a || !bt || !c) return fail(OXGPU_E_INVALID_ARG, "null operand pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(OXGPU_E_INVALID_ARG, "M, N and K must be positive");
  if (lda < k || ldb < k || ldc < n)
    return fail(OXGPU_E_INVALID_ARG, "leading dimension smaller than the row length");
  if (input_mode < 0 || input_mode > 2) return fail(OXGPU_E_INVALID_ARG, "input_mode must be 0, 1 or 2");
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  dim3 grid((n + kSimtTile - 1) / kSimtTile, (m + kSimtTile - 1) / kSimtTile, 1);
  if (grid.y > 65535) return fail(OXGPU_E_TOO_LARGE, "M too large for the exact kernel's grid");
  cudaStream_t s = (cudaStream_t)stream;
  if (input_mode == 0)
    simt_gemm_exact_kernel<0><<<grid, kSimtThreads, 0, s>>>(a, bt, c, m, n, k, lda, ldb, ldc);
  else if (input_mode == 1)
    simt_gemm_exact_kernel<1><<<grid, kSimtThreads, 0, s>>>(a, bt, c, m, n, k, lda, ldb, ldc);
  else
    simt_gemm_exact_kernel<2><<<grid, kSimtThreads, 0, s>>>(a, bt, c, m, n, k, lda, ldb, ldc);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

int oxgpu_b200_transpose(const void *b, void *bt, int k, int n, int element_bytes, void *stream) {
  if (!b || !bt) return fail(OXGPU_E_INVALID_ARG, "null pointer");
  if (k <= 0 || n <= 0) return fail(OXGPU_E_INVALID_ARG, "K and N must be positive");
  if (element_bytes != 2 && element_bytes != 4)
    return fail(OXGPU_E_INVALID_ARG, "element_bytes must be 2 or 4");
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  cudaStream_t s = (cudaStream_t)stream;
  const int tile_cols = 256 / element_bytes;
  if (k % 64 == 0 && n % tile_cols == 0 && k / 64 <= 65535 && aligned16(b) && aligned16(bt)) {
    // whole tiles of 64 rows x 256 bytes: 16-byte accesses on both sides
    dim3 grid64(n / tile_cols, k / 64, 1);
    if (element_bytes == 2)
      transpose64_pairs_kernel<<<grid64, 256, 0, s>>>((const uint16_t *)b, (uint16_t *)bt, k, n);
    else
      transpose64_kernel<float><<<grid64, 256, 0, s>>>((const float *)b, (float *)bt, k, n);
    OX_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return OXGPU_OK;
  }
  dim3 grid((n + 31) / 32, (k + 31) / 32, 1), block(32, 8, 1);
  if (grid.y > 65535) return fail(OXGPU_E_TOO_LARGE, "K too large for the transpose grid");
  if (element_bytes == 2)
    transpose_kernel<uint16_t><<<grid, block, 0, s>>>((const uint16_t *)b, (uint16_t *)bt, k, n);
  else
    transpose_kernel<float><<<grid, block, 0, s>>>((const float *)b, (float *)bt, k, n);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

int oxgpu_b200_transpose_f32_to_bf16(const float *b, uint16_t *bt, int k, int n, void *stream) {
  if (!b || !bt) return fail(OXGPU_E_INVALID_ARG, "null pointer");
  if (k <= 0 || n <= 0) return fail(OXGPU_E_INVALID_ARG, "K and N must be positive");
  if (k % 64 || n % 64) return fail(OXGPU_E_SHAPE, "the fused re-layout takes K and N that are multiples of 64");
  if (k / 64 > 65535) return fail(OXGPU_E_TOO_LARGE, "K too large for the transpose grid");
  if (!aligned16(b) || !aligned16(bt)) return fail(OXGPU_E_ALIGN, "pointers must be 16-byte aligned");
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  transpose64_f32_to_bf16_kernel<<<dim3(n / 64, k / 64, 1), 256, 0, (cudaStream_t)stream>>>(b, bt, k, n);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

int oxgpu_b200_f32_to_bf16(const float *src, uint16_t *dst, size_t count, void *stream) {
  if (!src || !dst) return fail(OXGPU_E_INVALID_ARG, "null pointer");
  if (count == 0) return OXGPU_OK;
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  const int vec = aligned16(src) && aligned16(dst) ? 1 : 0;
  size_t blocks = ((vec ? (count + 7) / 8 : count) + 255) / 256;
  if (blocks > (size_t)dev->sm_count * 16) blocks = (size_t)dev->sm_count * 16;
  f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(src, dst, count, vec);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

int oxgpu_b200_gemm_bf16_host(const uint16_t *a_host, const uint16_t *bt_host, float *c_host, int m,
                              int n, int k, unsigned flags) {
  return gemm_host(0, a_host, bt_host, c_host, m, n, k, flags);
}

int oxgpu_b200_gemm_tf32_host(const float *a_host, const float *bt_host, float *c_host, int m, int n,
                              int k, unsigned flags) {
  return gemm_host(1, a_host, bt_host, c_host, m, n, k, flags);
}

int oxgpu_b200_gemm_bf16_out16_host(const uint16_t *a_host, const uint16_t *bt_host, uint16_t *c_host, int m,
                                    int n, int k, unsigned flags) {
  unsigned v = flags & 0xffu;
  if (v == VARIANT_1CTA_256x128 || v == VARIANT_2CTA_256x128 || v == VARIANT_SPLITK ||
      v == VARIANT_CLUSTER_SPLITK_128x256 || v == VARIANT_CLUSTER_SPLITK_128x128)
    return fail(OXGPU_E_INVALID_ARG, "this variant has no bf16-output kernel");
  return gemm_host(0, a_host, bt_host, c_host, m, n, k, flags, true);
}

int oxgpu_b200_release_staging(void) {
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  std::lock_guard<std::mutex> lock(g_staging_mutex);
  Staging &s = dev->staging;
  OX_CUDA(cudaDeviceSynchronize());
  if (s.a) OX_CUDA(cudaFree(s.a));
  if (s.bt) OX_CUDA(cudaFree(s.bt));
  if (s.c) OX_CUDA(cudaFree(s.c));
  s.a = s.bt = s.c = nullptr;
  s.a_bytes = s.bt_bytes = s.c_bytes = 0;
  if (s.events) {
    for (int i = 0; i < 64; i++) {
      OX_CUDA(cudaEventDestroy(s.a_ready[i]));
      OX_CUDA(cudaEventDestroy(s.c_ready[i]));
    }
    s.events = false;
  }
  if (s.in) {
    OX_CUDA(cudaStreamDestroy(s.in));
    OX_CUDA(cudaStreamDestroy(s.compute));
    OX_CUDA(cudaStreamDestroy(s.out));
    s.in = s.compute = s.out = nullptr;
  }
  return OXGPU_OK;
}

static int fill(int dist, void *dst, size_t count, int element_bytes, uint32_t seed, float scale,
                uint64_t offset, void *stream) {
  if (!dst) return fail(OXGPU_E_INVALID_ARG, "null pointer");
  if (element_bytes != 2 && element_bytes != 4)
    return fail(OXGPU_E_INVALID_ARG, "element_bytes must be 2 or 4");
  if (count == 0) return OXGPU_OK;
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  const int vec = aligned16(dst) ? 1 : 0;
  size_t blocks = ((vec ? (count + 3) / 4 : count) + 255) / 256;
  if (blocks > (size_t)dev->sm_count * 16) blocks = (size_t)dev->sm_count * 16;
  cudaStream_t s = (cudaStream_t)stream;
  unsigned g = (unsigned)blocks;
  if (dist == 0 && element_bytes == 4) synth_fill_kernel<0, false><<<g, 256, 0, s>>>(dst, count, seed, scale, offset, vec);
  else if (dist == 0) synth_fill_kernel<0, true><<<g, 256, 0, s>>>(dst, count, seed, scale, offset, vec);
  else if (element_bytes == 4) synth_fill_kernel<1, false><<<g, 256, 0, s>>>(dst, count, seed, scale, offset, vec);
  else synth_fill_kernel<1, true><<<g, 256, 0, s>>>(dst, count, seed, scale, offset, vec);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return OXGPU_OK;
}

int oxgpu_b200_fill_uniform(void *dst, size_t count, int element_bytes, uint32_t seed,
                            uint64_t index_offset, void *stream) {
  return fill(0, dst, count, element_bytes, seed, 1.0f, index_offset, stream);
}

int oxgpu_b200_fill_normal(void *dst, size_t count, int element_bytes, uint32_t seed, float std_dev,
                           uint64_t index_offset, void *stream) {
  return fill(1, dst, count, element_bytes, seed, std_dev, index_offset, stream);
}

int oxgpu_b200_device_status(uint32_t words[8]) {
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  OX_CUDA(cudaDeviceSynchronize());
  uint32_t host[8];
  OX_CUDA(cudaMemcpyFromSymbol(host, g_device_status, sizeof host));
  if (words) std::memcpy(words, host, sizeof host);
  if (host[0] != 0) {
    uint32_t zero[8] = {};
    OX_CUDA(cudaMemcpyToSymbol(g_device_status, zero, sizeof zero));
    // a launch that gave up may have left its tile queue half used
    void *queue = nullptr;
    OX_CUDA(cudaGetSymbolAddress(&queue, g_tile_queue));
    OX_CUDA(cudaMemset(queue, 0, sizeof(unsigned int) * 2 * kSchedSlots));
    char text[160];
    std::snprintf(text, sizeof text,
                  "device wait timed out: kind %u, block %u, detail %u, parity %u", host[0], host[1],
                  host[2], host[3]);
    return fail(OXGPU_E_DEVICE_TIMEOUT, text);
  }
  return OXGPU_OK;
}

int oxgpu_b200_selftest_bounded_wait(uint64_t budget_ns) {
  int dev_index, st;
  DeviceState *dev = nullptr;
  if ((st = current_device(&dev_index, &dev))) return st;
  if (budget_ns == 0 || budget_ns > 1000000000ull)
    return fail(OXGPU_E_INVALID_ARG, "self-test budget must be in (0, 1 s]");
  bounded_wait_selftest_kernel<<<1, 32>>>((unsigned long long)budget_ns);
  OX_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return oxgpu_b200_device_status(nullptr);
}

uint64_t oxgpu_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char *oxgpu_b200_build_info(void) {
  return "oxgpu_b200: sm_100a; tcgen05 UMMA bf16+tf32; variants 1cta_128x256 1cta_128x128 "
         "1cta_256x128 2cta_256x256 2cta_256x128 2cta_512x256 splitk; cudart " OXGPU_STRINGIFY(CUDART_VERSION);
}

}  // extern "C"
