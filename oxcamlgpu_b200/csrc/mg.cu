// Multi-GPU driver behind the C ABI: one process, one host thread and one
// stream per device, a GEMM whose B^T and C are split by columns across the
// devices and whose A is replicated.  The reference has no multi-GPU code; the
// launcher this sits beside drives a single device through the driver API from
// one host thread (test/hardware/run_gemm_h100.cu:100-108,183-186).
//
// C[:, n0:n1] = A * B[:, n0:n1] needs no exchange: with B held K-major as
// B^T[N,K], a column block of B is a contiguous row block of B^T.  Every
// device therefore runs the ordinary single-GPU entry point on its shard.  A
// replicated C is optional and comes two ways:
//   * NCCL: ncclAllGather of the shards (NCCL gathers contiguous chunks, so
//     the result is block-column-major [g][M][N/g]) and, for a row-major
//     replica, a re-interleave pass on every device;
//   * fused: the GEMM's fan-out epilogue stores every tile into all devices'
//     row-major C over NVLink as it is produced (plain peer stores; no peer
//     loads, no multicast), so neither the gather nor the re-interleave exists.
// NCCL is resolved at run time with dlopen, so the library loads (and every
// other entry point works) on a machine without it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <string>
#include <thread>

#include "common.hpp"

namespace oxgpu {
namespace {

constexpr int kMgMaxDevices = 8;

// ---- the handful of NCCL entry points used, resolved with dlsym ---------------
// (declared here with their public C signatures so that building the library
// needs no NCCL header; ncclFloat32 is 7 in every NCCL 2 release)
typedef struct ncclComm *nccl_comm_t;
struct NcclApi {
  void *handle = nullptr;
  int (*CommInitAll)(nccl_comm_t *, int, const int *) = nullptr;
  int (*CommDestroy)(nccl_comm_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  int (*GetVersion)(int *) = nullptr;
};
constexpr int kNcclFloat32 = 7;
NcclApi g_nccl;
std::mutex g_nccl_mutex;

int load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.handle) return OXGPU_OK;
  const char *names[] = {std::getenv("OXGPU_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  void *h = nullptr;
  for (const char *name : names) {
    if (!name || !*name) continue;
    h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return fail(OXGPU_E_NO_DRIVER, "libnccl.so.2 could not be loaded (set OXGPU_NCCL_LIB to its path)");
  NcclApi api;
  api.handle = h;
  api.CommInitAll = (decltype(api.CommInitAll))dlsym(h, "ncclCommInitAll");
  api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
  api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
  api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
  api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
  api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
  api.GetVersion = (decltype(api.GetVersion))dlsym(h, "ncclGetVersion");
  if (!api.CommInitAll || !api.CommDestroy || !api.AllGather || !api.GroupStart || !api.GroupEnd ||
      !api.GetErrorString)
    return fail(OXGPU_E_NO_DRIVER, "the NCCL library lacks an entry point this driver needs");
  g_nccl = api;
  return OXGPU_OK;
}

int nccl_fail(int r, const char *what) {
  return fail(10000 + r, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error"));
}

int cuda_fail(cudaError_t e, const char *what) {
  return fail((int)e, std::string(what) + ": " + cudaGetErrorName(e) + ": " + cudaGetErrorString(e));
}
#define MG_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call); \
  } while (0)

// [g][M][W] block-column-major -> row-major C[M, g*W]; 16-byte accesses on both
// sides, one pass over the data (HBM-bound: reads and writes M*N*4 bytes each).
__global__ void __launch_bounds__(256)
blocks_to_row_major_kernel(const float4 *__restrict__ blocks, float4 *__restrict__ out, int m, int w4, int g) {
  const size_t row_pieces = (size_t)w4 * g, total = (size_t)m * row_pieces;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / row_pieces, c = i - r * row_pieces;
    const size_t b = c / (size_t)w4, cw = c - b * (size_t)w4;
    out[i] = __ldcs(blocks + (b * (size_t)m + r) * (size_t)w4 + cw);
  }
}

struct DeviceStaging {  // host-operand entry point: this device's copies of A, its B^T rows and its C shard
  void *a = nullptr, *bt = nullptr, *c = nullptr;
  size_t a_bytes = 0, bt_bytes = 0, c_bytes = 0;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t up[32] = {}, done[32] = {}, tail = nullptr;
  bool ready = false;
};

struct Job {
  int kind = 0;  // 1 = device-buffer GEMM, 2 = host-operand GEMM
  const uint16_t *const *a = nullptr;
  const uint16_t *const *bt = nullptr;
  float *const *c_shard = nullptr;
  float *const *c_full = nullptr;
  const uint16_t *a_host = nullptr, *bt_host = nullptr;
  float *c_host = nullptr;
  int c_host_layout = 0;
  int m = 0, n = 0, k = 0, gather = 0;
  unsigned flags = 0;
  int n0[kMgMaxDevices] = {}, n1[kMgMaxDevices] = {};
};

}  // namespace
}  // namespace oxgpu

using namespace oxgpu;

struct oxgpu_mg {
  int n = 0;
  int devices[kMgMaxDevices] = {};
  cudaStream_t stream[kMgMaxDevices] = {};
  cudaEvent_t start[kMgMaxDevices] = {}, mid[kMgMaxDevices] = {}, stop[kMgMaxDevices] = {};
  bool peers = false;  // every device can store into every other device's memory
  nccl_comm_t comm[kMgMaxDevices] = {};
  bool nccl_ready = false;
  void *scratch[kMgMaxDevices] = {};  // gathered blocks before the re-interleave
  size_t scratch_bytes[kMgMaxDevices] = {};
  DeviceStaging staging[kMgMaxDevices];
  bool timed = false;  // a job with events has run
  // one worker per device; a job is handed to all of them at once
  std::thread workers[kMgMaxDevices];
  std::mutex mu;
  std::condition_variable cv_job, cv_done;
  uint64_t generation = 0;
  int pending = 0;
  bool quit = false;
  Job job;
  int status[kMgMaxDevices] = {};
  std::string message[kMgMaxDevices];
};

namespace oxgpu {
namespace {

int grow(void **ptr, size_t *have, size_t want) {
  if (*have >= want) return OXGPU_OK;
  if (*ptr) {
    MG_CUDA(cudaFree(*ptr));
    *ptr = nullptr;
    *have = 0;
  }
  MG_CUDA(cudaMalloc(ptr, want));
  *have = want;
  return OXGPU_OK;
}

// Device-buffer job on device d (worker thread, device d current).
int run_device_job(oxgpu_mg *mg, int d, const Job &j) {
  cudaStream_t s = mg->stream[d];
  const int w = j.n1[d] - j.n0[d];
  MG_CUDA(cudaEventRecord(mg->start[d], s));
  int st = OXGPU_OK;
  if (w > 0) {
    if (j.gather == OXGPU_MG_GATHER_FUSED) {
      float *dests[kMgMaxDevices];
      for (int i = 0; i < mg->n; i++) dests[i] = j.c_full[i] + j.n0[d];
      st = oxgpu_b200_gemm_bf16_fanout(j.a[d], j.bt[d], dests, mg->n, j.m, w, j.k, j.k, j.k, j.n, j.flags, s);
    } else {
      st = oxgpu_b200_gemm_bf16(j.a[d], j.bt[d], j.c_shard[d], j.m, w, j.k, j.k, j.k, w, j.flags, s);
    }
    if (st) return st;
  }
  MG_CUDA(cudaEventRecord(mg->mid[d], s));
  if (j.gather == OXGPU_MG_GATHER_NCCL || j.gather == OXGPU_MG_GATHER_NCCL_BLOCKS) {
    const bool blocks = j.gather == OXGPU_MG_GATHER_NCCL_BLOCKS || mg->n == 1;
    float *recv = blocks ? j.c_full[d] : (float *)mg->scratch[d];
    // one thread per device, each on its own communicator: the call returns once
    // the collective is enqueued on this device's stream
    int r = g_nccl.AllGather(j.c_shard[d], recv, (size_t)j.m * w, kNcclFloat32, mg->comm[d], s);
    if (r != 0) return nccl_fail(r, "ncclAllGather");
    if (!blocks) {
      const size_t total = (size_t)j.m * (j.n / 4);
      size_t grid = (total + 255) / 256;
      if (grid > 148u * 16u) grid = 148u * 16u;
      blocks_to_row_major_kernel<<<(unsigned)grid, 256, 0, s>>>((const float4 *)recv, (float4 *)j.c_full[d], j.m,
                                                               w / 4, mg->n);
      MG_CUDA(cudaGetLastError());
    }
  }
  MG_CUDA(cudaEventRecord(mg->stop[d], s));
  return OXGPU_OK;
}

// Host-operand job on device d: B^T rows first, then A in row blocks; the rows
// of C a block of A yields are computed as soon as that block has landed and
// go down while the next block comes up.  Three streams per device, so both
// PCIe directions of every device stay busy.
int run_host_job(oxgpu_mg *mg, int d, const Job &j) {
  DeviceStaging &g = mg->staging[d];
  cudaStream_t s = mg->stream[d];
  const int w = j.n1[d] - j.n0[d];
  MG_CUDA(cudaEventRecord(mg->start[d], s));
  if (w > 0) {
    if (!g.ready) {
      MG_CUDA(cudaStreamCreateWithFlags(&g.in, cudaStreamNonBlocking));
      MG_CUDA(cudaStreamCreateWithFlags(&g.out, cudaStreamNonBlocking));
      for (int i = 0; i < 32; i++) {
        MG_CUDA(cudaEventCreateWithFlags(&g.up[i], cudaEventDisableTiming));
        MG_CUDA(cudaEventCreateWithFlags(&g.done[i], cudaEventDisableTiming));
      }
      MG_CUDA(cudaEventCreateWithFlags(&g.tail, cudaEventDisableTiming));
      g.ready = true;
    }
    const size_t row_bytes = (size_t)j.k * 2;
    int st;
    if ((st = grow(&g.a, &g.a_bytes, (size_t)j.m * row_bytes))) return st;
    if ((st = grow(&g.bt, &g.bt_bytes, (size_t)w * row_bytes))) return st;
    if ((st = grow(&g.c, &g.c_bytes, (size_t)j.m * w * 4))) return st;
    // the staging buffers may still be in use by the previous call's downloads
    MG_CUDA(cudaStreamWaitEvent(g.in, mg->start[d], 0));
    MG_CUDA(cudaMemcpyAsync(g.bt, (const char *)j.bt_host + (size_t)j.n0[d] * row_bytes, (size_t)w * row_bytes,
                            cudaMemcpyHostToDevice, g.in));
    int block = ((j.m / 8 + 255) / 256) * 256;
    if (block < 256) block = 256;
    while ((j.m + block - 1) / block > 32) block *= 2;
    int ev = 0;
    // where this device's columns go on the host: a column window of the
    // row-major C (pitch N), or its own contiguous [M][w] block
    float *c_dst = j.c_host_layout == OXGPU_MG_HOST_C_BLOCKS ? j.c_host + (size_t)j.n0[d] * j.m : j.c_host + j.n0[d];
    const size_t c_pitch = (j.c_host_layout == OXGPU_MG_HOST_C_BLOCKS ? (size_t)w : (size_t)j.n) * 4;
    for (int r0 = 0; r0 < j.m; r0 += block, ev++) {
      const int rows = j.m - r0 < block ? j.m - r0 : block;
      MG_CUDA(cudaMemcpyAsync((char *)g.a + (size_t)r0 * row_bytes, (const char *)j.a_host + (size_t)r0 * row_bytes,
                              (size_t)rows * row_bytes, cudaMemcpyHostToDevice, g.in));
      MG_CUDA(cudaEventRecord(g.up[ev], g.in));
      MG_CUDA(cudaStreamWaitEvent(s, g.up[ev], 0));
      float *c_dev = (float *)g.c + (size_t)r0 * w;
      st = oxgpu_b200_gemm_bf16((const uint16_t *)g.a + (size_t)r0 * j.k, (const uint16_t *)g.bt, c_dev, rows, w, j.k,
                                j.k, j.k, w, j.flags, s);
      if (st) {
        cudaStreamSynchronize(g.in);
        cudaStreamSynchronize(s);
        cudaStreamSynchronize(g.out);
        return st;
      }
      MG_CUDA(cudaEventRecord(g.done[ev], s));
      MG_CUDA(cudaStreamWaitEvent(g.out, g.done[ev], 0));
      MG_CUDA(cudaMemcpy2DAsync((char *)c_dst + (size_t)r0 * c_pitch, c_pitch, c_dev, (size_t)w * 4, (size_t)w * 4,
                                (size_t)rows, cudaMemcpyDeviceToHost, g.out));
    }
    // the device's main stream ends after the last download
    MG_CUDA(cudaEventRecord(g.tail, g.out));
    MG_CUDA(cudaStreamWaitEvent(s, g.tail, 0));
  }
  MG_CUDA(cudaEventRecord(mg->mid[d], s));
  MG_CUDA(cudaEventRecord(mg->stop[d], s));
  return OXGPU_OK;
}

void worker_main(oxgpu_mg *mg, int d) {
  cudaSetDevice(mg->devices[d]);
  uint64_t seen = 0;
  for (;;) {
    Job job;
    {
      std::unique_lock<std::mutex> lock(mg->mu);
      mg->cv_job.wait(lock, [&] { return mg->quit || mg->generation != seen; });
      if (mg->quit) return;
      seen = mg->generation;
      job = mg->job;
    }
    int st = job.kind == 2 ? run_host_job(mg, d, job) : run_device_job(mg, d, job);
    const char *text = st ? oxgpu_b200_last_error() : "";
    {
      std::lock_guard<std::mutex> lock(mg->mu);
      mg->status[d] = st;
      mg->message[d] = text ? text : "";
      if (--mg->pending == 0) mg->cv_done.notify_all();
    }
  }
}

// Hand `job` to every worker and wait until all of them have ENQUEUED their
// part (not until the devices have finished: that is oxgpu_b200_mg_sync).
int dispatch(oxgpu_mg *mg, const Job &job) {
  std::unique_lock<std::mutex> lock(mg->mu);
  mg->job = job;
  mg->pending = mg->n;
  mg->generation++;
  mg->cv_job.notify_all();
  mg->cv_done.wait(lock, [&] { return mg->pending == 0; });
  mg->timed = true;
  for (int d = 0; d < mg->n; d++)
    if (mg->status[d]) {
      char where[32];
      std::snprintf(where, sizeof where, "device %d: ", mg->devices[d]);
      return fail(mg->status[d], where + mg->message[d]);
    }
  return OXGPU_OK;
}

int fill_partition(const oxgpu_mg *mg, int n, Job *job) {
  return oxgpu_b200_mg_column_partition(n, mg->n, OXGPU_MG_COLUMN_ALIGN, job->n0, job->n1);
}

struct DeviceGuard {  // restores the caller's current device
  int saved = -1;
  DeviceGuard() { cudaGetDevice(&saved); }
  ~DeviceGuard() {
    if (saved >= 0) cudaSetDevice(saved);
  }
};

}  // namespace
}  // namespace oxgpu

extern "C" {

int oxgpu_b200_mg_column_partition(int n, int parts, int align, int *n0, int *n1) {
  if (n <= 0 || parts <= 0 || align <= 0 || !n0 || !n1)
    return fail(OXGPU_E_INVALID_ARG, "n, parts and align must be positive and the outputs non-null");
  // contiguous ranges of whole `align`-column blocks; block counts differ by at
  // most one (the first n_blocks % parts ranges get the extra block) and the
  // last non-empty range carries the ragged tail
  const long long blocks = ((long long)n + align - 1) / align;
  const long long base = blocks / parts, extra = blocks % parts;
  long long start = 0;
  for (int r = 0; r < parts; r++) {
    const long long width = base + (r < extra ? 1 : 0);
    long long lo = start * align, hi = (start + width) * align;
    if (lo > n) lo = n;
    if (hi > n) hi = n;
    n0[r] = (int)lo;
    n1[r] = (int)hi;
    start += width;
  }
  return OXGPU_OK;
}

int oxgpu_b200_mg_create(int ngpu, const int *devices, oxgpu_mg **out) {
  if (!out) return fail(OXGPU_E_INVALID_ARG, "null output pointer");
  *out = nullptr;
  if (ngpu < 1 || ngpu > kMgMaxDevices) return fail(OXGPU_E_INVALID_ARG, "between 1 and 8 devices");
  int count = 0;
  MG_CUDA(cudaGetDeviceCount(&count));
  DeviceGuard guard;
  oxgpu_mg *mg = new oxgpu_mg;
  mg->n = ngpu;
  for (int d = 0; d < ngpu; d++) {
    const int dev = devices ? devices[d] : d;
    if (dev < 0 || dev >= count) {
      delete mg;
      return fail(OXGPU_E_INVALID_ARG, "device index out of range");
    }
    for (int e = 0; e < d; e++)
      if (mg->devices[e] == dev) {
        delete mg;
        return fail(OXGPU_E_INVALID_ARG, "a device is listed twice");
      }
    mg->devices[d] = dev;
  }
  auto bail = [&](int st) {
    oxgpu_b200_mg_destroy(mg);
    return st;
  };
  for (int d = 0; d < ngpu; d++) {
    cudaError_t e = cudaSetDevice(mg->devices[d]);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&mg->stream[d], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&mg->start[d]);
    if (e == cudaSuccess) e = cudaEventCreate(&mg->mid[d]);
    if (e == cudaSuccess) e = cudaEventCreate(&mg->stop[d]);
    if (e != cudaSuccess) return bail(cuda_fail(e, "per-device set-up"));
  }
  // Peer access, once: needed only by the fused gather (stores into the other
  // devices' C); its absence is remembered, not an error.
  mg->peers = true;
  for (int d = 0; d < ngpu; d++) {
    cudaSetDevice(mg->devices[d]);
    for (int e = 0; e < ngpu; e++) {
      if (e == d) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, mg->devices[d], mg->devices[e]);
      if (!can) {
        mg->peers = false;
        continue;
      }
      cudaError_t r = cudaDeviceEnablePeerAccess(mg->devices[e], 0);
      if (r == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (r != cudaSuccess) {
        cudaGetLastError();
        mg->peers = false;
      }
    }
  }
  for (int d = 0; d < ngpu; d++) mg->workers[d] = std::thread(worker_main, mg, d);
  *out = mg;
  return OXGPU_OK;
}

int oxgpu_b200_mg_destroy(oxgpu_mg *mg) {
  if (!mg) return OXGPU_OK;
  DeviceGuard guard;
  {
    std::lock_guard<std::mutex> lock(mg->mu);
    mg->quit = true;
  }
  mg->cv_job.notify_all();
  for (int d = 0; d < mg->n; d++)
    if (mg->workers[d].joinable()) mg->workers[d].join();
  for (int d = 0; d < mg->n; d++) {
    if (cudaSetDevice(mg->devices[d]) != cudaSuccess) continue;
    if (mg->stream[d]) cudaStreamSynchronize(mg->stream[d]);
    if (mg->nccl_ready && mg->comm[d]) g_nccl.CommDestroy(mg->comm[d]);
    DeviceStaging &g = mg->staging[d];
    if (g.ready) {
      cudaStreamSynchronize(g.in);
      cudaStreamSynchronize(g.out);
      cudaStreamDestroy(g.in);
      cudaStreamDestroy(g.out);
      for (int i = 0; i < 32; i++) {
        cudaEventDestroy(g.up[i]);
        cudaEventDestroy(g.done[i]);
      }
      cudaEventDestroy(g.tail);
    }
    if (g.a) cudaFree(g.a);
    if (g.bt) cudaFree(g.bt);
    if (g.c) cudaFree(g.c);
    if (mg->scratch[d]) cudaFree(mg->scratch[d]);
    if (mg->start[d]) cudaEventDestroy(mg->start[d]);
    if (mg->mid[d]) cudaEventDestroy(mg->mid[d]);
    if (mg->stop[d]) cudaEventDestroy(mg->stop[d]);
    if (mg->stream[d]) cudaStreamDestroy(mg->stream[d]);
  }
  cudaGetLastError();
  delete mg;
  return OXGPU_OK;
}

int oxgpu_b200_mg_device_count(const oxgpu_mg *mg) { return mg ? mg->n : 0; }

int oxgpu_b200_mg_device(const oxgpu_mg *mg, int index) {
  return (mg && index >= 0 && index < mg->n) ? mg->devices[index] : -1;
}

int oxgpu_b200_mg_peer_access(const oxgpu_mg *mg) { return mg && (mg->peers || mg->n == 1) ? 1 : 0; }

int oxgpu_b200_mg_gemm_bf16(oxgpu_mg *mg, const uint16_t *const *a_repl, const uint16_t *const *bt_shard,
                            float *const *c_shard, int m, int n, int k, int gather_c, float *const *c_full,
                            unsigned flags) {
  if (!mg) return fail(OXGPU_E_INVALID_ARG, "null driver handle");
  if (!a_repl || !bt_shard) return fail(OXGPU_E_INVALID_ARG, "null operand array");
  if (m <= 0 || n <= 0 || k <= 0) return fail(OXGPU_E_INVALID_ARG, "M, N and K must be positive");
  if (gather_c < OXGPU_MG_GATHER_NONE || gather_c > OXGPU_MG_GATHER_NCCL_BLOCKS)
    return fail(OXGPU_E_INVALID_ARG, "gather_c must be one of OXGPU_MG_GATHER_*");
  if (gather_c != OXGPU_MG_GATHER_FUSED && !c_shard) return fail(OXGPU_E_INVALID_ARG, "null c_shard array");
  if (gather_c != OXGPU_MG_GATHER_NONE && !c_full) return fail(OXGPU_E_INVALID_ARG, "a gather needs c_full");
  Job job;
  job.kind = 1;
  int st = fill_partition(mg, n, &job);
  if (st) return st;
  for (int d = 0; d < mg->n; d++) {
    const bool has_columns = job.n1[d] > job.n0[d];
    if (has_columns && (!a_repl[d] || !bt_shard[d])) return fail(OXGPU_E_INVALID_ARG, "null operand pointer");
    if (has_columns && gather_c != OXGPU_MG_GATHER_FUSED && !c_shard[d])
      return fail(OXGPU_E_INVALID_ARG, "null c_shard pointer");
    if (gather_c != OXGPU_MG_GATHER_NONE && !c_full[d]) return fail(OXGPU_E_INVALID_ARG, "null c_full pointer");
  }
  // Everything a single device's launch would refuse is refused here, for all
  // devices, before anything is enqueued: a device that dropped out of a
  // collective after the others had entered it would leave them waiting.
  if (k % 8) return fail(OXGPU_E_SHAPE, "K must be a multiple of 8 (rows of 16 bytes)");
  auto misaligned = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
  for (int d = 0; d < mg->n; d++) {
    if (job.n1[d] <= job.n0[d]) continue;
    if (misaligned(a_repl[d]) || misaligned(bt_shard[d]) || (c_shard && misaligned(c_shard[d])) ||
        (c_full && misaligned(c_full[d])))
      return fail(OXGPU_E_ALIGN, "operand pointers must be 16-byte aligned");
    if ((job.n1[d] - job.n0[d]) % 4) return fail(OXGPU_E_SHAPE, "shard widths must be multiples of 4 columns");
  }
  if (gather_c == OXGPU_MG_GATHER_FUSED) {
    if (n % 4) return fail(OXGPU_E_SHAPE, "the fused gather needs N to be a multiple of 4");
    if (mg->n > 1 && !mg->peers)
      return fail(OXGPU_E_INVALID_ARG, "the fused gather needs peer access between all devices of the handle");
  }
  if (gather_c == OXGPU_MG_GATHER_NCCL || gather_c == OXGPU_MG_GATHER_NCCL_BLOCKS) {
    const int w = job.n1[0] - job.n0[0];
    for (int d = 0; d < mg->n; d++)
      if (job.n1[d] - job.n0[d] != w || w % 4)
        return fail(OXGPU_E_SHAPE, "the NCCL gather needs equal shard widths: N a multiple of 256 * devices");
    if ((st = load_nccl())) return st;
    DeviceGuard guard;
    if (!mg->nccl_ready) {
      int r = g_nccl.CommInitAll(mg->comm, mg->n, mg->devices);
      if (r != 0) return nccl_fail(r, "ncclCommInitAll");
      mg->nccl_ready = true;
    }
    if (gather_c == OXGPU_MG_GATHER_NCCL && mg->n > 1) {
      const size_t need = (size_t)m * n * 4;
      for (int d = 0; d < mg->n; d++) {
        MG_CUDA(cudaSetDevice(mg->devices[d]));
        if (mg->scratch_bytes[d] < need) MG_CUDA(cudaStreamSynchronize(mg->stream[d]));
        if ((st = grow(&mg->scratch[d], &mg->scratch_bytes[d], need))) return st;
      }
    }
  }
  job.a = a_repl;
  job.bt = bt_shard;
  job.c_shard = c_shard;
  job.c_full = c_full;
  job.m = m;
  job.n = n;
  job.k = k;
  job.gather = gather_c;
  job.flags = flags;
  return dispatch(mg, job);
}

int oxgpu_b200_mg_gemm_bf16_host(oxgpu_mg *mg, const uint16_t *a_host, const uint16_t *bt_host, float *c_host,
                                 int m, int n, int k, int c_layout, unsigned flags) {
  if (!mg) return fail(OXGPU_E_INVALID_ARG, "null driver handle");
  if (!a_host || !bt_host || !c_host) return fail(OXGPU_E_INVALID_ARG, "null host pointer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(OXGPU_E_INVALID_ARG, "M, N and K must be positive");
  if (k % 8 || n % 4) return fail(OXGPU_E_SHAPE, "K must be a multiple of 8 and N a multiple of 4");
  if (c_layout != OXGPU_MG_HOST_C_ROW_MAJOR && c_layout != OXGPU_MG_HOST_C_BLOCKS)
    return fail(OXGPU_E_INVALID_ARG, "c_layout must be OXGPU_MG_HOST_C_ROW_MAJOR or OXGPU_MG_HOST_C_BLOCKS");
  Job job;
  job.kind = 2;
  int st = fill_partition(mg, n, &job);
  if (st) return st;
  job.a_host = a_host;
  job.bt_host = bt_host;
  job.c_host = c_host;
  job.c_host_layout = c_layout;
  job.m = m;
  job.n = n;
  job.k = k;
  job.flags = flags;
  if ((st = dispatch(mg, job))) {
    oxgpu_b200_mg_sync(mg);  // nothing of this call stays in flight on the caller's buffers
    return st;
  }
  return oxgpu_b200_mg_sync(mg);  // C is complete on the host when this returns
}

int oxgpu_b200_mg_sync(oxgpu_mg *mg) {
  if (!mg) return fail(OXGPU_E_INVALID_ARG, "null driver handle");
  DeviceGuard guard;
  int first = OXGPU_OK;
  for (int d = 0; d < mg->n; d++) {
    cudaError_t e = cudaSetDevice(mg->devices[d]);
    if (e == cudaSuccess) e = cudaStreamSynchronize(mg->stream[d]);
    if (e != cudaSuccess && first == OXGPU_OK) first = cuda_fail(e, "cudaStreamSynchronize");
  }
  return first;
}

int oxgpu_b200_mg_elapsed_ms(oxgpu_mg *mg, float *total_ms, float *gemm_ms) {
  if (!mg) return fail(OXGPU_E_INVALID_ARG, "null driver handle");
  if (!mg->timed) return fail(OXGPU_E_INVALID_ARG, "no call has run on this handle yet");
  DeviceGuard guard;
  for (int d = 0; d < mg->n; d++) {
    MG_CUDA(cudaSetDevice(mg->devices[d]));
    MG_CUDA(cudaEventSynchronize(mg->stop[d]));
    float t = 0.f, g = 0.f;
    MG_CUDA(cudaEventElapsedTime(&t, mg->start[d], mg->stop[d]));
    MG_CUDA(cudaEventElapsedTime(&g, mg->start[d], mg->mid[d]));
    if (total_ms) total_ms[d] = t;
    if (gemm_ms) gemm_ms[d] = g;
  }
  return OXGPU_OK;
}

int oxgpu_b200_mg_alloc(oxgpu_mg *mg, int index, size_t bytes, void **ptr) {
  if (!mg || !ptr || index < 0 || index >= mg->n || bytes == 0)
    return fail(OXGPU_E_INVALID_ARG, "bad handle, index, size or output pointer");
  DeviceGuard guard;
  MG_CUDA(cudaSetDevice(mg->devices[index]));
  MG_CUDA(cudaMalloc(ptr, bytes));
  return OXGPU_OK;
}

int oxgpu_b200_mg_free(oxgpu_mg *mg, int index, void *ptr) {
  if (!mg || index < 0 || index >= mg->n) return fail(OXGPU_E_INVALID_ARG, "bad handle or index");
  if (!ptr) return OXGPU_OK;
  DeviceGuard guard;
  MG_CUDA(cudaSetDevice(mg->devices[index]));
  MG_CUDA(cudaFree(ptr));
  return OXGPU_OK;
}

int oxgpu_b200_mg_copy(oxgpu_mg *mg, int index, void *dst, const void *src, size_t bytes, int direction) {
  if (!mg || index < 0 || index >= mg->n || !dst || !src)
    return fail(OXGPU_E_INVALID_ARG, "bad handle, index or pointer");
  if (direction != OXGPU_MG_COPY_TO_DEVICE && direction != OXGPU_MG_COPY_TO_HOST)
    return fail(OXGPU_E_INVALID_ARG, "direction must be OXGPU_MG_COPY_TO_DEVICE or OXGPU_MG_COPY_TO_HOST");
  if (bytes == 0) return OXGPU_OK;
  DeviceGuard guard;
  MG_CUDA(cudaSetDevice(mg->devices[index]));
  MG_CUDA(cudaMemcpyAsync(dst, src, bytes,
                          direction == OXGPU_MG_COPY_TO_DEVICE ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                          mg->stream[index]));
  MG_CUDA(cudaStreamSynchronize(mg->stream[index]));
  return OXGPU_OK;
}

// ---- pinned host memory near a device ---------------------------------------------
// Host-operand calls are PCIe-bound, and on a two-socket host a buffer on the
// far socket crosses the socket interconnect on its way to the GPU.  The pages
// are therefore placed on the NUMA node the device hangs off (the node is read
// from sysfs, the placement is an mbind(2) preference on an anonymous mapping),
// touched, and registered with CUDA as pinned, portable memory.
int oxgpu_b200_host_alloc(size_t bytes, int device, void **ptr) {
  if (!ptr || bytes == 0) return fail(OXGPU_E_INVALID_ARG, "null output pointer or zero size");
  *ptr = nullptr;
  int node = -1;
  if (device >= 0) {
    char bus[32] = {};
    if (cudaDeviceGetPCIBusId(bus, sizeof bus, device) == cudaSuccess) {
      for (char *p = bus; *p; p++)
        if (*p >= 'A' && *p <= 'Z') *p = (char)(*p - 'A' + 'a');
      char path[128];
      std::snprintf(path, sizeof path, "/sys/bus/pci/devices/%s/numa_node", bus);
      if (FILE *f = std::fopen(path, "r")) {
        if (std::fscanf(f, "%d", &node) != 1) node = -1;
        std::fclose(f);
      }
    } else {
      cudaGetLastError();
    }
  }
  const size_t page = (size_t)sysconf(_SC_PAGESIZE);
  const size_t span = (bytes + page - 1) / page * page;
  void *q = mmap(nullptr, span, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (q == MAP_FAILED) return fail(OXGPU_E_INVALID_ARG, "mmap of the host buffer failed");
#ifdef SYS_mbind
  if (node >= 0 && node < 64) {
    unsigned long mask = 1ul << node;
    syscall(SYS_mbind, q, span, 1 /* MPOL_PREFERRED */, &mask, 65ul, 0u);  // a preference: failure is harmless
  }
#endif
  for (size_t off = 0; off < span; off += page) ((volatile char *)q)[off] = 0;  // place the pages now
  cudaError_t e = cudaHostRegister(q, span, cudaHostRegisterPortable);
  if (e != cudaSuccess) {
    munmap(q, span);
    return cuda_fail(e, "cudaHostRegister");
  }
  *ptr = q;
  return OXGPU_OK;
}

int oxgpu_b200_host_free(void *ptr, size_t bytes) {
  if (!ptr) return OXGPU_OK;
  const size_t page = (size_t)sysconf(_SC_PAGESIZE);
  const size_t span = (bytes + page - 1) / page * page;
  cudaError_t e = cudaHostUnregister(ptr);
  munmap(ptr, span);
  if (e != cudaSuccess) return cuda_fail(e, "cudaHostUnregister");
  return OXGPU_OK;
}

}  // extern "C"
