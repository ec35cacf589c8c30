/* oxgpu_b200 -- C ABI of the B200 (sm_100a) dense GEMM path.
 *
 * Plain C: pointers, sizes and ints only.  Every function returns a status:
 *   0   success
 *  <0   contract violation detected on the host before any launch (OXGPU_E_*)
 *  >0   a CUDA runtime/driver error code (cudaError_t / CUresult value)
 * oxgpu_b200_last_error() returns a thread-local message for the last non-zero
 * status.  Nothing here synchronises the device unless the comment says so;
 * launches go to the stream passed in (NULL = the legacy default stream).
 *
 * "Reference" below is the OxCaml compiler project this library is a drop-in
 * for; citations are path:line inside that project.  Both operands are
 * K-contiguous exactly as in the reference: A is [M,K] row-major and B is
 * supplied transposed as B^T [N,K] row-major (test/hardware/run_gemm_h100.cu:
 * 137-148, bench/bench.py:265-271).  C is f32 [M,N] row-major and is
 * overwritten (no alpha/beta), examples/kernels/gemm.ml:147-161.
 */
#ifndef OXGPU_B200_H
#define OXGPU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define OXGPU_API __attribute__((visibility("default")))
#else
#define OXGPU_API
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
  OXGPU_OK = 0,
  OXGPU_E_INVALID_ARG = -1,    /* null pointer, non-positive dimension, bad enum */
  OXGPU_E_CONFIG = -2,         /* tile_config rejected by validate / parse_config */
  OXGPU_E_UNKNOWN_KERNEL = -3, /* no catalog entry of that name / for that tile */
  OXGPU_E_SHAPE = -4,          /* M, N or K not divisible as the entry point requires */
  OXGPU_E_ALIGN = -5,          /* pointer or leading dimension not 16-byte aligned */
  OXGPU_E_TOO_LARGE = -6,      /* exceeds a documented maximum */
  OXGPU_E_DEVICE_TIMEOUT = -7, /* a bounded device-side wait ran out (see device_status) */
  OXGPU_E_NO_DRIVER = -8       /* the CUDA driver entry points could not be resolved */
};

OXGPU_API const char *oxgpu_b200_last_error(void);
OXGPU_API const char *oxgpu_b200_strerror(int status);

/* ---- tile catalog: test/gemm_catalog.ml -------------------------------- */

/* type tile_config (test/gemm_catalog.ml:9-15). */
typedef struct oxgpu_tile_config {
  int bm, bn, bk, stages, producers;
} oxgpu_tile_config;

/* warp_groups / consumers / threads (test/gemm_catalog.ml:17-19): the
 * reference's Hopper CTA width, kept for catalog parity.  The B200 kernels'
 * own launch facts come from oxgpu_b200_kernel_info. */
OXGPU_API int oxgpu_b200_config_threads(const oxgpu_tile_config *c);

/* validate (test/gemm_catalog.ml:21-35).  Returns OXGPU_E_CONFIG with the
 * reference's invalid_arg text in last_error on rejection. */
OXGPU_API int oxgpu_b200_validate_config(const oxgpu_tile_config *c);

/* string_of_config (test/gemm_catalog.ml:37-40):
 * "bm=..,bn=..,bk=..,stages=..,producers=..,threads=..".  Writes at most cap
 * bytes including the terminator. */
OXGPU_API int oxgpu_b200_string_of_config(const oxgpu_tile_config *c, char *buf, size_t cap);

/* parse_config (test/gemm_catalog.ml:42-73): comma-separated key=value, keys
 * bm bn bk producers required, stages defaults to 3, unknown keys ignored,
 * result validated. */
OXGPU_API int oxgpu_b200_parse_config(const char *spec, oxgpu_tile_config *out);

/* tile_catalog (test/gemm_catalog.ml:80-89) in order; entry 0 is the fallback
 * tile hopper_f32 (92-95). */
OXGPU_API int oxgpu_b200_catalog_size(void);
OXGPU_API int oxgpu_b200_catalog_get(int index, oxgpu_tile_config *out);

/* kernel_binding (test/gemm_catalog.ml:101-112): tile -> entry symbol of
 * examples/kernels/gemm.ml:165-199 ("gemm_fast", "gemm_bm128_bn256_s3", ...). */
OXGPU_API int oxgpu_b200_kernel_binding(const oxgpu_tile_config *c, const char **name);

/* choose_config ?m ?n ?k (test/gemm_catalog.ml:114-137): size -> tile. */
OXGPU_API int oxgpu_b200_choose_config(int m, int n, int k, oxgpu_tile_config *out);

/* `emit_gemm_ptx --info` (test/emit_gemm_ptx.ml:39-43): launch facts of a
 * catalog entry.  Reports the B200 kernel with the entry's own tile shape: CTA
 * width, dynamic shared bytes and total shared bytes.  (When M and N are
 * multiples of 256 the entry is launched on the one-CTA 256x256 kernel instead,
 * with the same CTA width and at most 227 KiB of shared memory; the library
 * launches the kernels itself, so these figures are informational.)  `name` is
 * one of the ten entry symbols (examples/kernels/gemm.ml:165-199,
 * gemm_bf16.ml:130-132). */
OXGPU_API int oxgpu_b200_kernel_info(const char *name, int *threads, int *dynamic_smem,
                                     int *total_smem);

/* Tile and input width a catalog entry was specialised for
 * (examples/kernels/gemm.ml:165-199): element_bytes 4 = f32/TF32, 2 = bf16. */
OXGPU_API int oxgpu_b200_kernel_tile(const char *name, oxgpu_tile_config *tile, int *element_bytes);

/* ---- `.gpu` kernel metadata: lib/frontend/gpu_metadata.ml (format 3) -------
 * The adapter writes one tab-separated text file per kernel; its header names
 * the kernel, its CTA width and the type and modes of every argument.  Reading
 * that header lets a caller check that the `.gpu` file it holds describes the
 * catalog entry it is about to launch through this library. */
enum {
  OXGPU_TY_SCALAR_I32 = 1, OXGPU_TY_SCALAR_F32, OXGPU_TY_BOOL, OXGPU_TY_UNIT, OXGPU_TY_BUFFER_F32,
  OXGPU_TY_BUFFER_BF16, OXGPU_TY_BUFFER_F16, OXGPU_TY_TENSOR_MAP, OXGPU_TY_SCALAR_U64
};
enum { OXGPU_OWN_UNIQUE = 1, OXGPU_OWN_ALIASED };
enum { OXGPU_LOC_LOCAL = 1, OXGPU_LOC_GLOBAL };
enum { OXGPU_PORT_PORTABLE = 1, OXGPU_PORT_NONPORTABLE, OXGPU_PORT_UNSPECIFIED };
enum { OXGPU_PERM_READ = 1, OXGPU_PERM_WRITE, OXGPU_PERM_READ_WRITE, OXGPU_PERM_IMMUTABLE };

typedef struct oxgpu_gpu_slot { /* Kernel_ast slot as encoded by `slot` (gpu_metadata.ml:112-128) */
  int type, ownership, locality, portability, permission;
  int start_line, start_col, end_line, end_col;
} oxgpu_gpu_slot;

typedef struct oxgpu_gpu_header {
  char kernel[64];
  int threads;   /* 0 when the file has no `threads` row */
  int nargs;
  oxgpu_gpu_slot args[16];
  oxgpu_gpu_slot result;
} oxgpu_gpu_header;

/* The header part of `parse` (lib/frontend/gpu_metadata.ml:289-343): rows
 * `format 3`, `kernel NAME`, optional `threads N` (1..1024), `arg I <slot>` with
 * contiguous ids, `result <slot>`; the instruction rows that follow are not
 * read.  Failures return OXGPU_E_CONFIG with the reference's Parse_error text. */
OXGPU_API int oxgpu_b200_parse_gpu_header(const char *text, size_t length, oxgpu_gpu_header *out);

/* Does this header describe a GEMM catalog entry this library serves?  The
 * kernel name must be one of the ten entry symbols, `threads` must be the
 * entry's Hopper CTA width 128*(bm/64)+32 (examples/kernels/gemm.ml:165-199),
 * and the arguments must be the entry point's: two tensor maps (aliased, read),
 * a f32 buffer (unique, read_write) and three i32 scalars (gemm.ml:50-53).
 * OXGPU_E_UNKNOWN_KERNEL / OXGPU_E_CONFIG say what does not match. */
OXGPU_API int oxgpu_b200_check_gpu_header(const oxgpu_gpu_header *header);

/* Gpu.grouped_tile_m / grouped_tile_n (tools/exporter/export_prims_index.ml:
 * 40-61; used at examples/kernels/gemm.ml:73-75): the grouped CTA order as a
 * pure function of the linear tile id, the one the persistent scheduler uses. */
OXGPU_API int oxgpu_b200_grouped_tile(int pid, int group, int tiles_m, int tiles_n, int *tile_m,
                                      int *tile_n);
/* The order in which the GEMM kernels of this library visit tiles: the grouped
 * order above, with the columns of every other group of tile rows walked in
 * reverse (the B^T panels used last in one group are used first in the next,
 * while they are still in L2).  Computed with the multiply-by-reciprocal
 * arithmetic the kernels use, so it also serves to check that arithmetic.  No
 * counterpart in the reference, whose kernels walk the plain grouped order. */
OXGPU_API int oxgpu_b200_tile_walk(int pid, int group, int tiles_m, int tiles_n, int *tile_m,
                                   int *tile_n);

/* ---- host launch layer: test/hardware/run_gemm_h100.cu, bench/bench.py -- */

/* Environment variables the launch layer reads (at every launch, so a process
 * may change them between calls); none is needed, all have defaults:
 *   OXGPU_WAIT_BUDGET_MS=<n>      budget of every device-side wait (default 5000)
 *   OXGPU_TILE_SCHEDULE=static    fixed-stride tile walk instead of the tile queue
 *   OXGPU_DEPENDENT_LAUNCH=0      ordinary launches: without it a GEMM kernel may
 *                                 start its set-up under the tail of the kernel
 *                                 before it in the stream (it waits for that kernel
 *                                 before it touches an operand or C)
 *   OXGPU_CLUSTER_REDUCE=dsmem    two-slice in-cluster split-K summed through
 *                                 distributed shared memory, not by TMA reductions
 * Results do not depend on any of them. */

/* encode_tiled_2d (test/hardware/run_gemm_h100.cu:46-72) /
 * encode_tensor_map_2d (bench/bench.py:126-147): 2-D tiled map, 128-byte
 * swizzle, L2 promotion 128 B, no out-of-bounds fill (zeros).  element_bytes 4
 * -> FLOAT32, 2 -> BFLOAT16.  map_out receives the 128-byte CUtensorMap
 * (host memory, 64-byte aligned). */
OXGPU_API int oxgpu_b200_encode_tmap_2d(void *map_out, const void *device_ptr, int element_bytes,
                                        uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                                        uint32_t box0, uint32_t box1);

/* The catalog entry points themselves -- `.visible .entry <name>(a_tmap,
 * b_tmap, c, m, n, k)` (lib/backend/ptx.ml:91-109), launched by
 * test/hardware/run_gemm_h100.cu:183-185 and bench/bench.py:281-292.
 * a_tmap / b_tmap are DEVICE pointers to 128-byte CUtensorMaps encoded as the
 * reference encodes them: A dims (K,M) box (BK,bm), B^T dims (K,N) box
 * (BK,bn) for the tile `name` was specialised for, 128-byte swizzle.  c is a
 * device f32 pointer with row stride (n/bn)*bn = n.  Requires m % bm == 0,
 * n % bn == 0, k % BK == 0 like the reference (bench/bench.py:247-250); BK is
 * 32 for the f32 entries and 64 for gemm_bf16_fast.  The library serves every
 * name with a 128-row (or 256-row) tcgen05 tile, issuing the per-stage loads in
 * units of the caller's boxes (a bm=64 entry by two 64-row loads per 128-row
 * tile; rows past M are zero-filled on load and clipped on store).
 * Replaces cuLaunchKernel(fn, n/bn, m/bm, 1, threads, ...). */
OXGPU_API int oxgpu_b200_gemm_tmap(const char *name, uint64_t a_tmap, uint64_t b_tmap, uint64_t c,
                                   int m, int n, int k, void *stream);

/* Variant selection for the buffer entry points (flags argument). */
enum {
  OXGPU_VARIANT_AUTO = 0,
  OXGPU_VARIANT_1CTA_128x256 = 1, /* one CTA, UMMA 128x256 */
  OXGPU_VARIANT_1CTA_128x128 = 2,
  OXGPU_VARIANT_1CTA_256x128 = 3, /* one CTA, two UMMA 128x128 sharing B */
  OXGPU_VARIANT_2CTA_256x256 = 4, /* CTA pair, cta_group::2 UMMA 256x256 */
  OXGPU_VARIANT_2CTA_256x128 = 5,
  OXGPU_VARIANT_SPLITK = 6,       /* 1-CTA 128x128 tiles over K slices + reduce; needs workspace */
  OXGPU_VARIANT_2CTA_512x256 = 7, /* CTA pair, 256 rows per CTA: two UMMA 256x256 per K step */
  OXGPU_VARIANT_1CTA_256x256 = 8, /* one CTA, two UMMA 128x256 sharing B */
  /* Split-K inside a thread-block cluster: the CTAs of a cluster take the K
   * slices of one 128-row tile and sum them inside the kernel -- two slices by
   * adding both partial tiles to a tile of C the kernel zeroes first (TMA
   * reductions), four or eight through distributed shared memory in ascending
   * order (no workspace, one kernel, the same bits at every launch).  For
   * problems with too few tiles to fill the GPU; OXGPU_FLAG_SPLITS picks the
   * cluster size (2, 4 or 8; 0 = chosen by the library). */
  OXGPU_VARIANT_CLUSTER_SPLITK_128x256 = 9,
  OXGPU_VARIANT_CLUSTER_SPLITK_128x128 = 10,
  /* CTA pair, 256 x 512 per pair: two UMMA 256x256 per K step sharing the staged
   * A rows; each CTA stages 128 rows of A and 256 contiguous rows of B^T.  The
   * tile that serves the reference's 128 x 256 catalog boxes with pair-tile
   * operand traffic. */
  OXGPU_VARIANT_2CTA_256x512 = 11
};
#define OXGPU_FLAG_VARIANT(v) ((unsigned)(v) & 0xffu)
#define OXGPU_FLAG_STAGES(s) (((unsigned)(s) & 0xfu) << 8)    /* 0 = deepest that fits */
#define OXGPU_FLAG_GROUP_M(g) (((unsigned)(g) & 0xffu) << 12) /* 0 = 16, the reference's */
#define OXGPU_FLAG_SPLITS(s) (((unsigned)(s) & 0xffu) << 20)  /* 0 = chosen by the library */
/* Tiles with two row blocks per CTA (256-row variants): K blocks issued
 * block-major at either end of a tile so the epilogue overlaps; 0 = library
 * default, 15 = never, else that many K blocks. */
#define OXGPU_FLAG_REORDER(g) (((unsigned)(g) & 0xfu) << 28)

/* Buffer entry points: the library encodes its own maps, so it may pick any
 * variant (2-CTA tiles, ragged edges).  a: [M,K] row-major with leading
 * dimension lda (elements); bt: B^T [N,K] with ldb; c: f32 [M,N] with ldc.
 * Pointers 16-byte aligned, lda*esize, ldb*esize and ldc*4 multiples of 16.
 * M and N may be ragged; K must make K*esize a multiple of 16.
 * hopper_gemm (examples/kernels/gemm.ml:47-163): TF32-rounded f32 inputs.
 * hopper_gemm_bf16 (examples/kernels/gemm_bf16.ml:33-128): bf16 inputs. */
OXGPU_API int oxgpu_b200_gemm_tf32(const float *a, const float *bt, float *c, int m, int n, int k,
                                   int64_t lda, int64_t ldb, int64_t ldc, unsigned flags,
                                   void *stream);
OXGPU_API int oxgpu_b200_gemm_bf16(const uint16_t *a, const uint16_t *bt, float *c, int m, int n,
                                   int k, int64_t lda, int64_t ldb, int64_t ldc, unsigned flags,
                                   void *stream);

/* bf16 inputs, bf16 OUTPUT (f32 accumulation in TMEM, one round-to-nearest-even
 * at the store): the narrow-output epilogue the reference lists as future work
 * (docs/roadmap.md:67-71).  c: bf16 bits [M,N], ldc a multiple of 8.  Variants:
 * auto, 1CTA_128x256, 1CTA_128x128, 2CTA_256x256, 2CTA_512x256. */
OXGPU_API int oxgpu_b200_gemm_bf16_out16(const uint16_t *a, const uint16_t *bt, uint16_t *c, int m,
                                         int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                                         unsigned flags, void *stream);

/* Same, with caller-provided scratch for OXGPU_VARIANT_SPLITK (f32 partial
 * tiles).  workspace_bytes must be at least
 * oxgpu_b200_splitk_workspace_bytes(m, n, splits). */
OXGPU_API size_t oxgpu_b200_splitk_workspace_bytes(int m, int n, int splits);
OXGPU_API int oxgpu_b200_gemm_bf16_ws(const uint16_t *a, const uint16_t *bt, float *c, int m,
                                      int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                                      unsigned flags, void *workspace, size_t workspace_bytes,
                                      void *stream);

/* f32 operands at close to f32 accuracy on the tensor cores ("3xTF32"): each
 * operand is split into its TF32 part and the exact remainder, and one TF32
 * GEMM over 3K accumulates hi*lo + lo*hi + hi*hi in f32 (the dropped lo*lo term
 * is 2^-20 relative).  For f32-in callers who need the host check's bound
 * 1e-5 * sqrt(K) * max|A| * max|B| against UNROUNDED inputs
 * (test/hardware/run_gemm_h100.cu:150-162 runs on the inputs as given) at more
 * than the exact kernel's CUDA-core rate; plain TF32 misses that bound by a
 * factor of about 20.  K % 4 == 0.  workspace: oxgpu_b200_f32_split_workspace_bytes
 * (m, n, k) = 12 * K * (M + N) bytes, 16-byte aligned, for the split operands.
 * flags as for oxgpu_b200_gemm_tf32 (applied to the M x N x 3K problem). */
OXGPU_API size_t oxgpu_b200_f32_split_workspace_bytes(int m, int n, int k);
OXGPU_API int oxgpu_b200_gemm_f32_split(const float *a, const float *bt, float *c, int m, int n,
                                        int k, int64_t lda, int64_t ldb, int64_t ldc,
                                        unsigned flags, void *workspace, size_t workspace_bytes,
                                        void *stream);

/* GEMM with an affine epilogue: C = alpha * (A B) + beta * C_in + bias, applied to
 * the accumulator on its way from TMEM to the store (the fused epilogue beyond
 * the reference's plain overwrite, examples/kernels/gemm.ml:143-161; its
 * roadmap lists only the narrow output, docs/roadmap.md:67-71).  bias: f32 [N],
 * broadcast over rows, 16-byte aligned, or NULL.  c_in: f32 [M,N] with leading
 * dimension ldc_in, read only when beta != 0 (so it may hold anything, NaN
 * included, when beta == 0); it may be C itself for an in-place update.  Each of
 * the three steps rounds to f32 on its own, in this order:
 * (alpha * acc + beta * c_in) + bias.  Same operand contracts and flags as
 * oxgpu_b200_gemm_bf16 / _tf32; variants: auto, 1CTA_128x128, 2CTA_256x256,
 * 2CTA_512x256. */
typedef struct oxgpu_epilogue {
  float alpha, beta;
  const float *bias;
  const float *c_in;
  int64_t ldc_in;
} oxgpu_epilogue;
OXGPU_API int oxgpu_b200_gemm_bf16_affine(const uint16_t *a, const uint16_t *bt, float *c, int m,
                                          int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                                          const oxgpu_epilogue *epilogue, unsigned flags,
                                          void *stream);
/* The same with bf16 C (bf16 inputs): the affine steps in f32, then one rounding
 * to nearest even.  c_in stays f32.  ldc a multiple of 8. */
OXGPU_API int oxgpu_b200_gemm_bf16_out16_affine(const uint16_t *a, const uint16_t *bt, uint16_t *c,
                                                int m, int n, int k, int64_t lda, int64_t ldb,
                                                int64_t ldc, const oxgpu_epilogue *epilogue,
                                                unsigned flags, void *stream);
OXGPU_API int oxgpu_b200_gemm_tf32_affine(const float *a, const float *bt, float *c, int m, int n,
                                          int k, int64_t lda, int64_t ldb, int64_t ldc,
                                          const oxgpu_epilogue *epilogue, unsigned flags,
                                          void *stream);

/* GEMM with a fan-out epilogue: every tile of C is written to n_dests (1..8)
 * destinations as it leaves the tensor cores.  (No counterpart in the reference,
 * which has no multi-GPU path; this is the "GEMM, then all-gather of the column
 * shards of C" of a column-sharded GEMM done by one kernel.)  c_dests[i] points
 * at the first element of this call's [M,N] window inside destination i, a
 * row-major f32 matrix with leading dimension ldc -- typically
 * C_full_i + column_offset_of_this_rank, with C_full_i the replicated result in
 * GPU i's memory.  A destination may be memory of another GPU that the caller
 * has made addressable (peer access inside one process, or
 * oxgpu_b200_shared_open across processes); tiles then cross NVLink as plain
 * (non-multicast) TMA tile stores while the main loop keeps running, and arrive
 * already interleaved in row-major order.  Same arithmetic, operand contracts and
 * flags as oxgpu_b200_gemm_bf16 / _tf32; variants: auto, 1CTA_128x128,
 * 2CTA_256x256, 2CTA_512x256.  A destination's contents are complete once the
 * work on `stream` has completed on the WRITING GPU; readers on other GPUs
 * need their own ordering after that point (a host barrier, an event). */
OXGPU_API int oxgpu_b200_gemm_bf16_fanout(const uint16_t *a, const uint16_t *bt,
                                          float *const *c_dests, int n_dests, int m, int n, int k,
                                          int64_t lda, int64_t ldb, int64_t ldc, unsigned flags,
                                          void *stream);
OXGPU_API int oxgpu_b200_gemm_tf32_fanout(const float *a, const float *bt, float *const *c_dests,
                                          int n_dests, int m, int n, int k, int64_t lda,
                                          int64_t ldb, int64_t ldc, unsigned flags, void *stream);

/* Device memory other processes on the same machine can map (set-up time, not
 * the hot path): _shared_alloc allocates `bytes` on the current device and
 * fills a 64-byte handle to send to the other processes by any host channel;
 * _shared_open maps a handle received from another process (peer access over
 * NVLink is enabled on first use) and returns a pointer valid in this process;
 * _shared_close unmaps it; _shared_free releases an allocation (after every
 * other process has closed it). */
OXGPU_API int oxgpu_b200_shared_alloc(size_t bytes, void **ptr, unsigned char handle[64]);
OXGPU_API int oxgpu_b200_shared_open(const unsigned char handle[64], void **ptr);
OXGPU_API int oxgpu_b200_shared_close(void *ptr);
OXGPU_API int oxgpu_b200_shared_free(void *ptr);

/* Split-K bf16 GEMM that allocates nothing.  (No counterpart in the reference:
 * its kernels use no scratch memory at all.)
 *
 * For callers that cannot obtain device memory at call time: a process whose
 * device memory is handed out up front by its own arena or by a fixed
 * per-tenant budget, so a late cudaMalloc may fail or is simply not permitted;
 * or a latency-sensitive loop that cannot afford the implicit device-wide
 * synchronisation an allocation or free may cause.  Such a caller passes only
 * its inputs and output; the f32 partial tiles of the K slices live in a
 * fixed array inside the library, OXGPU_STATIC_SCRATCH_BYTES (32 MiB) of device
 * memory that every GPU loading the library holds until the process exits.
 *
 * Same arithmetic and kernels as oxgpu_b200_gemm_bf16_ws with
 * OXGPU_VARIANT_SPLITK; `splits` = number of K slices (0: chosen by the
 * library, at most 16).  The slices need splits * roundup(m,128) * n * 4 bytes;
 * if that exceeds OXGPU_STATIC_SCRATCH_BYTES the call returns OXGPU_E_TOO_LARGE
 * and launches nothing (e.g. m=128, n=8192 allows up to 8 slices).  n % 4 == 0.
 *
 * The first call on each device looks up the array's device address (with that
 * device current) and later calls reuse it.
 * Neither that set-up nor any later call uses cudaMalloc, cudaFree or an
 * allocating library routine.  All calls on a device share the one array and it
 * keeps whatever the previous call left in it; that is harmless here, because
 * every element the reduction reads is overwritten by the same call first, so
 * nothing needs clearing.  Two calls whose kernels overlap on the same GPU
 * (different streams, or different host threads) race on the array: issue them
 * on one stream or otherwise order them. */
#define OXGPU_STATIC_SCRATCH_BYTES (32u << 20)
OXGPU_API int oxgpu_b200_gemm_bf16_splitk_static(const uint16_t *a, const uint16_t *bt, float *c,
                                                 int m, int n, int k, int64_t lda, int64_t ldb,
                                                 int64_t ldc, int splits, void *stream);

/* ---- multi-GPU driver ------------------------------------------------------
 * One process drives up to 8 GPUs of one machine: B^T and C are split by
 * columns (contiguous row blocks of B^T), A is replicated, every device runs
 * the single-GPU kernel on its shard, and nothing crosses NVLink unless a
 * replicated C is asked for.  The reference has no multi-GPU path, so these
 * have no counterpart there; the launcher they sit beside drives one device
 * from one host thread (test/hardware/run_gemm_h100.cu:100-108,183-186).
 * A handle owns one stream, three events and one host thread per device; peer
 * access between its devices is enabled once at creation.  Calls on one handle
 * are not reentrant: issue them from one thread at a time. */
typedef struct oxgpu_mg oxgpu_mg;

#define OXGPU_MG_COLUMN_ALIGN 256 /* shard widths are multiples of the widest tile */

/* The column partition the driver uses, as a pure host function: `parts`
 * contiguous ranges [n0[r], n1[r]) of whole `align`-column blocks, block counts
 * differing by at most one (the first ranges take the extra blocks), the last
 * non-empty range carrying the ragged tail; ranges may be empty when there are
 * fewer blocks than parts. */
OXGPU_API int oxgpu_b200_mg_column_partition(int n, int parts, int align, int *n0, int *n1);

/* devices: CUDA device ordinals (NULL = 0 .. ngpu-1), no repeats.  The caller's
 * current device is left as it was. */
OXGPU_API int oxgpu_b200_mg_create(int ngpu, const int *devices, oxgpu_mg **out);
OXGPU_API int oxgpu_b200_mg_destroy(oxgpu_mg *mg); /* waits for the handle's streams first */
OXGPU_API int oxgpu_b200_mg_device_count(const oxgpu_mg *mg);
OXGPU_API int oxgpu_b200_mg_device(const oxgpu_mg *mg, int index); /* CUDA ordinal of device `index` */
OXGPU_API int oxgpu_b200_mg_peer_access(const oxgpu_mg *mg);       /* 1: every device can store into every other's memory */

enum {
  OXGPU_MG_GATHER_NONE = 0,  /* C stays sharded */
  /* ncclAllGather of the shards over NVLink, then a re-interleave pass on every
   * device: c_full[i] is the row-major C[M,N].  Needs equal shard widths
   * (N a multiple of 256 * devices) and M*N*4 bytes of scratch per device, which
   * the handle allocates on first use and keeps. */
  OXGPU_MG_GATHER_NCCL = 1,
  /* One kernel: each device's GEMM stores every tile into all devices' row-major
   * C[M,N] as it is produced (plain peer stores over NVLink; no peer loads, no
   * multicast).  c_shard is not used.  Needs peer access. */
  OXGPU_MG_GATHER_FUSED = 2,
  /* ncclAllGather only: c_full[i] is block-column-major [devices][M][N/devices],
   * the layout NCCL's contiguous chunks give. */
  OXGPU_MG_GATHER_NCCL_BLOCKS = 3
};

/* C[:, n0_d:n1_d] = A * B[:, n0_d:n1_d] on device d, for the partition above.
 * a_repl[d]: A[M,K] bf16 row-major in device d's memory; bt_shard[d]: rows
 * [n0_d, n1_d) of B^T[N,K]; c_shard[d]: f32 [M, n1_d-n0_d], dense.  All dense
 * (leading dimension = row length) and 16-byte aligned.  c_full[d]: f32 M*N in
 * device d's memory, used when gather_c != NONE.  flags as for
 * oxgpu_b200_gemm_bf16.  Returns once every device's work is enqueued on the
 * handle's streams; oxgpu_b200_mg_sync waits for it.  The pointer arrays need
 * only live until the call returns. */
OXGPU_API int oxgpu_b200_mg_gemm_bf16(oxgpu_mg *mg, const uint16_t *const *a_repl,
                                      const uint16_t *const *bt_shard, float *const *c_shard, int m,
                                      int n, int k, int gather_c, float *const *c_full,
                                      unsigned flags);
OXGPU_API int oxgpu_b200_mg_sync(oxgpu_mg *mg);

/* Device time of the last call, per device (arrays of device_count floats,
 * either may be NULL): total_ms from its first to its last operation, gemm_ms
 * the GEMM alone (the rest is the gather).  Waits for the call to finish. */
OXGPU_API int oxgpu_b200_mg_elapsed_ms(oxgpu_mg *mg, float *total_ms, float *gemm_ms);

/* Host-operand form: A[M,K], B^T[N,K] and C in HOST memory (pinned for full
 * speed).  Every device uploads A and its own rows of B^T, computes its columns
 * block of rows by block of rows and downloads them while the next block comes
 * up.  c_layout: row-major C[M,N] (each device writes its column window, pitch
 * N), or OXGPU_MG_HOST_C_BLOCKS: device d's columns as a contiguous [M][w_d]
 * block at element offset n0_d * M (one long run per device instead of M short
 * ones).  Synchronises: C is complete on the host when it returns.  Device
 * staging buffers are allocated on first use and kept by the handle. */
enum { OXGPU_MG_HOST_C_ROW_MAJOR = 0, OXGPU_MG_HOST_C_BLOCKS = 1 };
OXGPU_API int oxgpu_b200_mg_gemm_bf16_host(oxgpu_mg *mg, const uint16_t *a_host,
                                           const uint16_t *bt_host, float *c_host, int m, int n,
                                           int k, int c_layout, unsigned flags);

/* Device memory and copies for callers with no other CUDA binding (set-up, not
 * the hot path).  `index` counts the handle's devices.  _copy is synchronous. */
enum { OXGPU_MG_COPY_TO_DEVICE = 0, OXGPU_MG_COPY_TO_HOST = 1 };
OXGPU_API int oxgpu_b200_mg_alloc(oxgpu_mg *mg, int index, size_t bytes, void **ptr);
OXGPU_API int oxgpu_b200_mg_free(oxgpu_mg *mg, int index, void *ptr);
OXGPU_API int oxgpu_b200_mg_copy(oxgpu_mg *mg, int index, void *dst, const void *src, size_t bytes,
                                 int direction);

/* Pinned host memory placed on the NUMA node `device` hangs off (device < 0: no
 * placement), for the host-operand entry points: on a two-socket machine a
 * buffer on the far socket crosses the socket interconnect on its way to the
 * GPU.  Portable across devices.  Free with the same byte count. */
OXGPU_API int oxgpu_b200_host_alloc(size_t bytes, int device, void **ptr);
OXGPU_API int oxgpu_b200_host_free(void *ptr, size_t bytes);

/* Exact GEMM on CUDA cores: one f32 accumulator per output, k ascending, a
 * rounded multiply then a rounded add (never fused) -- the arithmetic of the
 * host reference loop (test/hardware/run_gemm_h100.cu:150-162), so the result
 * is bit-identical to that loop.  input_mode: 0 = f32 operands as they are
 * (the path for f32 inputs that must meet the strict 1e-5*sqrt(K) bound),
 * 1 = f32 operands truncated to TF32 first (run_gemm_h100.cu:40-44),
 * 2 = bf16-bit operands widened exactly (32-36).  Also the full-matrix checker
 * for shapes too large for a CPU loop.  lda/ldb/ldc in elements; any M, N, K. */
OXGPU_API int oxgpu_b200_gemm_exact(const void *a, const void *bt, float *c, int m, int n, int k,
                                    int64_t lda, int64_t ldb, int64_t ldc, int input_mode,
                                    void *stream);

/* B[K,N] row-major -> B^T[N,K] row-major on the device, the re-layout the
 * reference performs on the host outside timing (run_gemm_h100.cu:142-148,
 * bench/bench.py:268).  element_bytes 2 or 4. */
OXGPU_API int oxgpu_b200_transpose(const void *b, void *bt, int k, int n, int element_bytes,
                                   void *stream);

/* f32 -> bf16 bits, round-to-nearest-even (run_gemm_h100.cu:26-30). */
OXGPU_API int oxgpu_b200_f32_to_bf16(const float *src, uint16_t *dst, size_t count, void *stream);

/* Both steps in one pass: f32 B[K,N] -> bf16 B^T[N,K] (round to nearest even as
 * above), for a caller holding a row-major f32 B (bench/bench.py:255-271 does the
 * two steps with torch).  K and N multiples of 64, pointers 16-byte aligned. */
OXGPU_API int oxgpu_b200_transpose_f32_to_bf16(const float *b, uint16_t *bt, int k, int n,
                                               void *stream);

/* Host-buffer entry point: A, B^T and C live in HOST memory (pinned or
 * pageable).  Uploads the operands, runs gemm_bf16 and downloads C, pipelined
 * over row blocks of A/C on internal streams; returns after C is complete on
 * the host (this call synchronises).  Device staging buffers are allocated on
 * first use and cached per device, with three streams and their events;
 * oxgpu_b200_release_staging frees all of it.  If a step fails, the work already
 * queued is waited for before the error is returned, so the caller's buffers are
 * no longer in use when the call returns.  A device-side wait that timed out is
 * reported by the next oxgpu_b200_device_status. */
OXGPU_API int oxgpu_b200_gemm_bf16_host(const uint16_t *a_host, const uint16_t *bt_host,
                                        float *c_host, int m, int n, int k, unsigned flags);
OXGPU_API int oxgpu_b200_gemm_tf32_host(const float *a_host, const float *bt_host, float *c_host,
                                        int m, int n, int k, unsigned flags);
/* The same with bf16 C (one rounding to nearest even at the store, as
 * oxgpu_b200_gemm_bf16_out16): half the bytes come back over PCIe, so the call is
 * bound by the upload alone.  N % 8 == 0. */
OXGPU_API int oxgpu_b200_gemm_bf16_out16_host(const uint16_t *a_host, const uint16_t *bt_host,
                                              uint16_t *c_host, int m, int n, int k, unsigned flags);
OXGPU_API int oxgpu_b200_release_staging(void);

/* ---- synthetic operands -------------------------------------------------- */
/* Counter-based generator, value = f(seed, linear index): uniform on [-1,1)
 * (f32) or normal(0,std) (f32 or bf16 bits).  dtype: 4 = f32, 2 = bf16. */
OXGPU_API int oxgpu_b200_fill_uniform(void *dst, size_t count, int element_bytes, uint32_t seed,
                                      uint64_t index_offset, void *stream);
OXGPU_API int oxgpu_b200_fill_normal(void *dst, size_t count, int element_bytes, uint32_t seed,
                                     float std, uint64_t index_offset, void *stream);

/* ---- device status ------------------------------------------------------- */
/* Every device-side wait (mbarrier, TMEM hand-off) has a spin budget.  When
 * one runs out the CTA records {code, block, stage/tile, parity} in a
 * per-device status block and leaves through the normal exit path.  This call
 * synchronises the device, copies the block out (words[0] != 0 means a wait
 * timed out since the last clear) and clears it.  Returns
 * OXGPU_E_DEVICE_TIMEOUT in that case.  The reference's waits are unbounded
 * (lib/backend/ptx.ml:174-181). */
OXGPU_API int oxgpu_b200_device_status(uint32_t words[8]);

/* Number of kernels this library has launched in this process (all entry
 * points), for accounting. */
OXGPU_API uint64_t oxgpu_b200_launch_count(void);

/* Runs the bounded-wait self test: one CTA waits, with the given budget, on a
 * barrier that nothing arrives on.  The wait must give up, the kernel must
 * return normally, and the status block must say so: returns
 * OXGPU_E_DEVICE_TIMEOUT when that happened (the expected outcome), OXGPU_OK
 * if the wait did not time out.  Synchronises the device. */
OXGPU_API int oxgpu_b200_selftest_bounded_wait(uint64_t budget_ns);

/* Library build facts: "sm_100a", CUDA runtime version, variants compiled. */
OXGPU_API const char *oxgpu_b200_build_info(void);

#ifdef __cplusplus
}
#endif
#endif /* OXGPU_B200_H */
