(* OCaml host bindings for liboxgpu_b200.so: the B200 replacement for launching
   the catalog entry points of examples/kernels/gemm.ml and gemm_bf16.ml.

   The reference has no OCaml host launcher (its Gpu.* externals in
   lib/dsl/gpu_dsl.ml are device-primitive markers for the compiler, and its
   kernels are launched from C and Python: test/hardware/run_gemm_h100.cu,
   bench/bench.py).  These externals give OCaml code the same launch surface
   through the C ABI in include/oxgpu_b200.h.  Device pointers and streams are
   nativeint (a CUdeviceptr / CUstream); statuses other than 0 raise Failure
   with the library's message.

   Source only: it is compiled where an OCaml toolchain exists, e.g.
     ocamlfind ocamlopt -package bigarray oxgpu_b200_stubs.c oxgpu_b200.ml \
       -cclib -loxgpu_b200 *)

type tile_config = { bm : int; bn : int; bk : int; stages : int; producers : int }
(* = Gemm_catalog.tile_config, test/gemm_catalog.ml:9-15 *)

(* catalog: test/gemm_catalog.ml and test/emit_gemm_ptx.ml *)
external validate : tile_config -> tile_config = "oxgpu_ml_validate"
external parse_config : string -> tile_config = "oxgpu_ml_parse_config"
external string_of_config : tile_config -> string = "oxgpu_ml_string_of_config"
external kernel_binding : tile_config -> string = "oxgpu_ml_kernel_binding"
external choose_config_raw : int -> int -> int -> tile_config = "oxgpu_ml_choose_config"
external kernel_info : string -> int * int * int = "oxgpu_ml_kernel_info"
external grouped_tile : int -> int -> int -> int -> int * int = "oxgpu_ml_grouped_tile"
(* the order this library's kernels visit tiles in (grouped, every other group of tile rows reversed) *)
external tile_walk : int -> int -> int -> int -> int * int = "oxgpu_ml_tile_walk"

let choose_config ?(m = 4096) ?(n = 4096) ?(k = 4096) () = choose_config_raw m n k

(* Catalog entry point: name, device pointers to the A and B^T tensor maps,
   device pointer to C, m, n, k, stream.  More than five arguments, so a
   bytecode and a native stub (lib/backend/ptx.ml:91-109 is the kernel
   signature this mirrors). *)
external gemm_tmap :
  string -> nativeint -> nativeint -> nativeint -> int -> int -> int -> nativeint -> unit
  = "oxgpu_ml_gemm_tmap_byte" "oxgpu_ml_gemm_tmap"

(* Buffer entry points: A[M,K], B^T[N,K], C[M,N] device pointers, m n k,
   leading dimensions in elements, flags, stream. *)
external gemm_bf16 :
  nativeint -> nativeint -> nativeint -> int -> int -> int -> int -> int -> int -> int ->
  nativeint -> unit
  = "oxgpu_ml_gemm_bf16_byte" "oxgpu_ml_gemm_bf16"

external gemm_tf32 :
  nativeint -> nativeint -> nativeint -> int -> int -> int -> int -> int -> int -> int ->
  nativeint -> unit
  = "oxgpu_ml_gemm_tf32_byte" "oxgpu_ml_gemm_tf32"

(* Host-buffer entry points on Bigarrays (bf16 as uint16 bits). *)
external gemm_bf16_host :
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t -> int -> unit
  = "oxgpu_ml_gemm_bf16_host"

external gemm_tf32_host :
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t -> int -> unit
  = "oxgpu_ml_gemm_tf32_host"

(* Synchronises the device; raises if a bounded device-side wait timed out. *)
external device_status : unit -> unit = "oxgpu_ml_device_status"

(* The same, followed by a device-status query: a bounded device-side wait
   that ran out during the call raises Failure here instead of at a later
   device_status. *)
external gemm_bf16_host_checked :
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t -> int -> unit
  = "oxgpu_ml_gemm_bf16_host_checked"

external gemm_tf32_host_checked :
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t -> int -> unit
  = "oxgpu_ml_gemm_tf32_host_checked"

(* encode_tiled_2d (test/hardware/run_gemm_h100.cu:46-72): device pointer,
   element bytes (4 = f32, 2 = bf16), dim0, dim1, stride1 in bytes, box0, box1 ->
   the 128-byte CUtensorMap.  Copy it to device memory with
   mg_copy_string_to_device and pass that address to gemm_tmap, as the
   reference's harness does (run_gemm_h100.cu:174-181). *)
external encode_tmap_2d : nativeint -> int -> int -> int -> int -> int -> int -> string
  = "oxgpu_ml_encode_tmap_2d_byte" "oxgpu_ml_encode_tmap_2d"

(* The host loop's arithmetic on the device, bit for bit
   (run_gemm_h100.cu:150-162): a, bt, c, m n k, lda ldb ldc, input mode
   (0 = f32, 1 = f32 truncated to TF32, 2 = bf16 bits), stream. *)
external gemm_exact :
  nativeint -> nativeint -> nativeint -> int -> int -> int -> int -> int -> int -> int ->
  nativeint -> unit
  = "oxgpu_ml_gemm_exact_byte" "oxgpu_ml_gemm_exact"

(* B[K,N] -> B^T[N,K] on the device (run_gemm_h100.cu:142-148): b, bt, k, n,
   element bytes, stream. *)
external transpose : nativeint -> nativeint -> int -> int -> int -> nativeint -> unit
  = "oxgpu_ml_transpose_byte" "oxgpu_ml_transpose"

(* Synthetic operands: dst, count, element bytes, seed, [std,] index offset, stream. *)
external fill_uniform : nativeint -> int -> int -> int -> int -> nativeint -> unit
  = "oxgpu_ml_fill_uniform_byte" "oxgpu_ml_fill_uniform"
external fill_normal : nativeint -> int -> int -> int -> float -> int -> nativeint -> unit
  = "oxgpu_ml_fill_normal_byte" "oxgpu_ml_fill_normal"

(* ---- multi-GPU driver: one process, up to 8 GPUs, B^T and C split by columns ---- *)
type mg = nativeint

let gather_none = 0 and gather_nccl = 1 and gather_fused = 2 and gather_nccl_blocks = 3
let host_c_row_major = 0 and host_c_blocks = 1

external mg_column_partition : int -> int -> int -> (int * int) array = "oxgpu_ml_mg_column_partition"
external mg_create : int array -> mg = "oxgpu_ml_mg_create"
external mg_destroy : mg -> unit = "oxgpu_ml_mg_destroy"
external mg_alloc : mg -> int -> int -> nativeint = "oxgpu_ml_mg_alloc"
external mg_free : mg -> int -> nativeint -> unit = "oxgpu_ml_mg_free"
external mg_copy_string_to_device : mg -> int -> nativeint -> string -> unit
  = "oxgpu_ml_mg_copy_string_to_device"
external mg_copy_to_device : mg -> int -> nativeint -> ('a, 'b, Bigarray.c_layout) Bigarray.Genarray.t -> unit
  = "oxgpu_ml_mg_copy_to_device"
external mg_copy_to_host : mg -> int -> ('a, 'b, Bigarray.c_layout) Bigarray.Genarray.t -> nativeint -> unit
  = "oxgpu_ml_mg_copy_to_host"

(* handle, A replicas, B^T shards, C shards, m n k, gather mode, full C per
   device, flags.  Returns when the work is enqueued; mg_sync waits. *)
external mg_gemm_bf16 :
  mg -> nativeint array -> nativeint array -> nativeint array -> int -> int -> int -> int ->
  nativeint array -> int -> unit
  = "oxgpu_ml_mg_gemm_bf16_byte" "oxgpu_ml_mg_gemm_bf16"
external mg_sync : mg -> unit = "oxgpu_ml_mg_sync"
external mg_elapsed_ms : mg -> float array = "oxgpu_ml_mg_elapsed_ms"

(* Operands and result on the host: handle, A, B^T, C, C layout, flags. *)
external mg_gemm_bf16_host :
  mg ->
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array2.t -> int -> int -> unit
  = "oxgpu_ml_mg_gemm_bf16_host_byte" "oxgpu_ml_mg_gemm_bf16_host"

(* Host operands, bf16 C (bits as uint16): half the bytes come back over PCIe. *)
external gemm_bf16_out16_host :
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t ->
  (int, Bigarray.int16_unsigned_elt, Bigarray.c_layout) Bigarray.Array2.t -> int -> unit
  = "oxgpu_ml_gemm_bf16_out16_host"
