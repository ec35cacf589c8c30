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
