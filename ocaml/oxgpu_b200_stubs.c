/* OCaml stubs over the C ABI in include/oxgpu_b200.h (see oxgpu_b200.ml).
 * Source only: built where the OCaml runtime headers exist.  Every stub maps
 * a non-zero status to Failure with the library's message; the host-buffer
 * calls release the runtime lock while the device works. */
#include <caml/alloc.h>
#include <caml/bigarray.h>
#include <caml/fail.h>
#include <caml/memory.h>
#include <caml/mlvalues.h>
#include <caml/threads.h>
#include <string.h>

#include "../include/oxgpu_b200.h"

static void check(int status) {
  if (status != 0) caml_failwith(oxgpu_b200_last_error());
}

static oxgpu_tile_config config_of_value(value v) {
  oxgpu_tile_config c = {Int_val(Field(v, 0)), Int_val(Field(v, 1)), Int_val(Field(v, 2)),
                         Int_val(Field(v, 3)), Int_val(Field(v, 4))};
  return c;
}

static value value_of_config(const oxgpu_tile_config *c) {
  CAMLparam0();
  CAMLlocal1(r);
  r = caml_alloc_tuple(5);
  Store_field(r, 0, Val_int(c->bm));
  Store_field(r, 1, Val_int(c->bn));
  Store_field(r, 2, Val_int(c->bk));
  Store_field(r, 3, Val_int(c->stages));
  Store_field(r, 4, Val_int(c->producers));
  CAMLreturn(r);
}

CAMLprim value oxgpu_ml_validate(value v) {
  CAMLparam1(v);
  oxgpu_tile_config c = config_of_value(v);
  check(oxgpu_b200_validate_config(&c));
  CAMLreturn(v);
}

CAMLprim value oxgpu_ml_parse_config(value spec) {
  CAMLparam1(spec);
  oxgpu_tile_config c;
  check(oxgpu_b200_parse_config(String_val(spec), &c));
  CAMLreturn(value_of_config(&c));
}

CAMLprim value oxgpu_ml_string_of_config(value v) {
  CAMLparam1(v);
  char buf[160];
  oxgpu_tile_config c = config_of_value(v);
  check(oxgpu_b200_string_of_config(&c, buf, sizeof buf));
  CAMLreturn(caml_copy_string(buf));
}

CAMLprim value oxgpu_ml_kernel_binding(value v) {
  CAMLparam1(v);
  const char *name = NULL;
  oxgpu_tile_config c = config_of_value(v);
  check(oxgpu_b200_kernel_binding(&c, &name));
  CAMLreturn(caml_copy_string(name));
}

CAMLprim value oxgpu_ml_choose_config(value m, value n, value k) {
  CAMLparam3(m, n, k);
  oxgpu_tile_config c;
  check(oxgpu_b200_choose_config(Int_val(m), Int_val(n), Int_val(k), &c));
  CAMLreturn(value_of_config(&c));
}

CAMLprim value oxgpu_ml_kernel_info(value name) {
  CAMLparam1(name);
  CAMLlocal1(r);
  int threads, dyn, total;
  check(oxgpu_b200_kernel_info(String_val(name), &threads, &dyn, &total));
  r = caml_alloc_tuple(3);
  Store_field(r, 0, Val_int(threads));
  Store_field(r, 1, Val_int(dyn));
  Store_field(r, 2, Val_int(total));
  CAMLreturn(r);
}

CAMLprim value oxgpu_ml_grouped_tile(value pid, value group, value tm, value tn) {
  CAMLparam4(pid, group, tm, tn);
  CAMLlocal1(r);
  int m, n;
  check(oxgpu_b200_grouped_tile(Int_val(pid), Int_val(group), Int_val(tm), Int_val(tn), &m, &n));
  r = caml_alloc_tuple(2);
  Store_field(r, 0, Val_int(m));
  Store_field(r, 1, Val_int(n));
  CAMLreturn(r);
}

CAMLprim value oxgpu_ml_tile_walk(value pid, value group, value tm, value tn) {
  CAMLparam4(pid, group, tm, tn);
  CAMLlocal1(r);
  int m, n;
  check(oxgpu_b200_tile_walk(Int_val(pid), Int_val(group), Int_val(tm), Int_val(tn), &m, &n));
  r = caml_alloc_tuple(2);
  Store_field(r, 0, Val_int(m));
  Store_field(r, 1, Val_int(n));
  CAMLreturn(r);
}

CAMLprim value oxgpu_ml_gemm_tmap(value name, value a, value b, value c, value m, value n,
                                  value k, value stream) {
  CAMLparam5(name, a, b, c, m);
  CAMLxparam3(n, k, stream);
  check(oxgpu_b200_gemm_tmap(String_val(name), (uint64_t)Nativeint_val(a),
                             (uint64_t)Nativeint_val(b), (uint64_t)Nativeint_val(c), Int_val(m),
                             Int_val(n), Int_val(k), (void *)Nativeint_val(stream)));
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_gemm_tmap_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_gemm_tmap(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7]);
}

#define BUFFER_STUB(NAME, CALL, ATYPE)                                                            \
  CAMLprim value NAME(value a, value bt, value c, value m, value n, value k, value lda,           \
                      value ldb, value ldc, value flags, value stream) {                          \
    CAMLparam5(a, bt, c, m, n);                                                                   \
    CAMLxparam5(k, lda, ldb, ldc, flags);                                                         \
    CAMLxparam1(stream);                                                                          \
    check(CALL((const ATYPE *)Nativeint_val(a), (const ATYPE *)Nativeint_val(bt),                 \
               (float *)Nativeint_val(c), Int_val(m), Int_val(n), Int_val(k), Int_val(lda),       \
               Int_val(ldb), Int_val(ldc), (unsigned)Int_val(flags),                              \
               (void *)Nativeint_val(stream)));                                                   \
    CAMLreturn(Val_unit);                                                                         \
  }                                                                                               \
  CAMLprim value NAME##_byte(value *argv, int argn) {                                             \
    (void)argn;                                                                                   \
    return NAME(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7], argv[8],  \
                argv[9], argv[10]);                                                               \
  }

BUFFER_STUB(oxgpu_ml_gemm_bf16, oxgpu_b200_gemm_bf16, uint16_t)
BUFFER_STUB(oxgpu_ml_gemm_tf32, oxgpu_b200_gemm_tf32, float)

CAMLprim value oxgpu_ml_gemm_bf16_host(value a, value bt, value c, value flags) {
  CAMLparam4(a, bt, c, flags);
  int m = (int)Caml_ba_array_val(a)->dim[0], k = (int)Caml_ba_array_val(a)->dim[1];
  int n = (int)Caml_ba_array_val(bt)->dim[0];
  if (Caml_ba_array_val(bt)->dim[1] != k || Caml_ba_array_val(c)->dim[0] != m ||
      Caml_ba_array_val(c)->dim[1] != n)
    caml_invalid_argument("gemm_bf16_host: expected A[M,K], B^T[N,K], C[M,N]");
  const uint16_t *pa = Caml_ba_data_val(a), *pb = Caml_ba_data_val(bt);
  float *pc = Caml_ba_data_val(c);
  unsigned f = (unsigned)Int_val(flags);
  caml_release_runtime_system(); /* Bigarray data does not move */
  int st = oxgpu_b200_gemm_bf16_host(pa, pb, pc, m, n, k, f);
  caml_acquire_runtime_system();
  check(st);
  CAMLreturn(Val_unit);
}

CAMLprim value oxgpu_ml_gemm_tf32_host(value a, value bt, value c, value flags) {
  CAMLparam4(a, bt, c, flags);
  int m = (int)Caml_ba_array_val(a)->dim[0], k = (int)Caml_ba_array_val(a)->dim[1];
  int n = (int)Caml_ba_array_val(bt)->dim[0];
  if (Caml_ba_array_val(bt)->dim[1] != k || Caml_ba_array_val(c)->dim[0] != m ||
      Caml_ba_array_val(c)->dim[1] != n)
    caml_invalid_argument("gemm_tf32_host: expected A[M,K], B^T[N,K], C[M,N]");
  const float *pa = Caml_ba_data_val(a), *pb = Caml_ba_data_val(bt);
  float *pc = Caml_ba_data_val(c);
  unsigned f = (unsigned)Int_val(flags);
  caml_release_runtime_system();
  int st = oxgpu_b200_gemm_tf32_host(pa, pb, pc, m, n, k, f);
  caml_acquire_runtime_system();
  check(st);
  CAMLreturn(Val_unit);
}

CAMLprim value oxgpu_ml_device_status(value unit) {
  CAMLparam1(unit);
  check(oxgpu_b200_device_status(NULL));
  CAMLreturn(Val_unit);
}

/* The host-buffer calls above return when C is complete on the host; a bounded
 * device-side wait that ran out during the call is only recorded on the device.
 * These variants ask for it before returning, so a timed-out kernel surfaces as
 * Failure from the call that ran it. */
CAMLprim value oxgpu_ml_gemm_bf16_host_checked(value a, value bt, value c, value flags) {
  CAMLparam4(a, bt, c, flags);
  oxgpu_ml_gemm_bf16_host(a, bt, c, flags);
  check(oxgpu_b200_device_status(NULL));
  CAMLreturn(Val_unit);
}

CAMLprim value oxgpu_ml_gemm_tf32_host_checked(value a, value bt, value c, value flags) {
  CAMLparam4(a, bt, c, flags);
  oxgpu_ml_gemm_tf32_host(a, bt, c, flags);
  check(oxgpu_b200_device_status(NULL));
  CAMLreturn(Val_unit);
}

/* encode_tiled_2d (test/hardware/run_gemm_h100.cu:46-72): returns the 128-byte
 * CUtensorMap as an OCaml string; the caller copies it to device memory
 * (mg_copy_to_device) as the reference's harness does (run_gemm_h100.cu:174-181). */
CAMLprim value oxgpu_ml_encode_tmap_2d(value ptr, value esize, value dim0, value dim1, value stride1,
                                       value box0, value box1) {
  CAMLparam5(ptr, esize, dim0, dim1, stride1);
  CAMLxparam2(box0, box1);
  CAMLlocal1(r);
  char raw[192];
  char *aligned = (char *)(((uintptr_t)raw + 63u) & ~(uintptr_t)63u);
  check(oxgpu_b200_encode_tmap_2d(aligned, (const void *)Nativeint_val(ptr), Int_val(esize),
                                  (uint64_t)Long_val(dim0), (uint64_t)Long_val(dim1),
                                  (uint64_t)Long_val(stride1), (uint32_t)Int_val(box0),
                                  (uint32_t)Int_val(box1)));
  r = caml_alloc_string(128);
  memcpy(Bytes_val(r), aligned, 128);
  CAMLreturn(r);
}
CAMLprim value oxgpu_ml_encode_tmap_2d_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_encode_tmap_2d(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6]);
}

CAMLprim value oxgpu_ml_gemm_exact(value a, value bt, value c, value m, value n, value k, value lda,
                                   value ldb, value ldc, value mode, value stream) {
  CAMLparam5(a, bt, c, m, n);
  CAMLxparam5(k, lda, ldb, ldc, mode);
  CAMLxparam1(stream);
  check(oxgpu_b200_gemm_exact((const void *)Nativeint_val(a), (const void *)Nativeint_val(bt),
                              (float *)Nativeint_val(c), Int_val(m), Int_val(n), Int_val(k),
                              Int_val(lda), Int_val(ldb), Int_val(ldc), Int_val(mode),
                              (void *)Nativeint_val(stream)));
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_gemm_exact_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_gemm_exact(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7],
                             argv[8], argv[9], argv[10]);
}

CAMLprim value oxgpu_ml_transpose(value b, value bt, value k, value n, value esize, value stream) {
  CAMLparam5(b, bt, k, n, esize);
  CAMLxparam1(stream);
  check(oxgpu_b200_transpose((const void *)Nativeint_val(b), (void *)Nativeint_val(bt), Int_val(k),
                             Int_val(n), Int_val(esize), (void *)Nativeint_val(stream)));
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_transpose_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_transpose(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5]);
}

CAMLprim value oxgpu_ml_fill_uniform(value dst, value count, value esize, value seed, value offset,
                                     value stream) {
  CAMLparam5(dst, count, esize, seed, offset);
  CAMLxparam1(stream);
  check(oxgpu_b200_fill_uniform((void *)Nativeint_val(dst), (size_t)Long_val(count), Int_val(esize),
                                (uint32_t)Long_val(seed), (uint64_t)Long_val(offset),
                                (void *)Nativeint_val(stream)));
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_fill_uniform_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_fill_uniform(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5]);
}

CAMLprim value oxgpu_ml_fill_normal(value dst, value count, value esize, value seed, value std,
                                    value offset, value stream) {
  CAMLparam5(dst, count, esize, seed, std);
  CAMLxparam2(offset, stream);
  check(oxgpu_b200_fill_normal((void *)Nativeint_val(dst), (size_t)Long_val(count), Int_val(esize),
                               (uint32_t)Long_val(seed), (float)Double_val(std),
                               (uint64_t)Long_val(offset), (void *)Nativeint_val(stream)));
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_fill_normal_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_fill_normal(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6]);
}

/* ---- multi-GPU driver (oxgpu_b200_mg_*): the handle is a nativeint --------------- */

CAMLprim value oxgpu_ml_mg_column_partition(value n, value parts, value align) {
  CAMLparam3(n, parts, align);
  CAMLlocal2(r, pair);
  int count = Int_val(parts), lo[64], hi[64];
  if (count < 1 || count > 64) caml_invalid_argument("mg_column_partition: between 1 and 64 parts");
  check(oxgpu_b200_mg_column_partition(Int_val(n), count, Int_val(align), lo, hi));
  r = caml_alloc_tuple(count);
  for (int i = 0; i < count; i++) {
    pair = caml_alloc_tuple(2);
    Store_field(pair, 0, Val_int(lo[i]));
    Store_field(pair, 1, Val_int(hi[i]));
    Store_field(r, i, pair);
  }
  CAMLreturn(r);
}

CAMLprim value oxgpu_ml_mg_create(value devices) { /* int array of CUDA ordinals */
  CAMLparam1(devices);
  int n = (int)Wosize_val(devices), dev[8];
  if (n < 1 || n > 8) caml_invalid_argument("mg_create: between 1 and 8 devices");
  for (int i = 0; i < n; i++) dev[i] = Int_val(Field(devices, i));
  oxgpu_mg *mg = NULL;
  check(oxgpu_b200_mg_create(n, dev, &mg));
  CAMLreturn(caml_copy_nativeint((intnat)mg));
}

CAMLprim value oxgpu_ml_mg_destroy(value mg) {
  CAMLparam1(mg);
  check(oxgpu_b200_mg_destroy((oxgpu_mg *)Nativeint_val(mg)));
  CAMLreturn(Val_unit);
}

CAMLprim value oxgpu_ml_mg_alloc(value mg, value index, value bytes) {
  CAMLparam3(mg, index, bytes);
  void *p = NULL;
  check(oxgpu_b200_mg_alloc((oxgpu_mg *)Nativeint_val(mg), Int_val(index), (size_t)Long_val(bytes), &p));
  CAMLreturn(caml_copy_nativeint((intnat)p));
}

CAMLprim value oxgpu_ml_mg_free(value mg, value index, value ptr) {
  CAMLparam3(mg, index, ptr);
  check(oxgpu_b200_mg_free((oxgpu_mg *)Nativeint_val(mg), Int_val(index), (void *)Nativeint_val(ptr)));
  CAMLreturn(Val_unit);
}

/* host -> device from an OCaml string (a tensor map, a small table) */
CAMLprim value oxgpu_ml_mg_copy_string_to_device(value mg, value index, value dst, value src) {
  CAMLparam4(mg, index, dst, src);
  check(oxgpu_b200_mg_copy((oxgpu_mg *)Nativeint_val(mg), Int_val(index), (void *)Nativeint_val(dst),
                           String_val(src), caml_string_length(src), OXGPU_MG_COPY_TO_DEVICE));
  CAMLreturn(Val_unit);
}

/* host <-> device on a Bigarray of any element kind (whole array) */
CAMLprim value oxgpu_ml_mg_copy_to_device(value mg, value index, value dst, value src) {
  CAMLparam4(mg, index, dst, src);
  check(oxgpu_b200_mg_copy((oxgpu_mg *)Nativeint_val(mg), Int_val(index), (void *)Nativeint_val(dst),
                           Caml_ba_data_val(src), caml_ba_byte_size(Caml_ba_array_val(src)),
                           OXGPU_MG_COPY_TO_DEVICE));
  CAMLreturn(Val_unit);
}

CAMLprim value oxgpu_ml_mg_copy_to_host(value mg, value index, value dst, value src) {
  CAMLparam4(mg, index, dst, src);
  check(oxgpu_b200_mg_copy((oxgpu_mg *)Nativeint_val(mg), Int_val(index), Caml_ba_data_val(dst),
                           (const void *)Nativeint_val(src), caml_ba_byte_size(Caml_ba_array_val(dst)),
                           OXGPU_MG_COPY_TO_HOST));
  CAMLreturn(Val_unit);
}

/* a_repl, bt_shard, c_shard, c_full: nativeint arrays, one device pointer per
 * device (c_shard / c_full may be empty arrays when the gather mode does not
 * use them) */
CAMLprim value oxgpu_ml_mg_gemm_bf16(value mg, value a, value bt, value c, value m, value n, value k,
                                     value gather, value full, value flags) {
  CAMLparam5(mg, a, bt, c, m);
  CAMLxparam5(n, k, gather, full, flags);
  oxgpu_mg *h = (oxgpu_mg *)Nativeint_val(mg);
  int g = oxgpu_b200_mg_device_count(h);
  const uint16_t *pa[8], *pb[8];
  float *pc[8], *pf[8];
  if (g < 1 || g > 8 || (int)Wosize_val(a) != g || (int)Wosize_val(bt) != g ||
      (Wosize_val(c) != 0 && (int)Wosize_val(c) != g) || (Wosize_val(full) != 0 && (int)Wosize_val(full) != g))
    caml_invalid_argument("mg_gemm_bf16: one pointer per device");
  for (int i = 0; i < g; i++) {
    pa[i] = (const uint16_t *)Nativeint_val(Field(a, i));
    pb[i] = (const uint16_t *)Nativeint_val(Field(bt, i));
    pc[i] = Wosize_val(c) ? (float *)Nativeint_val(Field(c, i)) : NULL;
    pf[i] = Wosize_val(full) ? (float *)Nativeint_val(Field(full, i)) : NULL;
  }
  check(oxgpu_b200_mg_gemm_bf16(h, pa, pb, Wosize_val(c) ? pc : NULL, Int_val(m), Int_val(n), Int_val(k),
                                Int_val(gather), Wosize_val(full) ? pf : NULL, (unsigned)Int_val(flags)));
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_mg_gemm_bf16_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_mg_gemm_bf16(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7],
                               argv[8], argv[9]);
}

CAMLprim value oxgpu_ml_mg_sync(value mg) {
  CAMLparam1(mg);
  oxgpu_mg *h = (oxgpu_mg *)Nativeint_val(mg);
  caml_release_runtime_system();
  int st = oxgpu_b200_mg_sync(h);
  caml_acquire_runtime_system();
  check(st);
  CAMLreturn(Val_unit);
}

CAMLprim value oxgpu_ml_mg_elapsed_ms(value mg) { /* float array: total device ms per device */
  CAMLparam1(mg);
  CAMLlocal1(r);
  oxgpu_mg *h = (oxgpu_mg *)Nativeint_val(mg);
  int g = oxgpu_b200_mg_device_count(h);
  float ms[8];
  if (g < 1 || g > 8) caml_invalid_argument("mg_elapsed_ms: bad handle");
  check(oxgpu_b200_mg_elapsed_ms(h, ms, NULL));
  r = caml_alloc_float_array(g);
  for (int i = 0; i < g; i++) Store_double_flat_field(r, i, (double)ms[i]);
  CAMLreturn(r);
}

CAMLprim value oxgpu_ml_mg_gemm_bf16_host(value mg, value a, value bt, value c, value layout, value flags) {
  CAMLparam5(mg, a, bt, c, layout);
  CAMLxparam1(flags);
  int m = (int)Caml_ba_array_val(a)->dim[0], k = (int)Caml_ba_array_val(a)->dim[1];
  int n = (int)Caml_ba_array_val(bt)->dim[0];
  if (Caml_ba_array_val(bt)->dim[1] != k ||
      Caml_ba_array_val(c)->dim[0] * Caml_ba_array_val(c)->dim[1] != (intnat)m * n)
    caml_invalid_argument("mg_gemm_bf16_host: expected A[M,K], B^T[N,K] and M*N elements of C");
  oxgpu_mg *h = (oxgpu_mg *)Nativeint_val(mg);
  const uint16_t *pa = Caml_ba_data_val(a), *pb = Caml_ba_data_val(bt);
  float *pc = Caml_ba_data_val(c);
  int lay = Int_val(layout);
  unsigned f = (unsigned)Int_val(flags);
  caml_release_runtime_system();
  int st = oxgpu_b200_mg_gemm_bf16_host(h, pa, pb, pc, m, n, k, lay, f);
  caml_acquire_runtime_system();
  check(st);
  CAMLreturn(Val_unit);
}
CAMLprim value oxgpu_ml_mg_gemm_bf16_host_byte(value *argv, int argn) {
  (void)argn;
  return oxgpu_ml_mg_gemm_bf16_host(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5]);
}

/* bf16 C on the host (bits as uint16): half the bytes come back over PCIe. */
CAMLprim value oxgpu_ml_gemm_bf16_out16_host(value a, value bt, value c, value flags) {
  CAMLparam4(a, bt, c, flags);
  int m = (int)Caml_ba_array_val(a)->dim[0], k = (int)Caml_ba_array_val(a)->dim[1];
  int n = (int)Caml_ba_array_val(bt)->dim[0];
  if (Caml_ba_array_val(bt)->dim[1] != k || Caml_ba_array_val(c)->dim[0] != m ||
      Caml_ba_array_val(c)->dim[1] != n)
    caml_invalid_argument("gemm_bf16_out16_host: expected A[M,K], B^T[N,K], C[M,N]");
  const uint16_t *pa = Caml_ba_data_val(a), *pb = Caml_ba_data_val(bt);
  uint16_t *pc = Caml_ba_data_val(c);
  unsigned f = (unsigned)Int_val(flags);
  caml_release_runtime_system();
  int st = oxgpu_b200_gemm_bf16_out16_host(pa, pb, pc, m, n, k, f);
  caml_acquire_runtime_system();
  check(st);
  CAMLreturn(Val_unit);
}
