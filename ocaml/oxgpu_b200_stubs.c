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
