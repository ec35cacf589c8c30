/* Stand-in for the OCaml runtime's C headers, for `gcc -fsyntax-only` on
 * ocaml/oxgpu_b200_stubs.c where no OCaml toolchain exists: just enough
 * declarations, with the runtime's public names and argument types, for the
 * compiler to check every stub's arity and every argument it passes to the
 * library.  Nothing here is ever linked or run. */
#ifndef OXGPU_CAML_STANDIN_H
#define OXGPU_CAML_STANDIN_H
#include <stddef.h>
#include <stdint.h>
typedef intptr_t intnat;
typedef uintptr_t uintnat;
typedef intnat value;
typedef uintnat mlsize_t;
#define CAMLprim
#define Val_unit ((value)1)
#define Val_int(x) ((value)(((intnat)(x) << 1) + 1))
#define Int_val(v) ((int)((v) >> 1))
#define Long_val(v) ((intnat)((v) >> 1))
#define Field(v, i) (((value *)(v))[i])
#define Wosize_val(v) ((mlsize_t)(((uintnat *)(v))[-1] >> 10))
#define String_val(v) ((const char *)(v))
#define Bytes_val(v) ((unsigned char *)(v))
#define Nativeint_val(v) (*((intnat *)(v) + 1))
#define Double_val(v) (*(double *)(v))
#define Store_double_flat_field(v, i, d) (((double *)(v))[i] = (d))
void caml_modify(value *slot, value v);
#define Store_field(block, i, v) caml_modify(&Field(block, i), v)
mlsize_t caml_string_length(value s);
#endif
