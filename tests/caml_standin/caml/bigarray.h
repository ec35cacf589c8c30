#include "mlvalues.h"
struct caml_ba_array {
  void *data;
  intnat num_dims;
  intnat flags;
  void *proxy;
  intnat dim[16];
};
#define Caml_ba_array_val(v) ((struct caml_ba_array *)((value *)(v) + 1))
#define Caml_ba_data_val(v) (Caml_ba_array_val(v)->data)
uintnat caml_ba_byte_size(struct caml_ba_array *b);
