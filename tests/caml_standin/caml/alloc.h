#include "mlvalues.h"
value caml_alloc_tuple(mlsize_t n);
value caml_alloc_string(mlsize_t len);
value caml_copy_string(const char *s);
value caml_copy_nativeint(intnat i);
value caml_alloc_float_array(mlsize_t len);
