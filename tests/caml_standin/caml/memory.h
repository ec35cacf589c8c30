#include "mlvalues.h"
#define CAMLparam0() int caml__frame = 0
#define CAMLparam1(a) int caml__frame = 0; (void)(a)
#define CAMLparam2(a, b) CAMLparam1(a); (void)(b)
#define CAMLparam3(a, b, c) CAMLparam2(a, b); (void)(c)
#define CAMLparam4(a, b, c, d) CAMLparam3(a, b, c); (void)(d)
#define CAMLparam5(a, b, c, d, e) CAMLparam4(a, b, c, d); (void)(e)
#define CAMLxparam1(a) (void)(a)
#define CAMLxparam2(a, b) (void)(a); (void)(b)
#define CAMLxparam3(a, b, c) CAMLxparam2(a, b); (void)(c)
#define CAMLxparam4(a, b, c, d) CAMLxparam3(a, b, c); (void)(d)
#define CAMLxparam5(a, b, c, d, e) CAMLxparam4(a, b, c, d); (void)(e)
#define CAMLlocal1(a) value a = Val_unit
#define CAMLlocal2(a, b) value a = Val_unit, b = Val_unit
#define CAMLreturn(x) do { (void)caml__frame; return (x); } while (0)
