void caml_release_runtime_system(void);
void caml_acquire_runtime_system(void);
