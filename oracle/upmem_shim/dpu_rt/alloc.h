/* Device-side stand-in for <alloc.h> (the kernel includes it but allocates nothing).
 * TEST INFRASTRUCTURE ONLY (see ../dpu.h). */
#ifndef LUTAMM_SHIM_ALLOC_H
#define LUTAMM_SHIM_ALLOC_H
#include <stdlib.h>
static inline void* mem_alloc(size_t n) { return malloc(n); }
static inline void mem_reset(void) {}
#endif
