/* Device-side stand-in for the UPMEM runtime header <defs.h>: tasklet identity.
 * TEST INFRASTRUCTURE ONLY (see ../dpu.h). */
#ifndef LUTAMM_SHIM_DEFS_H
#define LUTAMM_SHIM_DEFS_H
#include <stdint.h>
extern __thread uint32_t shim_tasklet_id;
static inline uint32_t me(void) { return shim_tasklet_id; }
#define __host
#define __dma_aligned __attribute__((aligned(8)))
#endif
