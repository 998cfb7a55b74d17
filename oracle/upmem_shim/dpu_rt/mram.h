/* Device-side stand-in for <mram.h>: MRAM is ordinary memory, a DMA is a memcpy.
 * TEST INFRASTRUCTURE ONLY (see ../dpu.h). */
#ifndef LUTAMM_SHIM_MRAM_H
#define LUTAMM_SHIM_MRAM_H
#include <string.h>
#define __mram_noinit
#define __mram
#define __mram_ptr
static inline void mram_read(const void* from_mram, void* to_wram, unsigned nb_bytes) { memcpy(to_wram, from_mram, nb_bytes); }
static inline void mram_write(const void* from_wram, void* to_mram, unsigned nb_bytes) { memcpy(to_mram, from_wram, nb_bytes); }
#endif
