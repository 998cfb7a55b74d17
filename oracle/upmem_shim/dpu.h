/*
 * Host-side stand-in for the UPMEM SDK header <dpu.h>.
 *
 * TEST INFRASTRUCTURE ONLY.  The reference's LUT path (inference-engine/src/host/
 * pim_lut_host.cpp, amm_host.cpp) is written against the UPMEM host API, which is not
 * installed here and cannot be fetched.  This header declares the dozen calls that code
 * uses, with the SDK's names and argument order, so the reference sources compile
 * UNMODIFIED; dpu_shim.cpp implements them on host threads: a "DPU" is an instance of
 * the reference's own DPU kernel (src/dpu/pim_lut_kernel.c, also unmodified, built as a
 * shared object with the headers in dpu_rt/), its MRAM symbols are the kernel's global
 * arrays, a launch runs the kernel's main() on NR_TASKLETS threads.  It is a functional
 * model: results are the reference's, timings are not UPMEM timings.
 */
#ifndef LUTAMM_SHIM_DPU_H
#define LUTAMM_SHIM_DPU_H
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h> /* the SDK header brings this in; amm_host.cpp relies on it for memset */

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { DPU_OK = 0, DPU_ERR_SHIM = 1 } dpu_error_t;
typedef enum { DPU_XFER_TO_DPU = 0, DPU_XFER_FROM_DPU = 1 } dpu_xfer_t;
typedef enum { DPU_XFER_DEFAULT = 0, DPU_XFER_ASYNC = 1 } dpu_xfer_flags_t;
typedef enum { DPU_SYNCHRONOUS = 0, DPU_ASYNCHRONOUS = 1 } dpu_launch_policy_t;

struct shim_set;
struct dpu_set_t {
    struct shim_set* impl;
    int32_t single; /* -1: the whole set; otherwise the index of one DPU */
};

dpu_error_t dpu_alloc(uint32_t nr_dpus, const char* profile, struct dpu_set_t* set);
dpu_error_t dpu_alloc_ranks(uint32_t nr_ranks, const char* profile, struct dpu_set_t* set);
dpu_error_t dpu_get_nr_dpus(struct dpu_set_t set, uint32_t* nr_dpus);
dpu_error_t dpu_load(struct dpu_set_t set, const char* binary_path, void* program);
dpu_error_t dpu_prepare_xfer(struct dpu_set_t dpu, void* buffer);
dpu_error_t dpu_push_xfer(struct dpu_set_t set, dpu_xfer_t xfer, const char* symbol, uint32_t offset, size_t length,
                          dpu_xfer_flags_t flags);
dpu_error_t dpu_launch(struct dpu_set_t set, dpu_launch_policy_t policy);
dpu_error_t dpu_sync(struct dpu_set_t set);
dpu_error_t dpu_free(struct dpu_set_t set);
dpu_error_t dpu_log_read(struct dpu_set_t dpu, FILE* stream);

uint32_t shim_count(struct dpu_set_t set);
struct dpu_set_t shim_nth(struct dpu_set_t set, uint32_t i);

#define DPU_FOREACH(set, dpu, idx) \
    for ((idx) = 0; (idx) < shim_count(set) && (((dpu) = shim_nth((set), (idx))), 1); ++(idx))

#define DPU_ASSERT(stmt)                                                                  \
    do {                                                                                  \
        if ((stmt) != DPU_OK) {                                                           \
            fprintf(stderr, "DPU shim call failed: %s (%s:%d)\n", #stmt, __FILE__, __LINE__); \
            abort();                                                                      \
        }                                                                                 \
    } while (0)

#ifndef NR_DPUS_PER_RANK
#define NR_DPUS_PER_RANK 64
#endif

#ifdef __cplusplus
}
#endif
#endif
