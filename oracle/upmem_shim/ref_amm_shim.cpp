// C-linkage door onto the reference's own amm_host() (inference-engine/src/host/amm_host.cpp)
// running on the UPMEM stand-in of dpu.h.  TEST INFRASTRUCTURE ONLY.
// The parameter blocks are the reference's structs (src/host/defines.h), passed by pointer so
// that ctypes callers need no by-value struct passing.
#include "amm_host.h"    /* the reference's header, found through -I */
#include "dpu_common.h"  /* the reference's allocate_dpu / load_binary / free_dpu_set */

struct RefAmm {
    dpu_set_t set;
};

extern "C" RefAmm* ref_amm_open(uint32_t dpu_num, const char* kernel_object) {
    RefAmm* h = new RefAmm();
    allocate_dpu(&h->set, dpu_num);
    load_binary(&h->set, kernel_object);
    return h;
}

// `lut_dpu_layout` is the LUT after reorder_pim_lut() (test/test_amm.cpp:71-121); the output
// comes back in the DPU-tiled layout the reference produces (test/test_amm.cpp:193-202).
extern "C" void ref_amm_run(RefAmm* h, float* input, float* centroid, int8_t* lut_dpu_layout, float* bias,
                            float* output_tiled, const IndexCalcParams* ip, const LUTParams* lp) {
    amm_host(&h->set, input, centroid, lut_dpu_layout, bias, output_tiled, *ip, *lp);
}

extern "C" void ref_amm_close(RefAmm* h) {
    free_dpu_set(&h->set);
    delete h;
}
