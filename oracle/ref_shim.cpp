/*
 * C-linkage door onto the reference's own index_calculation().
 *
 * TEST INFRASTRUCTURE ONLY.  This file is ours; the function it forwards to is the
 * reference's inference-engine/src/host/index_calc_host.cpp, compiled unmodified from
 * where it lies (see the Makefile).  The wrapper exists so that tests can call the
 * reference through ctypes without passing a C++ struct by value.
 */
#include "index_calc_host.h"   /* the reference's header, found through -I */

extern "C" void ref_index_calculation(float* input, float* centroid, uint16_t* index_out,
                                      uint32_t n, uint32_t input_feature_len, uint32_t sub_vec_len,
                                      uint32_t num_codebook, uint32_t num_centroid,
                                      uint32_t num_threads, uint32_t n_stile_size, uint32_t cb_mtile_size)
{
    IndexCalcParams p;
    p.n = n;
    p.input_feature_len = input_feature_len;
    p.sub_vec_len = sub_vec_len;
    p.num_codebook = num_codebook;
    p.num_centroid = num_centroid;
    p.num_threads = num_threads;
    p.n_stile_size = n_stile_size;
    p.cb_mtile_size = cb_mtile_size;
    index_calculation(input, centroid, index_out, p);
}
