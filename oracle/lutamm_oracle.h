/*
 * CPU oracle for the LUT-NN approximate matrix multiply (AMM).
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * algorithm; it is the checker for the CUDA path and the timed CPU baseline.
 * Nothing in the shipped library may call it.
 *
 * Parity status: the closest-centroid search is pinned bit-for-bit against the
 * reference's own, unmodified index_calc_host.cpp (built into oracle/_ref by the
 * Makefile beside this file) and against the golden vectors generated from it.
 * The gather (integer addition, order-free) and the dequantisation (restated
 * operation by operation) are pinned bit-for-bit against the reference's whole
 * operator - amm_host.cpp, pim_lut_host.cpp and the DPU kernel pim_lut_kernel.c,
 * unmodified - run on the functional UPMEM stand-in in upmem_shim/, for all six
 * loop orders and three LUT load types (tests/test_reference_operator.py).
 *
 * Reference files followed (paths inside the reference project):
 *   inference-engine/src/host/index_calc_host.cpp:8-53   closest-centroid search
 *   inference-engine/test/test_amm.cpp:126-183           canonical-layout CPU AMM
 *   inference-engine/src/host/pim_lut_host.cpp:191-203   production dequantisation
 *   inference-engine/test/test_amm.cpp:187-213           DPU-tiled output offsets
 *   inference-engine/test/test_amm.cpp:71-121            DPU LUT re-tiling
 */
#ifndef LUTAMM_ORACLE_H
#define LUTAMM_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* idx[m*CB + cb] = hysteresis argmin (index_calc_host.cpp:11-40), canonical row-major. */
void oracle_index_calculation(const float* x, const float* centroid, uint16_t* idx,
                              uint32_t M, uint32_t K, uint32_t v, uint32_t CB, uint32_t CT,
                              int nthreads);

/* Same search, output in the reference's tiled layout (index_calc_host.cpp:41-49). */
void oracle_index_calculation_tiled(const float* x, const float* centroid, uint16_t* idx,
                                    uint32_t M, uint32_t K, uint32_t v, uint32_t CB, uint32_t CT,
                                    uint32_t n_stile, uint32_t cb_mtile, int nthreads);

/* acc[m*N + n] = sum_cb lut[cb][idx[m][cb]][n]  (test_amm.cpp:164-175). */
void oracle_lut_gather(const uint16_t* idx, const int8_t* lut, int32_t* acc,
                       uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, int nthreads);

/* out = (float)acc*scale + lut_bias*(float)CB + bias[n]   (pim_lut_host.cpp:201). */
void oracle_dequant(const int32_t* acc, const float* bias, float* out,
                    uint32_t M, uint32_t N, uint32_t CB, float scale, float lut_bias, int nthreads);

/* out = (float)acc*scale + lut_bias + bias[n]   (test_amm.cpp:181, the reference's
 * own checker; equals oracle_dequant whenever lut_bias == 0). */
void oracle_dequant_checker_variant(const int32_t* acc, const float* bias, float* out,
                                    uint32_t M, uint32_t N, float scale, float lut_bias, int nthreads);

/* Whole operator: search + gather + dequant.  idx_out / acc_out may be NULL. */
void oracle_amm(const float* x, const float* centroid, const int8_t* lut, const float* bias,
                float* out, uint16_t* idx_out, int32_t* acc_out,
                uint32_t M, uint32_t K, uint32_t v, uint32_t CB, uint32_t CT, uint32_t N,
                float scale, float lut_bias, int nthreads);

/* Offset of logical element (i, j) in the DPU-tiled output tensor (test_amm.cpp:193-202). */
uint64_t oracle_tiled_output_offset(uint32_t i, uint32_t j, uint32_t n_stile, uint32_t f_stile,
                                    uint32_t f_mtile, uint32_t lut_parallelism);

/* Canonical LUT[cb][ct][N] -> the per-DPU layout of reorder_pim_lut (test_amm.cpp:71-121);
 * tile = feature_stile_size for the static load type, feature_load_tile_size otherwise. */
void oracle_reorder_lut(const int8_t* canonical, int8_t* tiled,
                        uint32_t CB, uint32_t CT, uint32_t N, uint32_t tile);

#ifdef __cplusplus
}
#endif
#endif
