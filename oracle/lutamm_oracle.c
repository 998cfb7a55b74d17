/*
 * CPU oracle for the LUT-NN AMM: see lutamm_oracle.h for scope and parity status.
 * TEST INFRASTRUCTURE ONLY - never linked into or called from the shipped library.
 *
 * Build flags matter: the reference is compiled for baseline x86-64 with -O3 and
 * neither -march nor -ffast-math (inference-engine/src/host/CMakeLists.txt:1), so
 * every fp32 operation rounds separately and nothing is fused.  The Makefile
 * beside this file passes -ffp-contract=off to make that explicit.
 */
#include "lutamm_oracle.h"
#include <stdlib.h>
#include <string.h>

/* One (token, codebook) search.  index_calc_host.cpp:17-39:
 *   dist[c] = sum_d (x_d - cent[c][d])^2, accumulated in fp32 in dimension order from 0;
 *   scan c = 1..CT-1, replace the running minimum only when (min - dist[c]) > 1e-6.
 * The comparison is done in double against the double literal 1e-6, exactly as the
 * reference's C++ expression promotes it. */
static inline uint16_t search_one(const float* xs, const float* cents, uint32_t v, uint32_t CT,
                                  float* dist)
{
    for (uint32_t c = 0; c < CT; ++c) {
        float t = 0;
        for (uint32_t d = 0; d < v; ++d) {
            float e = xs[d] - cents[c * v + d];
            float sq = e * e;
            t = t + sq;
        }
        dist[c] = t;
    }
    float mn = dist[0];
    uint16_t best = 0;
    for (uint32_t c = 1; c < CT; ++c) {
        float diff = mn - dist[c];
        if ((double)diff > 1e-6) {
            mn = dist[c];
            best = (uint16_t)c;
        }
    }
    return best;
}

void oracle_index_calculation_tiled(const float* x, const float* centroid, uint16_t* idx,
                                    uint32_t M, uint32_t K, uint32_t v, uint32_t CB, uint32_t CT,
                                    uint32_t n_stile, uint32_t cb_mtile, int nthreads)
{
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static)
    for (uint32_t i = 0; i < M; ++i) {
        float* dist = (float*)malloc(sizeof(float) * CT);
        for (uint32_t cb = 0; cb < CB; ++cb) {
            uint16_t best = search_one(x + (size_t)i * K + (size_t)cb * v,
                                       centroid + (size_t)cb * CT * v, v, CT, dist);
            /* index_calc_host.cpp:41-49 */
            uint32_t n_tile = i / n_stile, n_in = i % n_stile;
            uint32_t cb_tile = cb / cb_mtile, cb_in = cb % cb_mtile;
            size_t off = (size_t)n_tile * n_stile * CB + (size_t)cb_tile * n_stile * cb_mtile
                       + (size_t)n_in * cb_mtile + cb_in;
            idx[off] = best;
        }
        free(dist);
    }
}

void oracle_index_calculation(const float* x, const float* centroid, uint16_t* idx,
                              uint32_t M, uint32_t K, uint32_t v, uint32_t CB, uint32_t CT,
                              int nthreads)
{
    /* n_stile = M and cb_mtile = CB collapse the tiled offset to i*CB + cb. */
    oracle_index_calculation_tiled(x, centroid, idx, M, K, v, CB, CT, M ? M : 1, CB ? CB : 1, nthreads);
}

void oracle_lut_gather(const uint16_t* idx, const int8_t* lut, int32_t* acc,
                       uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, int nthreads)
{
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static)
    for (uint32_t i = 0; i < M; ++i) {
        int32_t* row = acc + (size_t)i * N;
        memset(row, 0, sizeof(int32_t) * N);
        for (uint32_t cb = 0; cb < CB; ++cb) {
            const int8_t* src = lut + ((size_t)cb * CT + idx[(size_t)i * CB + cb]) * N;
            for (uint32_t j = 0; j < N; ++j) row[j] += src[j];
        }
    }
}

void oracle_dequant(const int32_t* acc, const float* bias, float* out,
                    uint32_t M, uint32_t N, uint32_t CB, float scale, float lut_bias, int nthreads)
{
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static)
    for (uint32_t i = 0; i < M; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            /* pim_lut_host.cpp:201, left to right, each operation rounded to fp32 */
            float a = (float)acc[(size_t)i * N + j] * scale;
            float b = lut_bias * (float)CB;
            float s = a + b;
            out[(size_t)i * N + j] = s + bias[j];
        }
}

void oracle_dequant_checker_variant(const int32_t* acc, const float* bias, float* out,
                                    uint32_t M, uint32_t N, float scale, float lut_bias, int nthreads)
{
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static)
    for (uint32_t i = 0; i < M; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            float a = (float)acc[(size_t)i * N + j] * scale;
            float s = a + lut_bias;
            out[(size_t)i * N + j] = s + bias[j];
        }
}

void oracle_amm(const float* x, const float* centroid, const int8_t* lut, const float* bias,
                float* out, uint16_t* idx_out, int32_t* acc_out,
                uint32_t M, uint32_t K, uint32_t v, uint32_t CB, uint32_t CT, uint32_t N,
                float scale, float lut_bias, int nthreads)
{
    uint16_t* idx = idx_out ? idx_out : (uint16_t*)malloc(sizeof(uint16_t) * (size_t)M * CB + 2);
    int32_t* acc = acc_out ? acc_out : (int32_t*)malloc(sizeof(int32_t) * (size_t)M * N + 4);
    oracle_index_calculation(x, centroid, idx, M, K, v, CB, CT, nthreads);
    oracle_lut_gather(idx, lut, acc, M, CB, CT, N, nthreads);
    oracle_dequant(acc, bias, out, M, N, CB, scale, lut_bias, nthreads);
    if (!idx_out) free(idx);
    if (!acc_out) free(acc);
}

uint64_t oracle_tiled_output_offset(uint32_t i, uint32_t j, uint32_t n_stile, uint32_t f_stile,
                                    uint32_t f_mtile, uint32_t lut_parallelism)
{
    /* test_amm.cpp:193-202 */
    uint64_t dpu = (uint64_t)(i / n_stile) * lut_parallelism + (j / f_stile);
    uint32_t row = i % n_stile;
    uint32_t dim = j % f_stile;
    uint32_t mt = dim / f_mtile, in_mt = dim % f_mtile;
    return dpu * n_stile * f_stile + (uint64_t)mt * n_stile * f_mtile + (uint64_t)row * f_mtile + in_mt;
}

void oracle_reorder_lut(const int8_t* canonical, int8_t* tiled,
                        uint32_t CB, uint32_t CT, uint32_t N, uint32_t tile)
{
    for (uint32_t cb = 0; cb < CB; ++cb)
        for (uint32_t ct = 0; ct < CT; ++ct)
            for (uint32_t f = 0; f < N; ++f) {
                uint32_t t = f / tile, in_t = f % tile;
                size_t src = ((size_t)cb * CT + ct) * N + f;
                size_t dst = (size_t)t * CB * CT * tile + ((size_t)cb * CT + ct) * tile + in_t;
                tiled[dst] = canonical[src];
            }
}
