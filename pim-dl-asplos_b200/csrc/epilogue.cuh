// Step 3 of the AMM, fused into the tail of both gather variants: dequantise + bias.
//
// Follows the reference's production expression (inference-engine/src/host/pim_lut_host.cpp:201)
//     out = (float)acc * scale + lut_bias * (float)CB + bias[col]
// evaluated left to right with one fp32 rounding per operation and no fused multiply-add,
// as the reference's x86-64 build does.  |acc| <= 128*CB < 2^24 for any CB the library
// accepts in practice, so the int -> float conversion is exact.
#pragma once
#include <cstdint>
#include "kernels.h"

namespace lutamm {

__device__ __forceinline__ float dequant_one(int32_t acc, float scale, float lut_bias_cb, float bias) {
    return __fadd_rn(__fadd_rn(__fmul_rn(__int2float_rn(acc), scale), lut_bias_cb), bias);
}

// lut_bias * (float)CB, one rounding (host and device agree: IEEE fp32 multiply)
__device__ __forceinline__ float lut_bias_times_cb(float lut_bias, uint32_t CB) {
    return __fmul_rn(lut_bias, __uint2float_rn(CB));
}

// Offset of logical element (i, j) in the reference's DPU-tiled output tensor
// [dpu][f_mtile][n_in_stile][f_in_mtile] (inference-engine/test/test_amm.cpp:193-202,
// inference-engine/src/dpu/pim_lut_kernel.c:183).
__device__ __forceinline__ size_t tiled_out_offset(uint32_t i, uint32_t j, const OutLayout& L) {
    size_t dpu = (size_t)(i / L.n_stile) * L.lut_par + (j / L.f_stile);
    uint32_t row = i % L.n_stile;
    uint32_t dim = j % L.f_stile;
    uint32_t mt = dim / L.f_mtile, in_mt = dim % L.f_mtile;
    return dpu * L.n_stile * L.f_stile + (size_t)mt * L.n_stile * L.f_mtile + (size_t)row * L.f_mtile + in_mt;
}

}  // namespace lutamm
