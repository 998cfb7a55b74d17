// Step 3 of the AMM, fused into the tail of both gather variants: dequantise + bias.
//
// Follows the reference's production expression (inference-engine/src/host/pim_lut_host.cpp:201)
//     out = (float)acc * scale + lut_bias * (float)CB + bias[col]
// evaluated left to right with one fp32 rounding per operation and no fused multiply-add,
// as the reference's x86-64 build does.  |acc| <= 128*CB < 2^24 for any CB the library
// accepts in practice, so the int -> float conversion is exact.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include "kernels.h"

namespace lutamm {

__device__ __forceinline__ float dequant_one(int32_t acc, float scale, float lut_bias_cb, float bias) {
    return __fadd_rn(__fadd_rn(__fmul_rn(__int2float_rn(acc), scale), lut_bias_cb), bias);
}

// lut_bias * (float)CB, one rounding (host and device agree: IEEE fp32 multiply)
__device__ __forceinline__ float lut_bias_times_cb(float lut_bias, uint32_t CB) {
    return __fmul_rn(lut_bias, __uint2float_rn(CB));
}

__device__ __forceinline__ float exp2f_approx(float a) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}
__device__ __forceinline__ float rcp_approx(float a) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}

// Optional activation on the dequantised value (the reference runs GELU as a separate pass over the
// FFN1 output, inference-engine/src/host/transformer_layer.cpp:503).  act: 0 none, 1 tanh-form GELU
// in fp32, 2 the same through fp16 in and out (the precision of a per-fp16-value table).
//
// 0.5 x (1 + tanh(u)), u = sqrt(2/pi) x (1 + 0.044715 x^2), is evaluated as x / (1 + exp(-2u)): the
// same function without the cancellation of 1 + tanh(u) for negative x, and seven instructions
// (ex2.approx and rcp.approx, 2 ulp each) instead of tanhf's forty - the epilogue warps are four per
// SM, so a long per-element chain would outlast the main loop of the next tile.  Relative error
// below 1e-6 over the fp32 range; exp overflow gives x * 0 = -0, the limit.
__device__ __forceinline__ float activate_one(float y, uint32_t act) {
    if (act == 0u) return y;
    float x = y;
    if (act == 2u) x = __half2float(__float2half_rn(y));
    // -2u * log2(e) = x * (k0 + k1 x^2)
    const float k0 = -2.0f * 0.79788456080286535588f * 1.44269504088896340736f;
    const float k1 = k0 * 0.044715f;
    const float e = exp2f_approx(x * fmaf(k1, x * x, k0));
    float g = x * rcp_approx(1.0f + e);
    if (act == 2u) g = __half2float(__float2half_rn(g));
    return g;
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
