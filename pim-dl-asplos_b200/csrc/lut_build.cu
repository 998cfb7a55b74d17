// Load-time construction of a layer's int8 lookup table from its centroids and its dense
// weight: what model-calibration/pim_weight_converter.py:21-36,83-91 of the reference does with
// torch.bmm + lut_quant, as two HBM-bound passes that never materialise the fp32 table.
//
//   lut_f[cb][ct][n] = sum_d centroid[cb][ct][d] * weight[cb*v + d][n]     (fp32, d ascending, unfused)
//   scale            = max|lut_f| / 127                                    (zero point 0)
//   lut[cb][ct][n]   = int8( rint( clamp( lut_f / scale, -128, 127 ) ) )   (round half to even)
//
// Pass 1 reduces max|lut_f|; pass 2 recomputes the products and writes the bytes.  Compulsory
// traffic: the weight twice (8*K*N bytes) plus the table once (CB*CT*N bytes).
#include "kernels.h"

namespace lutamm {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxV = 1024;  // run-time path; bounded by the shared-memory check below

// One block: one codebook x one chunk of kThreads*4 output columns.  A thread owns four
// adjacent columns (one 16-byte weight load per sub-vector dimension, one 4-byte table
// store per centroid, so a warp writes 128 contiguous bytes per centroid row).
// V > 0: compile-time sub-vector length, the thread's weight slice lives in registers.
// V == 0: run-time length, the slice is re-read (L1 resident) per centroid.
template <int V, bool kWrite>
__global__ void __launch_bounds__(kThreads)
lut_build_kernel(const float* __restrict__ centroid, const float* __restrict__ weight, int8_t* __restrict__ lut,
                 uint32_t* __restrict__ absmax_bits, uint32_t CT, uint32_t v_rt, uint32_t N) {
    extern __shared__ float s_cent[];  // [CT][v]
    const uint32_t v = V > 0 ? (uint32_t)V : v_rt;
    const uint32_t cb = blockIdx.y;
    for (uint32_t i = threadIdx.x; i < CT * v; i += kThreads) s_cent[i] = centroid[(size_t)cb * CT * v + i];
    __syncthreads();

    const uint32_t n0 = (blockIdx.x * kThreads + threadIdx.x) * 4;
    float amax = 0.f;
    if (n0 < N) {
        const float* wrow = weight + (size_t)cb * v * N + n0;
        float4 w[V > 0 ? V : 1];
        if (V > 0) {
#pragma unroll
            for (int d = 0; d < V; ++d) w[d] = __ldg(reinterpret_cast<const float4*>(wrow + (size_t)d * N));
        }
        float scale = 1.f, inv_scale = 1.f;
        if (kWrite) {
            scale = __fdiv_rn(__uint_as_float(*absmax_bits), 127.f);
            inv_scale = __fdiv_rn(1.f, scale);
        }
        for (uint32_t ct = 0; ct < CT; ++ct) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            auto step = [&a](float c, const float4& wd) {
                a.x = __fadd_rn(a.x, __fmul_rn(c, wd.x));
                a.y = __fadd_rn(a.y, __fmul_rn(c, wd.y));
                a.z = __fadd_rn(a.z, __fmul_rn(c, wd.z));
                a.w = __fadd_rn(a.w, __fmul_rn(c, wd.w));
            };
            if (V > 0) {
#pragma unroll
                for (int d = 0; d < V; ++d) step(s_cent[ct * V + d], w[d]);
            } else {
                for (uint32_t d = 0; d < v; ++d)
                    step(s_cent[ct * v + d], __ldg(reinterpret_cast<const float4*>(wrow + (size_t)d * N)));
            }
            if (!kWrite) {
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
            } else {
                // rint(x / scale) with the IEEE division only where it can matter: x * (1/scale) is within
                // a few ulp of the quotient (|r| <= 128, so < 1e-4 absolute), hence both round to the same
                // integer unless the product lies within 1e-3 of a half-way point.
                auto q = [scale, inv_scale](float x) -> int {
                    float r = __fmul_rn(x, inv_scale);
                    if (fabsf(fabsf(r - floorf(r)) - 0.5f) < 1e-3f) r = __fdiv_rn(x, scale);
                    return (int)rintf(fminf(fmaxf(r, -128.f), 127.f));
                };
                char4 o;
                if (scale > 0.f) {
                    o.x = (signed char)q(a.x); o.y = (signed char)q(a.y);
                    o.z = (signed char)q(a.z); o.w = (signed char)q(a.w);
                } else {
                    o = make_char4(0, 0, 0, 0);  // an all-zero table has no scale; the reference would emit NaN bytes
                }
                *reinterpret_cast<char4*>(lut + ((size_t)cb * CT + ct) * N + n0) = o;
            }
        }
    }
    if (!kWrite) {
        // non-negative floats order like their bit patterns
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        __shared__ float s_w[kThreads / 32];
        if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = amax;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = s_w[0];
            for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, s_w[i]);
            if (m == m) atomicMax(absmax_bits, __float_as_uint(m));
        }
    }
}

template <int V>
void launch_both(const LutBuildArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
    lut_build_kernel<V, false><<<grid, kThreads, smem, s>>>(a.centroid, a.weight, nullptr, a.absmax_bits, a.CT, a.v, a.N);
    lut_build_kernel<V, true><<<grid, kThreads, smem, s>>>(a.centroid, a.weight, a.lut, a.absmax_bits, a.CT, a.v, a.N);
}

__global__ void lut_build_finish_kernel(const uint32_t* absmax_bits, float* scale_out, float* lut_bias_out) {
    const float scale = __fdiv_rn(__uint_as_float(*absmax_bits), 127.f);
    *scale_out = scale;
    *lut_bias_out = -scale * 0.f;  // -scale * zero_point, zero_point = 0 (pim_weight_converter.py:35)
}

}  // namespace

// The reference keeps the LUT it sends to the DPUs re-tiled along the output features
// (reorder_pim_lut, inference-engine/test/test_amm.cpp:71-121):
//   dpu[(f / T) * rows * T + row * T + f % T] = canonical[row * N + f],   row = cb * CT + ct,
// T = feature_stile_size (STATIC load type) or feature_load_tile_size (FINE / COARSE).  This
// turns such a table back into the canonical [CB][CT][N] layout the kernels read.
namespace {
__global__ void lut_untile_kernel(const int8_t* __restrict__ dpu, int8_t* __restrict__ canonical, uint32_t rows,
                                  uint32_t N, uint32_t T) {
    const uint32_t row = blockIdx.y;
    for (uint32_t f = blockIdx.x * blockDim.x + threadIdx.x; f < N; f += gridDim.x * blockDim.x)
        canonical[(size_t)row * N + f] = dpu[(size_t)(f / T) * rows * T + (size_t)row * T + f % T];
}
}  // namespace

cudaError_t launch_lut_untile(const int8_t* dpu, int8_t* canonical, uint32_t rows, uint32_t N, uint32_t T,
                              cudaStream_t s, const char** why) {
    *why = nullptr;
    if (T == 0 || N % T != 0) { *why = "output_feature_len must be a multiple of the LUT tile width"; return cudaErrorInvalidValue; }
    if (rows == 0 || rows > 65535u * 32u) { *why = "LUT has too many rows"; return cudaErrorInvalidValue; }
    // rows can exceed the 65535 limit of grid.y: fold the excess into a loop over row blocks
    const uint32_t per = 65535u;
    for (uint32_t r0 = 0; r0 < rows; r0 += per) {
        const uint32_t nr = rows - r0 < per ? rows - r0 : per;
        const dim3 grid((N + 255) / 256 > 64 ? 64 : (N + 255) / 256, nr);
        // the tile term of the source index uses the full row count, the row term the absolute row
        lut_untile_kernel<<<grid, 256, 0, s>>>(dpu + (size_t)r0 * T, canonical + (size_t)r0 * N, rows, N, T);
    }
    return cudaGetLastError();
}

cudaError_t launch_lut_build(const LutBuildArgs& a, cudaStream_t s, const char** why) {
    *why = nullptr;
    if (a.v == 0 || a.v > kMaxV) { *why = "sub-vector length must be 1..1024"; return cudaErrorInvalidValue; }
    if (a.CB == 0 || a.CB > 65535 || a.CT == 0) { *why = "num_codebook must be 1..65535 and num_centroid non-zero"; return cudaErrorInvalidValue; }
    if (a.N % 4 != 0) { *why = "output features must be a multiple of 4"; return cudaErrorInvalidValue; }
    if ((reinterpret_cast<uintptr_t>(a.weight) & 15) || (reinterpret_cast<uintptr_t>(a.lut) & 3)) {
        *why = "weight must be 16-byte aligned, table 4-byte aligned"; return cudaErrorInvalidValue;
    }
    const size_t smem = (size_t)a.CT * a.v * sizeof(float);
    if (smem > 48 * 1024) { *why = "centroids of one codebook exceed 48 KB"; return cudaErrorInvalidValue; }
    cudaError_t e = cudaMemsetAsync(a.absmax_bits, 0, sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    const dim3 grid((a.N / 4 + kThreads - 1) / kThreads, a.CB);
    switch (a.v) {
        case 1: launch_both<1>(a, grid, smem, s); break;
        case 2: launch_both<2>(a, grid, smem, s); break;
        case 4: launch_both<4>(a, grid, smem, s); break;
        case 8: launch_both<8>(a, grid, smem, s); break;
        case 16: launch_both<16>(a, grid, smem, s); break;
        default: launch_both<0>(a, grid, smem, s); break;
    }
    lut_build_finish_kernel<<<1, 1, 0, s>>>(a.absmax_bits, a.scale_out, a.lut_bias_out);
    return cudaGetLastError();
}

}  // namespace lutamm
