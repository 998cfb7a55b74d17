// Steps 2+3 of the AMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The gather  acc[m][n] = sum_cb LUT[cb][idx[m][cb]][n]  is the contraction
//     acc[M x N] = OneHot[M x (CB*CT)] * LUT[(CB*CT) x N]
// with OneHot[m][cb*CT + c] = (idx[m][cb] == c).  All operands are small integers and the
// accumulator is int32, so tcgen05.mma kind::i8 gives exactly the sums the reference's DPU
// kernel produces (inference-engine/src/dpu/pim_lut_kernel.c:159-175; canonical statement
// inference-engine/test/test_amm.cpp:164-175), in a different but irrelevant order.
// It does CT times more multiply-adds than the gather, on a pipe that is far more than
// CT times faster.  The dequantisation (inference-engine/src/host/pim_lut_host.cpp:201)
// is fused into the epilogue.
//
// Per CTA: one 128-token x N_TILE-column output tile, optionally only a slice of the
// contraction axis (split > 1; partial sums meet in an int32 scratch tile in L2 with
// coalesced red.add, and the CTA that arrives last dequantises and re-zeroes it).
//
//   warp 0      TMA producer: B slabs = LUT^T[n0:n0+N_TILE][k:k+128] (K-major, 128-byte
//               swizzle) from the load-time transposed copy of the LUT
//   warp 1      owns TMEM (alloc/dealloc); one lane issues tcgen05.mma, 4 per 128-byte slab
//   warps 2-5   build the one-hot A slab in shared memory straight from the uint8 indices
//               (it never exists in HBM): for CT = 16 one codebook is exactly one 16-byte
//               swizzle chunk, so a row is 8 vector stores; then run the epilogue, each
//               warp reading its own 32-lane quadrant of the accumulator
//
// HBM traffic: M*CB (indices) + CB*CT*N (LUT^T, once if L2-resident across M tiles)
//              + 4*N (bias) + 4*M*N (output).
#include "kernels.h"
#include "ptx.cuh"
#include "epilogue.cuh"

namespace lutamm {

namespace {

constexpr uint32_t kMTile = 128;
constexpr uint32_t kSlabK = 128;              // bytes of K per pipeline stage = one swizzle row
constexpr uint32_t kABytes = kMTile * kSlabK;  // 16 KiB
constexpr uint32_t kThreads = 192;
constexpr uint32_t kEpiThreads = 128;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kStagingPitch = 33;        // words; conflict-free transposes

struct UmmaParams {
    LutArgs a;
    uint32_t slabs_total;   // ceil(CB*CT / 128)
    uint32_t slabs_per_cta; // ceil(slabs_total / split)
    uint32_t split;
    uint32_t stages;
    int32_t* acc_scratch;   // [M][N] int32, all zero between launches (split > 1)
    uint32_t* tile_counters;
    uint32_t* dev_err;
};

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t n) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}

// 16 bytes with byte `i` (0..15) set to 1; i >= 16 gives zeros.
__device__ __forceinline__ uint4 onehot16(uint32_t i) {
    const uint32_t bit = 1u << ((i & 3u) * 8u);
    const uint32_t q = i >> 2;
    return make_uint4(q == 0 ? bit : 0u, q == 1 ? bit : 0u, q == 2 ? bit : 0u, q == 3 ? bit : 0u);
}

template <uint32_t N_TILE>
__global__ void __launch_bounds__(kThreads, 1)
lut_onehot_umma_kernel(const __grid_constant__ CUtensorMap lut_t_map, const UmmaParams p) {
    constexpr uint32_t kBBytes = N_TILE * kSlabK;
    constexpr uint32_t kIdesc = umma_idesc_i8(kMTile, N_TILE, /*a_signed=*/1, /*b_signed=*/1);
    constexpr uint32_t kTmemCols = N_TILE < 32 ? 32 : N_TILE;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t S = p.stages;
    unsigned char* s_a = smem;                                  // [S][16 KiB], 1024-aligned
    unsigned char* s_b = s_a + (size_t)S * kABytes;             // [S][N_TILE*128], 1024-aligned
    float* s_bias = reinterpret_cast<float*>(s_b + (size_t)S * kBBytes);              // [N_TILE]
    uint32_t* s_stage = reinterpret_cast<uint32_t*>(s_bias + N_TILE);                 // [4][32][33]
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_stage + 4 * 32 * kStagingPitch);  // 3*S + 1
    uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 3 * kMaxStages + 1);       // tmem base, abort, last
    volatile uint32_t* s_abort = s_misc + 1;

    const uint32_t full_a0 = smem_u32(s_bar), full_b0 = smem_u32(s_bar + kMaxStages),
                   empty0 = smem_u32(s_bar + 2 * kMaxStages), acc_full = smem_u32(s_bar + 3 * kMaxStages);

    const LutArgs& a = p.a;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.x * N_TILE, m0 = blockIdx.y * kMTile;
    const uint32_t slab_begin = blockIdx.z * p.slabs_per_cta;
    const uint32_t slab_end = min(p.slabs_total, slab_begin + p.slabs_per_cta);
    const uint32_t nslab = slab_end > slab_begin ? slab_end - slab_begin : 0u;
    const uint32_t Kg = a.CB * a.CT;

    if (threadIdx.x == 0) {
        s_misc[0] = 0; s_misc[1] = 0; s_misc[2] = 0;
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(full_a0 + 8 * s, kEpiThreads);
            mbar_init(full_b0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        fence_barrier_init();
        tma_prefetch_desc(&lut_t_map);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(smem_u32(s_misc), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s_misc);

    uint32_t b_issued = 0;
    if (warp == 0) {
        // ---------------- TMA producer (the LUT never depends on the preceding kernel)
        if (lane == 0) {
            for (uint32_t i = 0; i < nslab; ++i) {
                const uint32_t s = i % S, ph = (i / S) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1, s_abort)) break;
                mbar_arrive_expect_tx(full_b0 + 8 * s, kBBytes);
                tma_load_2d(smem_u32(s_b + (size_t)s * kBBytes), &lut_t_map, full_b0 + 8 * s,
                            (int32_t)((slab_begin + i) * kSlabK), (int32_t)n0);
                b_issued = i + 1;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (uint32_t i = 0; i < nslab && ok; ++i) {
                const uint32_t s = i % S, ph = (i / S) & 1;
                ok = mbar_wait(full_a0 + 8 * s, ph, s_abort) && mbar_wait(full_b0 + 8 * s, ph, s_abort);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t da = umma_desc_k_sw128(smem_u32(s_a + (size_t)s * kABytes));
                const uint64_t db = umma_desc_k_sw128(smem_u32(s_b + (size_t)s * kBBytes));
#pragma unroll
                for (uint32_t kk = 0; kk < kSlabK / 32; ++kk)  // 32 bytes of K per instruction
                    umma_i8(tmem_base, da + 2 * kk, db + 2 * kk, kIdesc, (i | kk) != 0 ? 1u : 0u);
                umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
            }
            if (ok && nslab) umma_commit(acc_full);
        }
        __syncwarp();
    } else {
        // ---------------- one-hot A builder, then epilogue (warps 2..5 -> TMEM quadrants 2,3,0,1)
        // The indices come from the kernel launched just before; they are read with ld.cg
        // (L2) because under programmatic dependent launch this CTA may have started, on an
        // SM with older lines in L1, before that kernel finished.
        pdl_wait_prior_grid();
        const uint32_t quad = warp & 3u;
        const uint32_t r = quad * 32 + lane;       // row of the tile == TMEM lane
        const uint32_t m = m0 + r;
        const bool row_ok = m < a.M;
        const uint8_t* idx_row = a.idx + (size_t)(row_ok ? m : 0) * a.CB;
        const uint32_t et = threadIdx.x - 64;      // 0..127
        for (uint32_t i = et; i < N_TILE; i += kEpiThreads) s_bias[i] = (n0 + i < a.N) ? __ldg(a.bias + n0 + i) : 0.f;

        const uint32_t sw = r & 7u;
        const bool fast16 = (a.CT == 16) && (a.CB % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.idx) & 7u) == 0);
        bool ok = true;
        for (uint32_t i = 0; i < nslab && ok; ++i) {
            const uint32_t s = i % S, ph = (i / S) & 1;
            const uint32_t kbase = (slab_begin + i) * kSlabK;
            uint4 chunk[8];
            if (fast16) {
                // one codebook == one 16-byte chunk; 8 codebooks per slab
                uint2 raw = make_uint2(0xFFFFFFFFu, 0xFFFFFFFFu);
                if (row_ok) raw = __ldcg(reinterpret_cast<const uint2*>(idx_row + (kbase >> 4)));
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t word = j < 4 ? raw.x : raw.y;
                    const uint32_t ix = (word >> (8 * (j & 3))) & 0xFFu;
                    chunk[j] = onehot16(row_ok ? ix : 16u);
                }
            } else {
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t k0 = kbase + j * 16;
                    uint4 c = make_uint4(0, 0, 0, 0);
                    if (row_ok && k0 < Kg) {
                        if (a.CT >= 16) {
                            const uint32_t cb = k0 / a.CT, sub = (k0 % a.CT) >> 4;
                            const uint32_t ix = __ldcg(idx_row + cb);
                            if ((ix >> 4) == sub) c = onehot16(ix & 15u);
                        } else {  // CT == 8: two codebooks share the chunk
                            const uint32_t cb = k0 >> 3;
                            const uint32_t i0 = __ldcg(idx_row + cb);
                            const uint32_t i1 = (cb + 1 < a.CB) ? __ldcg(idx_row + cb + 1) : 8u;
                            const uint4 lo = onehot16(i0 & 7u), hi = onehot16(i1 < 8u ? i1 + 8u : 16u);
                            c = make_uint4(lo.x | hi.x, lo.y | hi.y, lo.z | hi.z, lo.w | hi.w);
                        }
                    }
                    chunk[j] = c;
                }
            }
            ok = mbar_wait(empty0 + 8 * s, ph ^ 1, s_abort);
            if (!ok) break;
            unsigned char* row_ptr = s_a + (size_t)s * kABytes + r * kSlabK;
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j)  // 128-byte swizzle: 16-byte chunk j of row r lands at j ^ (r & 7)
                *reinterpret_cast<uint4*>(row_ptr + ((j ^ sw) << 4)) = chunk[j];
            fence_proxy_async_smem();
            mbar_arrive(full_a0 + 8 * s);
        }

        // ---------------- epilogue
        if (ok && nslab) ok = mbar_wait(acc_full, 0, s_abort);
        // Bias tile visible; every epilogue thread is past its waits, so the abort word is
        // final from here on and the branch below is uniform across the 128 threads (it
        // contains further named barriers).
        named_bar_sync(1, kEpiThreads);
        if (nslab && !*s_abort) {
            tc_fence_after_sync();
            const float lbcb = lut_bias_times_cb(a.lut_bias, a.CB);
            uint32_t* stg = s_stage + quad * 32 * kStagingPitch;
            for (uint32_t c = 0; c < N_TILE / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((quad * 32u) << 16) + c * 32u, v);
                tmem_ld_wait();
                const uint32_t nc = n0 + c * 32;
                if (p.split == 1 && !a.layout.tiled) {
                    if (row_ok && nc < a.N) {
                        // N % 16 == 0 and nc % 32 == 0: the 32 columns are in range in groups of 16
                        const uint32_t lim = min(32u, a.N - nc);
                        float4* dst = reinterpret_cast<float4*>(a.out + (size_t)m * a.N + nc);
                        int4* adst = a.acc_out ? reinterpret_cast<int4*>(a.acc_out + (size_t)m * a.N + nc) : nullptr;
#pragma unroll
                        for (uint32_t q = 0; q < 8; ++q) {
                            if (4 * q < lim) {
                                const float4 b = *reinterpret_cast<const float4*>(s_bias + c * 32 + 4 * q);
                                float4 o;
                                o.x = dequant_one((int32_t)v[4 * q + 0], a.scale, lbcb, b.x);
                                o.y = dequant_one((int32_t)v[4 * q + 1], a.scale, lbcb, b.y);
                                o.z = dequant_one((int32_t)v[4 * q + 2], a.scale, lbcb, b.z);
                                o.w = dequant_one((int32_t)v[4 * q + 3], a.scale, lbcb, b.w);
                                dst[q] = o;
                                if (adst) adst[q] = make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                            }
                        }
                    }
                } else {
                    // transpose through shared memory so that a warp touches 32 consecutive
                    // columns of one row per instruction (coalesced stores / reductions)
                    __syncwarp();
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) stg[lane * kStagingPitch + j] = v[j];
                    __syncwarp();
                    const uint32_t n = nc + lane;
                    for (uint32_t rr = 0; rr < 32; ++rr) {
                        const uint32_t mm = m0 + quad * 32 + rr;
                        if (mm >= a.M) break;
                        if (n < a.N) {
                            const int32_t val = (int32_t)stg[rr * kStagingPitch + lane];
                            if (p.split == 1) {
                                const float o = dequant_one(val, a.scale, lbcb, s_bias[c * 32 + lane]);
                                a.out[tiled_out_offset(mm, n, a.layout)] = o;
                                if (a.acc_out) a.acc_out[(size_t)mm * a.N + n] = val;
                            } else {
                                atomicAdd(p.acc_scratch + (size_t)mm * a.N + n, val);
                            }
                        }
                    }
                }
            }
            if (p.split > 1) {
                // last CTA of this output tile dequantises the summed tile and re-zeroes it
                __threadfence();
                named_bar_sync(1, kEpiThreads);
                if (et == 0) {
                    uint32_t* ctr = p.tile_counters + blockIdx.y * gridDim.x + blockIdx.x;
                    const uint32_t old = atomicAdd(ctr, 1u);
                    const uint32_t last = (old == p.split - 1) ? 1u : 0u;
                    if (last) *ctr = 0u;
                    s_misc[2] = last;
                }
                named_bar_sync(1, kEpiThreads);
                if (s_misc[2]) {
                    __threadfence();
                    for (uint32_t rr = 0; rr < 32; ++rr) {
                        const uint32_t mm = m0 + quad * 32 + rr;
                        if (mm >= a.M) break;
                        for (uint32_t c = 0; c < N_TILE / 32; ++c) {
                            const uint32_t n = n0 + c * 32 + lane;
                            if (n < a.N) {
                                int32_t* src = p.acc_scratch + (size_t)mm * a.N + n;
                                const int32_t val = __ldcg(src);
                                __stcg(src, 0);
                                const float o = dequant_one(val, a.scale, lbcb, s_bias[c * 32 + lane]);
                                if (a.layout.tiled) a.out[tiled_out_offset(mm, n, a.layout)] = o;
                                else a.out[(size_t)mm * a.N + n] = o;
                                if (a.acc_out) a.acc_out[(size_t)mm * a.N + n] = val;
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
        }
    }

    // ---------------- tear-down (also the way out after a wait that ran out)
    __syncthreads();
    if (*s_abort) {
        if (threadIdx.x == 0) {
            // let B copies still in flight land before the shared memory is given back
            const uint32_t first = b_issued > S ? b_issued - S : 0u;
            for (uint32_t i = first; i < b_issued; ++i)
                for (uint32_t it = 0; it < kWaitLimit; ++it)
                    if (mbar_try_wait(full_b0 + 8 * (i % S), (i / S) & 1)) break;
            atomicExch(p.dev_err, 2u);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

size_t umma_smem_bytes(uint32_t n_tile, uint32_t stages) {
    return (size_t)stages * (kABytes + n_tile * kSlabK) + n_tile * 4 + 4 * 32 * kStagingPitch * 4 +
           (3 * kMaxStages + 1) * 8 + 16 + 1024;
}

template <uint32_t N_TILE>
cudaError_t run(const CUtensorMap& map, const UmmaParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    auto k = lut_onehot_umma_kernel<N_TILE>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k, map, p);
}

}  // namespace

bool umma_supported(uint32_t CB, uint32_t CT, uint32_t N) {
    const bool ct_ok = CT == 8 || CT == 16 || CT == 32 || CT == 64 || CT == 128 || CT == 256;
    return ct_ok && ((uint64_t)CB * CT) % 16 == 0 && N % 16 == 0 && CB > 0 && N > 0;
}

void umma_default_plan(uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, int sm_count, UmmaPlan* p) {
    uint32_t n_tile = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    const uint32_t slabs = (uint32_t)(((uint64_t)CB * CT + kSlabK - 1) / kSlabK);
    uint32_t tiles = ((M + kMTile - 1) / kMTile) * ((N + n_tile - 1) / n_tile);
    if (n_tile == 256 && tiles < (uint32_t)sm_count / 2 && N >= 512) {
        // few tiles: narrower tiles first, then split the contraction axis
        n_tile = 128;
        tiles = ((M + kMTile - 1) / kMTile) * ((N + n_tile - 1) / n_tile);
    }
    uint32_t split = 1;
    if (tiles < (uint32_t)sm_count) {
        split = (uint32_t)sm_count / tiles;
        const uint32_t max_split = slabs / 8 ? slabs / 8 : 1;  // keep at least 8 slabs per CTA
        if (split > max_split) split = max_split;
        if (split > 16) split = 16;
        if (split < 1) split = 1;
    }
    p->n_tile = n_tile;
    p->split = split;
    p->stages = n_tile == 256 ? 4 : (n_tile == 128 ? 6 : 8);
}

cudaError_t umma_make_tmap(CUtensorMap* out, const int8_t* lut_t, uint32_t CB, uint32_t CT, uint32_t N,
                           uint32_t n_tile, const char** why) {
    *why = nullptr;
    if (!umma_supported(CB, CT, N)) { *why = "tcgen05 variant: needs num_centroid in {8,16,32,64,128,256}, CB*CT % 16 == 0, N % 16 == 0"; return cudaErrorInvalidValue; }
    if (n_tile != 64 && n_tile != 128 && n_tile != 256) { *why = "tcgen05 variant: N tile must be 64, 128 or 256"; return cudaErrorInvalidValue; }
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) { *why = "cuTensorMapEncodeTiled is not available from this driver"; return cudaErrorNotSupported; }
    const uint64_t Kg = (uint64_t)CB * CT;
    cuuint64_t dims[2] = {Kg, N};
    cuuint64_t strides[1] = {Kg};
    cuuint32_t box[2] = {kSlabK, n_tile};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(lut_t), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the transposed LUT map"; return cudaErrorInvalidValue; }
    return cudaSuccess;
}

cudaError_t launch_umma(const LutArgs& a, const CUtensorMap& lut_t_map, const UmmaPlan& plan, int32_t* acc_scratch,
                        uint32_t* tile_counters, uint32_t* dev_err, cudaStream_t s, const char** why) {
    *why = nullptr;
    if (a.M == 0 || a.N == 0) return cudaSuccess;
    UmmaParams p;
    p.a = a;
    p.slabs_total = (uint32_t)(((uint64_t)a.CB * a.CT + kSlabK - 1) / kSlabK);
    uint32_t split = plan.split ? plan.split : 1;
    if (split > p.slabs_total) split = p.slabs_total;
    p.slabs_per_cta = (p.slabs_total + split - 1) / split;
    split = (p.slabs_total + p.slabs_per_cta - 1) / p.slabs_per_cta;  // no empty slices
    p.split = split;
    p.stages = plan.stages ? plan.stages : 4;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    if (p.stages < 2) p.stages = 2;
    while (p.stages > 2 && umma_smem_bytes(plan.n_tile, p.stages) > 227 * 1024) --p.stages;
    p.acc_scratch = acc_scratch;
    p.tile_counters = tile_counters;
    p.dev_err = dev_err;
    if (split > 1 && (!acc_scratch || !tile_counters)) { *why = "tcgen05 variant: split > 1 needs scratch"; return cudaErrorInvalidValue; }
    const size_t smem = umma_smem_bytes(plan.n_tile, p.stages);
    dim3 grid((a.N + plan.n_tile - 1) / plan.n_tile, (a.M + kMTile - 1) / kMTile, split);
    switch (plan.n_tile) {
        case 64: return run<64>(lut_t_map, p, grid, smem, s);
        case 128: return run<128>(lut_t_map, p, grid, smem, s);
        case 256: return run<256>(lut_t_map, p, grid, smem, s);
        default: *why = "tcgen05 variant: N tile must be 64, 128 or 256"; return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------- LUT [rows][cols] -> [cols][rows]
namespace {
__global__ void transpose_i8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, uint32_t rows,
                                    uint32_t cols) {
    __shared__ int8_t tile[64][65];
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (uint32_t i = threadIdx.y; i < 64; i += blockDim.y) {
        const uint32_t r = r0 + i, c = c0 + threadIdx.x;
        tile[i][threadIdx.x] = (r < rows && c < cols) ? in[(size_t)r * cols + c] : (int8_t)0;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.y; i < 64; i += blockDim.y) {
        const uint32_t c = c0 + i, r = r0 + threadIdx.x;
        if (c < cols && r < rows) out[(size_t)c * rows + r] = tile[threadIdx.x][i];
    }
}
}  // namespace

cudaError_t launch_transpose_lut(const int8_t* lut, int8_t* lut_t, uint32_t rows, uint32_t cols, cudaStream_t s) {
    dim3 block(64, 8), grid((cols + 63) / 64, (rows + 63) / 64);
    transpose_i8_kernel<<<grid, block, 0, s>>>(lut, lut_t, rows, cols);
    return cudaGetLastError();
}

}  // namespace lutamm
