// Steps 2+3 of the AMM on CUDA cores: int8 LUT gather-accumulate to int32, fused dequantise.
//
// Replaces the DPU kernel lut_kernel() (inference-engine/src/dpu/pim_lut_kernel.c:95-2294,
// all loop orders and load modes compute the same sums), the host side around it
// (inference-engine/src/host/pim_lut_host.cpp:121-222) and the index pre-scaling
// prepare_input_index() (:40-118), which becomes address arithmetic here.
//
//   acc[m][n] = sum_cb LUT[cb][idx[m][cb]][n]       int8 -> int32, exact in any order
//   out[m][n] = dequant(acc[m][n])                  see epilogue.cuh
//
// One CTA owns an (M_TILE tokens) x (N_TILE columns) output tile and walks the codebooks
// in blocks.  The LUT block [cb_blk][CT][N_TILE] is staged by one 3-D TMA tile per stage
// into a ring of shared-memory buffers (full/empty mbarriers).  A warp owns TOK tokens;
// its 32 lanes span the N_TILE columns (COLS consecutive int8 each), so one token's
// index is a warp-wide broadcast and the LUT row read is conflict-free.  Bytes are
// widened and added with dp4a against a one-hot selector, straight into int32.
//
// HBM traffic: M*CB (indices) + CB*CT*N (LUT, once if it stays in L2 across M tiles)
//              + 4*N (bias) + 4*M*N (output).
#include "kernels.h"
#include "ptx.cuh"
#include "epilogue.cuh"

namespace lutamm {

namespace {

constexpr int kStages = 3;
constexpr uint32_t kStageBudget = 32 * 1024;  // bytes of LUT per stage
constexpr uint32_t kMaxCbBlk = 16;

struct GatherCfg {
    int cols;   // int8 columns per lane: 4 or 8
    int warps;  // consumer warps per CTA
    int tok;    // tokens per warp
};
constexpr GatherCfg kCfgs[] = {
    {8, 8, 8},   // 0: 256 columns x  64 tokens
    {4, 8, 8},   // 1: 128 columns x  64 tokens
    {8, 16, 8},  // 2: 256 columns x 128 tokens
    {4, 16, 8},  // 3: 128 columns x 128 tokens
    {4, 8, 4},   // 4: 128 columns x  32 tokens
};
constexpr uint32_t kNumCfgs = sizeof(kCfgs) / sizeof(kCfgs[0]);

__host__ __device__ inline uint32_t cb_block_for(uint32_t CT, uint32_t n_tile, uint32_t CB) {
    uint32_t b = kStageBudget / (CT * n_tile);
    if (b < 1) b = 1;
    if (b > kMaxCbBlk) b = kMaxCbBlk;
    if (b > CB) b = CB;
    return b;
}

template <int COLS>
struct LutWord;
template <>
struct LutWord<4> {
    uint32_t w[1];
    __device__ __forceinline__ void load(const uint8_t* p) { w[0] = *reinterpret_cast<const uint32_t*>(p); }
};
template <>
struct LutWord<8> {
    uint32_t w[2];
    __device__ __forceinline__ void load(const uint8_t* p) {
        uint2 t = *reinterpret_cast<const uint2*>(p);
        w[0] = t.x; w[1] = t.y;
    }
};

template <int COLS, int WARPS, int TOK>
__global__ void __launch_bounds__(WARPS * 32)
lut_gather_kernel(const __grid_constant__ CUtensorMap lut_map, LutArgs a, uint32_t cb_blk, uint32_t* dev_err) {
    constexpr int N_TILE = 32 * COLS;
    constexpr int M_TILE = WARPS * TOK;
    constexpr int MAX_PRE = (TOK * kMaxCbBlk + 31) / 32;

    extern __shared__ unsigned char smem_raw[];
    // TMA destinations want 128-byte alignment; the dynamic window only promises 16.
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // layout: [kStages][stage_bytes] LUT ring | [WARPS][TOK*kMaxCbBlk] index bytes | barriers | abort word
    const uint32_t stage_bytes = cb_blk * a.CT * N_TILE;
    const uint32_t stage_pitch = (stage_bytes + 127u) & ~127u;
    unsigned char* s_lut = smem;
    uint8_t* s_idx = smem + (size_t)kStages * stage_pitch;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_idx + WARPS * TOK * kMaxCbBlk);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(s_bar + 2 * kStages);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.x * N_TILE;
    const uint32_t m0 = blockIdx.y * M_TILE + warp * TOK;
    const uint32_t n_blocks = (a.CB + cb_blk - 1) / cb_blk;

    const uint32_t full0 = smem_u32(s_bar), empty0 = smem_u32(s_bar + kStages);
    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, WARPS);
        }
        fence_barrier_init();
        tma_prefetch_desc(&lut_map);
    }
    __syncthreads();

    // The LUT does not depend on the kernel that produced the indices: start fetching it,
    // then wait for that kernel (programmatic dependent launch; a no-op otherwise).
    uint32_t issued = 0;
    if (threadIdx.x == 0) {
        for (; issued < (uint32_t)kStages && issued < n_blocks; ++issued) {
            mbar_arrive_expect_tx(full0 + 8 * issued, stage_bytes);
            tma_load_3d(smem_u32(s_lut + (size_t)issued * stage_pitch), &lut_map, full0 + 8 * issued, (int32_t)n0, 0,
                        (int32_t)(issued * cb_blk));
        }
    }
    pdl_wait_prior_grid();

    int32_t acc[TOK][COLS];
#pragma unroll
    for (int t = 0; t < TOK; ++t)
#pragma unroll
        for (int k = 0; k < COLS; ++k) acc[t][k] = 0;

    // index prefetch: entry e = t*cb_blk + c of block b, spread over the lanes
    const uint32_t entries = TOK * cb_blk;
    uint8_t pre[MAX_PRE];
    auto fetch_idx = [&](uint32_t b) {
#pragma unroll
        for (int j = 0; j < MAX_PRE; ++j) {
            uint32_t e = lane + 32 * j;
            if (e < entries) {
                uint32_t t = e / cb_blk, c = e % cb_blk;
                uint32_t m = min(m0 + t, a.M - 1), cb = min(b * cb_blk + c, a.CB - 1);
                pre[j] = __ldcg(a.idx + (size_t)m * a.CB + cb);  // L2: see the note on programmatic launch
            }
        }
    };
    uint8_t* my_idx = s_idx + warp * TOK * kMaxCbBlk;
    if (n_blocks) fetch_idx(0);

    bool ok = true;
    for (uint32_t b = 0; b < n_blocks && ok; ++b) {
        const uint32_t s = b % kStages, phase = (b / kStages) & 1;
        __syncwarp();
#pragma unroll
        for (int j = 0; j < MAX_PRE; ++j) {
            uint32_t e = lane + 32 * j;
            if (e < entries) my_idx[e] = pre[j];
        }
        __syncwarp();
        if (b + 1 < n_blocks) fetch_idx(b + 1);

        ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, phase, s_abort) ? 1 : 0) != 0;
        if (!ok) break;
        const uint32_t valid = min(cb_blk, a.CB - b * cb_blk);
        const unsigned char* base = s_lut + (size_t)s * stage_pitch + lane * COLS;
        for (uint32_t c = 0; c < valid; ++c) {
            const unsigned char* row0 = base + (size_t)c * a.CT * N_TILE;
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                // An index may come from a caller (lutamm_pim_lut): one that is out of range for the
                // codebook reads the last row, inside the stage, and contributes nothing - the same as
                // the tcgen05 kernel, whose one-hot row is all zero for such an index.
                const uint32_t i_raw = my_idx[t * cb_blk + c];
                const uint32_t i = min(i_raw, a.CT - 1u);
                const uint32_t keep = i_raw < a.CT ? 0xFFFFFFFFu : 0u;
                LutWord<COLS> w;
                w.load(row0 + i * N_TILE);
#pragma unroll
                for (int k = 0; k < COLS; ++k)
                    acc[t][k] = __dp4a((int)(w.w[k >> 2] & keep), (int)(1u << (8 * (k & 3))), acc[t][k]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);
        // producer: refill this stage with block b + kStages once every warp released it
        if (threadIdx.x == 0 && issued < n_blocks) {
            ok = mbar_wait(empty0 + 8 * s, phase, s_abort);
            if (ok) {
                mbar_arrive_expect_tx(full0 + 8 * s, stage_bytes);
                tma_load_3d(smem_u32(s_lut + (size_t)s * stage_pitch), &lut_map, full0 + 8 * s, (int32_t)n0, 0,
                            (int32_t)(issued * cb_blk));
                ++issued;
            }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }

    __syncthreads();
    if (*s_abort) {
        // A wait ran out.  Let the copies this CTA still has in flight land (bounded, so the
        // shared memory is quiet before the CTA retires), report, write nothing.
        if (threadIdx.x == 0) {
            for (uint32_t blk = (issued > (uint32_t)kStages ? issued - kStages : 0u); blk < issued; ++blk)
                for (uint32_t it = 0; it < kWaitLimit; ++it)
                    if (mbar_try_wait(full0 + 8 * (blk % kStages), (blk / kStages) & 1)) break;
            atomicExch(dev_err, 1u);
        }
        __syncthreads();
        return;
    }

    // ---- epilogue: dequantise + bias, straight from registers
    const float lbcb = lut_bias_times_cb(a.lut_bias, a.CB);
    const uint32_t n = n0 + lane * COLS;
    if (n < a.N) {
        float bias[COLS];
#pragma unroll
        for (int k = 0; k < COLS; ++k) bias[k] = __ldg(a.bias + n + k);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            const uint32_t m = m0 + t;
            if (m >= a.M) break;
            float o[COLS];
#pragma unroll
            for (int k = 0; k < COLS; ++k) o[k] = dequant_one(acc[t][k], a.scale, lbcb, bias[k]);
            if (a.act) {
#pragma unroll
                for (int k = 0; k < COLS; ++k) o[k] = activate_one(o[k], a.act);
            }
            if (a.layout.tiled) {
#pragma unroll
                for (int k = 0; k < COLS; ++k) a.out[tiled_out_offset(m, n + k, a.layout)] = o[k];
            } else {
                float4* dst = reinterpret_cast<float4*>(a.out + (size_t)m * a.N + n);
#pragma unroll
                for (int q = 0; q < COLS / 4; ++q) dst[q] = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
            }
            if (a.acc_out) {
                int4* dst = reinterpret_cast<int4*>(a.acc_out + (size_t)m * a.N + n);
#pragma unroll
                for (int q = 0; q < COLS / 4; ++q)
                    dst[q] = make_int4(acc[t][4 * q], acc[t][4 * q + 1], acc[t][4 * q + 2], acc[t][4 * q + 3]);
            }
        }
    }
}

template <int COLS, int WARPS, int TOK>
cudaError_t run(const LutArgs& a, const CUtensorMap& map, uint32_t* dev_err, cudaStream_t s) {
    constexpr int N_TILE = 32 * COLS;
    constexpr int M_TILE = WARPS * TOK;
    const uint32_t cb_blk = cb_block_for(a.CT, N_TILE, a.CB);
    const uint32_t stage_bytes = cb_blk * a.CT * N_TILE;
    const uint32_t stage_pitch = (stage_bytes + 127u) & ~127u;
    const size_t smem = (size_t)kStages * stage_pitch + WARPS * TOK * kMaxCbBlk + 2 * kStages * 8 + 16 + 1024;
    auto k = lut_gather_kernel<COLS, WARPS, TOK>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.N + N_TILE - 1) / N_TILE, (a.M + M_TILE - 1) / M_TILE);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k, map, a, cb_blk, dev_err);
}

}  // namespace

uint32_t gather_num_cfgs() { return kNumCfgs; }

cudaError_t gather_make_tmap(CUtensorMap* out, const int8_t* lut, uint32_t CB, uint32_t CT, uint32_t N, uint32_t cfg,
                             const char** why) {
    *why = nullptr;
    if (cfg >= kNumCfgs) { *why = "gather: unknown tile configuration"; return cudaErrorInvalidValue; }
    if (N % 16 != 0) { *why = "gather: output_feature_len must be a multiple of 16 (TMA row pitch)"; return cudaErrorInvalidValue; }
    if (CT > 256) { *why = "gather: num_centroid must be <= 256"; return cudaErrorInvalidValue; }
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) { *why = "cuTensorMapEncodeTiled is not available from this driver"; return cudaErrorNotSupported; }
    const uint32_t n_tile = 32u * kCfgs[cfg].cols;
    const uint32_t cb_blk = cb_block_for(CT, n_tile, CB);
    cuuint64_t dims[3] = {N, CT, CB};
    cuuint64_t strides[2] = {N, (cuuint64_t)N * CT};  // bytes, dims 1 and 2
    cuuint32_t box[3] = {n_tile, CT, cb_blk};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(lut), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the gather LUT map"; return cudaErrorInvalidValue; }
    return cudaSuccess;
}

cudaError_t launch_gather(const LutArgs& a, const CUtensorMap& lut_map, uint32_t cfg, uint32_t* dev_err,
                          cudaStream_t s, const char** why) {
    *why = nullptr;
    if (a.M == 0 || a.N == 0) return cudaSuccess;
    switch (cfg) {
        case 0: return run<8, 8, 8>(a, lut_map, dev_err, s);
        case 1: return run<4, 8, 8>(a, lut_map, dev_err, s);
        case 2: return run<8, 16, 8>(a, lut_map, dev_err, s);
        case 3: return run<4, 16, 8>(a, lut_map, dev_err, s);
        case 4: return run<4, 8, 4>(a, lut_map, dev_err, s);
        default: *why = "gather: unknown tile configuration"; return cudaErrorInvalidValue;
    }
}

}  // namespace lutamm
