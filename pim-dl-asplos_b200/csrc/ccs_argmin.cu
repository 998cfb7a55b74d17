// Step 1 of the AMM: closest-centroid search (CCS).
//
// Replaces index_calculation() of the reference (inference-engine/src/host/index_calc_host.cpp:8-53).
// The result has to match that function bit for bit, which pins three things:
//   * every fp32 operation rounds on its own (the reference is built for baseline x86-64,
//     no FMA): __fsub_rn / __fmul_rn / __fadd_rn are never contracted by nvcc;
//   * the squared distance accumulates in dimension order starting from 0;
//   * the "argmin" is a sequential scan with hysteresis - centroid c replaces the running
//     minimum only if fl(min - dist[c]) > 1e-6 - so it is order dependent and each
//     (token, codebook) scan runs in one thread, centroids 0..CT-1 in order.  A tree or
//     shuffle reduction gives different indices on near-ties.
//
// Two mappings:
//   reg path    thread <-> codebook, centroids of that codebook live in registers, the
//               thread walks a run of tokens; activations load as coalesced float2/float4.
//               Used when CT*v <= 64 (all v in {2,4,8} x CT in {8,16,32} points with
//               CT*v <= 64).
//   smem path   thread <-> token, centroids of a block of codebooks sit in shared memory
//               and are read as warp-wide broadcasts; any v, any CT <= 256.
//
// HBM traffic: 4*M*K (activations) + 4*CB*CT*v (centroids) + M*CB (uint8 indices).
#include "kernels.h"
#include "../../include/lutamm.h"

namespace lutamm {

namespace {

constexpr float kEps = 1e-6f;  // (double)diff > 1e-6  <=>  diff > 1e-6f for fp32 diff

template <int V>
__device__ __forceinline__ void load_x(const float* __restrict__ p, float (&f)[V]) {
    if constexpr (V % 4 == 0) {
#pragma unroll
        for (int i = 0; i < V / 4; ++i) {
            float4 t = __ldg(reinterpret_cast<const float4*>(p) + i);
            f[4 * i + 0] = t.x; f[4 * i + 1] = t.y; f[4 * i + 2] = t.z; f[4 * i + 3] = t.w;
        }
    } else if constexpr (V % 2 == 0) {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
            float2 t = __ldg(reinterpret_cast<const float2*>(p) + i);
            f[2 * i + 0] = t.x; f[2 * i + 1] = t.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) f[i] = __ldg(p + i);
    }
}

__device__ __forceinline__ size_t tiled_index_offset(uint32_t m, uint32_t cb, uint32_t CB, uint32_t n_stile,
                                                     uint32_t cb_mtile) {
    // index_calc_host.cpp:41-49
    uint32_t n_tile = m / n_stile, n_in = m % n_stile;
    uint32_t cb_tile = cb / cb_mtile, cb_in = cb % cb_mtile;
    return (size_t)n_tile * n_stile * CB + (size_t)cb_tile * n_stile * cb_mtile + (size_t)n_in * cb_mtile + cb_in;
}

// ------------------------------------------------------------------ reg path
constexpr int kRegThreads = 128;

// kTok tokens are in flight per thread, which gives the scheduler kTok independent dependency
// chains per warp.

// Whether an instance keeps its (negated) centroids in shared memory rather than in registers: see the kernel.
__host__ __device__ constexpr bool cent_in_smem(int V, int CT) { return (V % 2 == 0) && (CT * V >= 64 || (V >= 4 && CT * V >= 32)); }

// TOKW: the CTA takes 32 codebooks and its four warps take different tokens, so that the four share one copy of the
// centroids in shared memory (8.7 KB per CTA instead of 34.8 KB: shared memory no longer limits how many CTAs an SM
// holds, and the staging reads a quarter of the bytes).  Otherwise the CTA takes 128 codebooks, one per thread.
// Measured with the centroids in shared memory: up to 8192 tokens TOKW is 3-22 % faster (BERT-large linears 29.0 ->
// 27.0 us, 78.2 -> 76.2 us; 1024 tokens 13.7 -> 10.7 us), at 65536 tokens 3-5 % slower; the launcher chooses by
// token count.
template <int V, int CT, bool TILED, int kTok, bool TOKW = false>
__global__ void __launch_bounds__(kRegThreads)
ccs_reg_kernel(const float* __restrict__ x, const float* __restrict__ cent, void* __restrict__ out, uint32_t M,
               uint32_t K, uint32_t CB, uint32_t tokens_per_cta, uint32_t n_stile, uint32_t cb_mtile) {
    // Let the kernel queued behind this one (the LUT kernel) start its prologue - barrier
    // set-up, tensor-memory allocation, the first LUT tiles - while the search runs; it
    // waits for this grid to finish before it touches the indices.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // This kernel is itself launched as a programmatic dependent of whatever precedes it in the stream, so
    // that its launch latency and the staging of its centroids - weights, which no preceding kernel writes -
    // overlap that kernel's tail.  Everything else it reads or overwrites - the activations, the index buffer
    // the previous LUT kernel may still be reading - comes after griddepcontrol.wait below, which returns
    // once the preceding grid has completed and its writes are visible.
    // tokens_per_cta is the run of ONE thread: the CTA's run, or each warp's where the warps take different tokens
    constexpr uint32_t kCbCta = TOKW ? 32u : (uint32_t)kRegThreads, kTokWarps = TOKW ? (uint32_t)kRegThreads / 32u : 1u;
    const uint32_t col = kTokWarps > 1 ? (threadIdx.x & 31u) : threadIdx.x;   // codebook of the CTA this thread works on
    const uint32_t cb = blockIdx.x * kCbCta + col;
    const uint32_t m0 = (blockIdx.y * kTokWarps + (kTokWarps > 1 ? threadIdx.x >> 5 : 0u)) * tokens_per_cta;
    const uint32_t m1 = min(M, m0 + tokens_per_cta);
    const bool active = cb < CB && m0 < M;

    float xs[kTok][V];
    const float* xp = x + (size_t)(active ? cb : 0) * V;

    // Centroids are kept negated (the sign is flipped while they are staged) so that x - c becomes x + (-c): the same IEEE result, and
    // for even V two dimensions go through one packed add.rn.f32x2 / mul.rn.f32x2 (each lane
    // of a packed operation rounds on its own, and add and mul stay separate instructions,
    // so this is still the reference's unfused arithmetic).
    // The CTA's 128 codebooks x CT x V centroid floats are contiguous in memory: fetch them
    // coalesced into shared memory (row pitch CT*V + 1 floats, so both the staging stores and the
    // per-thread reads below are bank-conflict free), instead of every lane walking its own
    // 128-byte stretch of global memory.
    constexpr int kRow = CT * V;
    // With more than 32 centroid floats per codebook the negated centroids stay in shared memory and
    // are read per centroid as 16-byte (V % 4 == 0) or 8-byte loads shared by the kTok tokens in flight:
    // held in registers they cost CT*V registers per thread (126 in all at V = 4, CT = 16: four CTAs per
    // SM, a fifth of the warps the SM can hold).  The row pitch keeps the loads aligned and conflict free
    // (kRow + 4 words for 16-byte loads: the eight threads of a quarter warp land in eight different
    // four-bank groups; kRow + 2 for 8-byte loads: the sixteen threads of a half warp in sixteen pairs).
    constexpr int kVec = (V % 4 == 0) ? 4 : 2;   // floats per shared-memory load of a centroid
    constexpr bool kCentInSmem = cent_in_smem(V, CT);
    constexpr int kPitch = kCentInSmem ? kRow + kVec : kRow + 1;
    __shared__ __align__(16) float s_cent[kCbCta * kPitch];
    {
        const uint32_t cb0 = blockIdx.x * kCbCta;
        const uint32_t n_cb = min(kCbCta, CB - cb0);
        const float* gp = cent + (size_t)cb0 * kRow;
        for (uint32_t e = threadIdx.x; e < n_cb * kRow; e += kRegThreads) {
            const uint32_t r = e / kRow, i = e % kRow;
            s_cent[r * kPitch + i] = -__ldg(gp + e);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // first batch of activations: in flight while the CTA waits at the barrier for the centroids
#pragma unroll
    for (int t = 0; t < kTok; ++t) load_x<V>(xp + (size_t)min(m0 + t, M - 1) * K, xs[t]);
    __syncthreads();
    if (!active) return;
    float nc[kCentInSmem ? 1 : CT][V];
    const float* my_cent = s_cent + col * kPitch;
    if constexpr (!kCentInSmem) {
#pragma unroll
        for (int ct = 0; ct < CT; ++ct)
#pragma unroll
            for (int d = 0; d < V; ++d) nc[ct][d] = my_cent[ct * V + d];
    }

    for (uint32_t m = m0; m < m1; m += kTok) {
        float cur[kTok][V];
#pragma unroll
        for (int t = 0; t < kTok; ++t)
#pragma unroll
            for (int d = 0; d < V; ++d) cur[t][d] = xs[t][d];
        if (m + kTok < m1) {  // next batch while this one is scanned
#pragma unroll
            for (int t = 0; t < kTok; ++t) load_x<V>(xp + (size_t)min(m + kTok + t, M - 1) * K, xs[t]);
        }
        float mn[kTok];
        uint32_t best[kTok];
#pragma unroll
        for (int ct = 0; ct < CT; ++ct) {
            float ncv[V];   // this centroid, negated
            if constexpr (kCentInSmem) {
                if constexpr (kVec == 4) {
#pragma unroll
                    for (int q = 0; q < V / 4; ++q) {
                        const float4 c4 = *reinterpret_cast<const float4*>(my_cent + ct * V + 4 * q);
                        ncv[4 * q + 0] = c4.x; ncv[4 * q + 1] = c4.y; ncv[4 * q + 2] = c4.z; ncv[4 * q + 3] = c4.w;
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < V / 2; ++q) {
                        const float2 c2 = *reinterpret_cast<const float2*>(my_cent + ct * V + 2 * q);
                        ncv[2 * q + 0] = c2.x; ncv[2 * q + 1] = c2.y;
                    }
                }
            } else {
#pragma unroll
                for (int d = 0; d < V; ++d) ncv[d] = nc[ct][d];
            }
#pragma unroll
            for (int t = 0; t < kTok; ++t) {
                float acc = 0.f;
                if constexpr (V % 2 == 0) {
#pragma unroll
                    for (int d = 0; d < V; d += 2) {
                        const float2 e = __fadd2_rn(make_float2(cur[t][d], cur[t][d + 1]), make_float2(ncv[d], ncv[d + 1]));
                        const float2 sq = __fmul2_rn(e, e);
                        acc = (d == 0) ? sq.x : __fadd_rn(acc, sq.x);  // 0 + sq.x is exact
                        acc = __fadd_rn(acc, sq.y);
                    }
                } else {
#pragma unroll
                    for (int d = 0; d < V; ++d) {
                        const float e = __fadd_rn(cur[t][d], ncv[d]);
                        acc = __fadd_rn(acc, __fmul_rn(e, e));
                    }
                }
                if (ct == 0) {
                    mn[t] = acc;
                    best[t] = 0;
                } else {
                    bool take = __fsub_rn(mn[t], acc) > kEps;  // false for NaN: keeps the earlier index
                    mn[t] = take ? acc : mn[t];
                    best[t] = take ? (uint32_t)ct : best[t];
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kTok; ++t) {
            const uint32_t mm = m + t;
            if (mm < m1) {
                if constexpr (TILED) {
                    reinterpret_cast<uint16_t*>(out)[tiled_index_offset(mm, cb, CB, n_stile, cb_mtile)] = (uint16_t)best[t];
                } else {
                    reinterpret_cast<uint8_t*>(out)[(size_t)mm * CB + cb] = (uint8_t)best[t];
                }
            }
        }
    }
}

// ------------------------------------------------------------------ smem path
constexpr int kSmemThreads = 128;  // tokens per CTA

// V > 0: compile-time sub-vector length, the token's slice sits in registers.
// V == 0: run-time length, the slice is re-read (L1 resident) per centroid.
template <int V, bool TILED>
__global__ void __launch_bounds__(kSmemThreads)
ccs_smem_kernel(const float* __restrict__ x, const float* __restrict__ cent, void* __restrict__ out, uint32_t M,
                uint32_t K, uint32_t v_rt, uint32_t CB, uint32_t CT, uint32_t cb_per_cta, uint32_t n_stile,
                uint32_t cb_mtile) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see ccs_reg_kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t v = V > 0 ? (uint32_t)V : v_rt;
    float* s_cent = reinterpret_cast<float*>(smem_raw);                   // [cbs][CT][v]
    const uint32_t cb0 = blockIdx.x * cb_per_cta;
    const uint32_t cbs = min(cb_per_cta, CB - cb0);
    uint8_t* s_idx = smem_raw + (size_t)cb_per_cta * CT * v * sizeof(float);  // [128][cb_per_cta]

    const uint32_t n_c = cbs * CT * v;
    const float* gc = cent + (size_t)cb0 * CT * v;
    for (uint32_t i = threadIdx.x; i < n_c; i += kSmemThreads) s_cent[i] = __ldg(gc + i);
    __syncthreads();

    const uint32_t m_base = blockIdx.y * kSmemThreads;
    const uint32_t m = m_base + threadIdx.x;
    if (m < M) {
        const float* xp = x + (size_t)m * K + (size_t)cb0 * v;
        for (uint32_t cl = 0; cl < cbs; ++cl, xp += v) {
            const float* cp = s_cent + (size_t)cl * CT * v;
            float mn = 0.f;
            uint32_t best = 0;
            if constexpr (V > 0) {
                float xs[V > 0 ? V : 1];
                load_x<(V > 0 ? V : 1)>(xp, xs);
                for (uint32_t ct = 0; ct < CT; ++ct) {
                    float t = 0.f;
#pragma unroll
                    for (int d = 0; d < V; ++d) {
                        float e = __fsub_rn(xs[d], cp[ct * V + d]);
                        t = __fadd_rn(t, __fmul_rn(e, e));
                    }
                    bool take = (ct > 0) && (__fsub_rn(mn, t) > kEps);
                    if (ct == 0) mn = t;
                    mn = take ? t : mn;
                    best = take ? ct : best;
                }
            } else {
                for (uint32_t ct = 0; ct < CT; ++ct) {
                    float t = 0.f;
                    for (uint32_t d = 0; d < v; ++d) {
                        float e = __fsub_rn(__ldg(xp + d), cp[ct * v + d]);
                        t = __fadd_rn(t, __fmul_rn(e, e));
                    }
                    bool take = (ct > 0) && (__fsub_rn(mn, t) > kEps);
                    if (ct == 0) mn = t;
                    mn = take ? t : mn;
                    best = take ? ct : best;
                }
            }
            s_idx[threadIdx.x * cb_per_cta + cl] = (uint8_t)best;
        }
    }
    __syncthreads();
    // write-out: consecutive threads -> consecutive codebooks of one token
    const uint32_t rows = min((uint32_t)kSmemThreads, M > m_base ? M - m_base : 0u);
    for (uint32_t i = threadIdx.x; i < rows * cbs; i += kSmemThreads) {
        uint32_t r = i / cbs, cl = i % cbs;
        uint8_t b = s_idx[r * cb_per_cta + cl];
        if constexpr (TILED) {
            reinterpret_cast<uint16_t*>(out)[tiled_index_offset(m_base + r, cb0 + cl, CB, n_stile, cb_mtile)] = b;
        } else {
            reinterpret_cast<uint8_t*>(out)[(size_t)(m_base + r) * CB + cb0 + cl] = b;
        }
    }
}

// Launch with programmatic stream serialisation allowed: the grid may be scheduled while the preceding
// kernel of the stream is still running; the kernels above wait for it (griddepcontrol.wait) before they
// touch memory, so the ordering is that of a plain launch and only the launch latency overlaps.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k, static_cast<KArgs>(args)...);
}

template <int V, int CT, int kTok, bool TOKW>
cudaError_t run_reg_tok(const CcsArgs& a, cudaStream_t s) {
    constexpr uint32_t kCbCta = TOKW ? 32u : (uint32_t)kRegThreads, kTokWarps = TOKW ? (uint32_t)kRegThreads / 32u : 1u;
    // Run length per thread.  The grid is sized in whole waves of what the GPU holds at once - SMs x CTAs
    // resident per SM for this instance (registers and shared memory decide: 6 to 8) - because a last wave
    // that is a third full costs as much as a full one: a small batch is spread over as many CTAs as it has
    // 4-token runs (one partial wave), a large one gets runs of up to 128 tokens, which also amortise the
    // centroid staging, in an integral number of nearly full waves.
    uint32_t tpt = a.tokens_per_thread;
    if (!tpt) {
        static int resident = 0, sms = 0;   // per instance; the same for every device of one kind
        if (!resident) {
            int dev = 0, r = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, ccs_reg_kernel<V, CT, false, kTok, TOKW>, kRegThreads, 0) != cudaSuccess || r < 1) r = 4;
            if (sms < 1) sms = 148;
            resident = r;
        }
        const uint64_t cb_blocks = (a.CB + kCbCta - 1) / kCbCta;
        const uint64_t wave = (uint64_t)sms * resident;
        constexpr uint64_t kCap = 128;   // longest run of one thread
        const uint64_t ctas_at_cap = cb_blocks * ((a.M + kCap * kTokWarps - 1) / (kCap * kTokWarps));
        const uint64_t waves = ctas_at_cap <= wave ? 1 : (ctas_at_cap + wave - 1) / wave;
        tpt = (uint32_t)(((uint64_t)a.M * cb_blocks + waves * wave * kTokWarps - 1) / (waves * wave * kTokWarps));
        if (tpt < (uint32_t)kTok) tpt = kTok;
        if (tpt > kCap) tpt = kCap;
    }
    tpt = (tpt + kTok - 1) / kTok * kTok;
    dim3 grid((a.CB + kCbCta - 1) / kCbCta, (a.M + tpt * kTokWarps - 1) / (tpt * kTokWarps));
    if (a.format == LUTAMM_INDEX_U16_TILED)
        return launch_dependent(ccs_reg_kernel<V, CT, true, kTok, TOKW>, grid, dim3(kRegThreads), 0, s, a.x, a.centroid, a.idx_out,
                                a.M, a.K, a.CB, tpt, a.n_stile, a.cb_mtile);
    return launch_dependent(ccs_reg_kernel<V, CT, false, kTok, TOKW>, grid, dim3(kRegThreads), 0, s, a.x, a.centroid, a.idx_out,
                            a.M, a.K, a.CB, tpt, a.n_stile, a.cb_mtile);
}

template <int V, int CT>
cudaError_t run_reg(const CcsArgs& a, cudaStream_t s) {
    // Four tokens in flight per thread: their activations are loaded together (one round trip to
    // memory instead of four) and their scans interleave.  Two or one measured no faster.
    // The instances with their centroids in registers gain from the shared copy only while the staging is a
    // large part of the kernel: 512 tokens x 768 features 10.7 -> 8.6 us, 12608 tokens 33.2 -> 35.2 us.
    if (a.M <= (cent_in_smem(V, CT) ? 16384u : 512u)) return run_reg_tok<V, CT, 4, true>(a, s);
    return run_reg_tok<V, CT, 4, false>(a, s);
}

template <int V>
cudaError_t run_smem(const CcsArgs& a, cudaStream_t s) {
    // centroid tile + index tile per CTA; keep under ~96 KB so two CTAs fit an SM
    const size_t per_cb = (size_t)a.CT * a.v * sizeof(float) + kSmemThreads;
    uint32_t cb_per_cta = (uint32_t)((96 * 1024) / per_cb);
    if (cb_per_cta == 0) cb_per_cta = 1;
    if (cb_per_cta > 64) cb_per_cta = 64;
    if (cb_per_cta > a.CB) cb_per_cta = a.CB;
    const size_t smem = per_cb * cb_per_cta;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    dim3 grid((a.CB + cb_per_cta - 1) / cb_per_cta, (a.M + kSmemThreads - 1) / kSmemThreads);
    cudaError_t e;
    if (a.format == LUTAMM_INDEX_U16_TILED) {
        auto k = ccs_smem_kernel<V, true>;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        return launch_dependent(k, grid, dim3(kSmemThreads), smem, s, a.x, a.centroid, a.idx_out, a.M, a.K, a.v, a.CB, a.CT,
                                cb_per_cta, a.n_stile, a.cb_mtile);
    } else {
        auto k = ccs_smem_kernel<V, false>;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        return launch_dependent(k, grid, dim3(kSmemThreads), smem, s, a.x, a.centroid, a.idx_out, a.M, a.K, a.v, a.CB, a.CT,
                                cb_per_cta, a.n_stile, a.cb_mtile);
    }
}

}  // namespace

cudaError_t launch_ccs(const CcsArgs& a, cudaStream_t s, const char** why) {
    *why = nullptr;
    if (a.M == 0 || a.CB == 0) return cudaSuccess;
    if (a.CT == 0 || a.CT > 256 || a.v == 0 || a.K != a.CB * a.v) {
        *why = "closest-centroid search: need 1 <= num_centroid <= 256 and input_feature_len == num_codebook*sub_vec_len";
        return cudaErrorInvalidValue;
    }
    // vector loads need the row pitch and the base address aligned to the vector width
    const uintptr_t xa = reinterpret_cast<uintptr_t>(a.x), ca = reinterpret_cast<uintptr_t>(a.centroid);
    const uint32_t vec_bytes = (a.v % 4 == 0) ? 16u : (a.v % 2 == 0) ? 8u : 4u;
    const bool aligned = (xa % vec_bytes == 0) && (ca % vec_bytes == 0);
    if (aligned) {
#define LUTAMM_CCS_REG(V_, CT_) \
    if (a.v == V_ && a.CT == CT_) return run_reg<V_, CT_>(a, s);
        LUTAMM_CCS_REG(2, 8)
        LUTAMM_CCS_REG(2, 16)
        LUTAMM_CCS_REG(2, 32)
        LUTAMM_CCS_REG(4, 8)
        LUTAMM_CCS_REG(4, 16)
        LUTAMM_CCS_REG(8, 8)
#undef LUTAMM_CCS_REG
        switch (a.v) {
            case 1: return run_smem<1>(a, s);
            case 2: return run_smem<2>(a, s);
            case 4: return run_smem<4>(a, s);
            case 8: return run_smem<8>(a, s);
            case 16: return run_smem<16>(a, s);
            case 32: return run_smem<32>(a, s);
            // hidden sizes that are not a power of two times the codebook count (2560 / 256, 5120 / 256, ...)
            case 3: return run_smem<3>(a, s);
            case 5: return run_smem<5>(a, s);
            case 6: return run_smem<6>(a, s);
            case 10: return run_smem<10>(a, s);
            case 12: return run_smem<12>(a, s);
            case 20: return run_smem<20>(a, s);
            case 24: return run_smem<24>(a, s);
            default: break;
        }
    }
    return run_smem<0>(a, s);
}

}  // namespace lutamm
