// Internal launcher interface between the C ABI (lutamm_capi.cu) and the kernels.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace lutamm {

// ---- step 1: closest-centroid search -------------------------------------------------
struct CcsArgs {
    const float* x;         // [M][K]
    const float* centroid;  // [CB][CT][v]
    void* idx_out;          // uint8 [M][CB] or uint16 tiled
    uint32_t M, K, v, CB, CT;
    uint32_t format;        // LUTAMM_INDEX_*
    uint32_t n_stile, cb_mtile;  // tiled format only
    uint32_t tokens_per_thread;  // 0 = default
};
cudaError_t launch_ccs(const CcsArgs& a, cudaStream_t s, const char** why);

// ---- step 2+3: gather-accumulate + dequantise -----------------------------------------
// Output addressing: row-major [M][N], or the reference's DPU-tiled layout.
struct OutLayout {
    uint32_t tiled;  // 0 = row-major
    uint32_t n_stile, f_stile, f_mtile, lut_par;
};

struct LutArgs {
    const uint8_t* idx;   // [M][CB]
    const float* bias;    // [N]
    float* out;           // fp32, layout per `layout`
    int32_t* acc_out;     // optional int32 [M][N] row-major (parity checks), may be null
    uint32_t M, CB, CT, N;
    float scale, lut_bias;
    OutLayout layout;
    uint32_t act;         // LUTAMM_ACT_*: applied after the dequantisation
    // Column sharding with the exchange fused into the kernel: the [M][N] block is also stored, by plain
    // st.global over NVLink, at the same offsets of n_peers - 1 other GPUs' buffers (peer_out[g] points at
    // this rank's block inside GPU g's gathered buffer; the entry for this GPU itself equals `out` and is
    // skipped).  n_peers == 0: a purely local store.  tcgen05 variant, row-major output only.
    uint32_t n_peers;
    float* peer_out[8];
};
constexpr uint32_t kMaxPeers = 8;

// Gather variant: LUT canonical [CB][CT][N] staged by 3-D TMA tiles.
struct GatherPlan {
    uint32_t cfg;  // tile configuration id
};
uint32_t gather_num_cfgs();
// Encodes the tensor map the configuration needs (box sizes depend on it).
cudaError_t gather_make_tmap(CUtensorMap* out, const int8_t* lut, uint32_t CB, uint32_t CT, uint32_t N, uint32_t cfg,
                             const char** why);
cudaError_t launch_gather(const LutArgs& a, const CUtensorMap& lut_map, uint32_t cfg, uint32_t* dev_err,
                          cudaStream_t s, const char** why);

// tcgen05 variant: LUT transposed to K-major [N][CB*CT] at load time, 2-D TMA tiles with
// 128-byte swizzle; the one-hot operand is synthesised in shared memory from the indices.
struct UmmaPlan {
    uint32_t n_tile;    // 64 / 128 / 256 (A in shared memory), 64 / 128 / 192 (A in tensor memory)
    uint32_t a_tmem;    // 1: the one-hot operand is written to tensor memory instead of shared memory
    uint32_t split;     // work items sharing one output tile along the codebook axis
    uint32_t stages;    // LUT slabs in flight in shared memory (0 = as many as fit)
    uint32_t groups;    // one-hot builder groups of four warps (0 = default)
    uint32_t sps;       // 128-byte slabs a one-hot builder group takes per turn: 1 or 2 (0 = by ring depth)
    uint32_t max_ctas;  // persistent grid size cap: the SM count
    uint32_t epilogue;  // 1 = transposing stores; 0 / 2 = tiled bulk stores where the launch admits them
};
bool umma_supported(uint32_t CB, uint32_t CT, uint32_t N);
bool umma_tile_ok(uint32_t n_tile, bool a_tmem);
cudaError_t umma_make_tmap(CUtensorMap* out, const int8_t* lut_t, uint32_t CB, uint32_t CT, uint32_t N,
                           uint32_t n_tile, const char** why);
// `acc_scratch` (int32 [split][M][N]) and `tile_counters` (two words per output tile, zeroed once)
// are needed when split > 1.
cudaError_t launch_umma(const LutArgs& a, const CUtensorMap& lut_t_map, const UmmaPlan& p, int32_t* acc_scratch,
                        uint32_t* tile_counters, uint32_t* dev_err, cudaStream_t s, const char** why);
void umma_default_plan(uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, int sm_count, uint32_t operand,
                       uint32_t n_tile, uint32_t sps, UmmaPlan* p);
uint32_t umma_auto_split(uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, uint32_t n_tile, int sm_count);

// LUT [CB*CT][N] -> [N][CB*CT]
cudaError_t launch_transpose_lut(const int8_t* lut, int8_t* lut_t, uint32_t rows, uint32_t cols, cudaStream_t s);

// ---- load time: int8 table from centroids x dense weight -------------------------------
struct LutBuildArgs {
    const float* centroid;  // [CB][CT][v]
    const float* weight;    // [K = CB*v][N], row-major
    int8_t* lut;            // out: [CB][CT][N]
    uint32_t* absmax_bits;  // device scratch word
    float* scale_out;       // device, one float
    float* lut_bias_out;    // device, one float
    uint32_t CB, CT, v, N;
};
// Three launches on `s`: abs-max pass, quantising pass, scalar finish.
cudaError_t launch_lut_build(const LutBuildArgs& a, cudaStream_t s, const char** why);

// LUT in the reference's DPU layout (re-tiled along the output features, tile width T) -> canonical.
cudaError_t launch_lut_untile(const int8_t* dpu, int8_t* canonical, uint32_t rows, uint32_t N, uint32_t T,
                              cudaStream_t s, const char** why);

// ---- measurement aid: the int8 tensor rate itself --------------------------------------
// `slabs` x four 128 x n_tile x 32 instructions per CTA, `grid` CTAs; the cycles CTA 0 took land in *d_cycles.
cudaError_t launch_int8_peak(uint32_t n_tile, uint32_t slabs, uint32_t grid, unsigned long long* d_cycles, uint32_t* dev_err,
                             cudaStream_t s, const char** why);

// Self-test: a bounded wait on a barrier nobody arrives at; the kernel reports through *dev_err and returns.
cudaError_t launch_stalled_wait(uint32_t polls, uint32_t* dev_err, cudaStream_t s);

// Driver entry point for tensor-map encoding, resolved through the runtime so the library
// carries no link-time dependency on the driver and loads on machines without one.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

}  // namespace lutamm
