/*
 * lutamm.h - C ABI of the B200-native LUT-NN approximate matrix multiply (AMM).
 *
 * One AMM replaces one linear layer  out[M][N] = f(x[M][K]):
 *   1. closest-centroid search: for every token m and codebook cb, the index of the
 *      centroid nearest (squared L2, fp32, hysteresis scan) to the length-v slice
 *      x[m][cb*v : cb*v+v];
 *   2. gather-accumulate: acc[m][n] = sum_cb LUT[cb][idx[m][cb]][n]  (int8 -> int32);
 *   3. dequantise: out = (float)acc*scale + lut_bias*(float)CB + bias[n].
 *
 * Every entry point below names the piece of the reference inference engine it stands
 * in for (paths inside the reference project).  All calls return 0 on success or a
 * negative LUTAMM_E* code; lutamm_last_error() gives the text.  Nothing here aborts
 * the process.  Data pointers may be host or device addresses unless stated.  Host
 * buffers are copied by cudaMemcpyAsync straight between the caller's memory and device
 * staging owned by the context: with pinned (page-locked) caller memory the copies overlap
 * the kernels and each other; pageable memory works but the CUDA runtime serialises such
 * copies, so the overlap is lost.
 *
 * Layouts (all dense, row-major, the "canonical" forms the reference's weight
 * converter writes): input [M][K] fp32, centroid [CB][CT][v] fp32, LUT [CB][CT][N]
 * int8, bias [N] fp32, output [M][N] fp32, indices [M][CB] uint8.
 */
#ifndef LUTAMM_H
#define LUTAMM_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LUTAMM_OK            0
#define LUTAMM_EINVAL       -1   /* bad argument, shape or alignment                       */
#define LUTAMM_ECUDA        -2   /* a CUDA runtime / driver call failed                    */
#define LUTAMM_ENOLAYER     -3   /* layer_id has no weights loaded                         */
#define LUTAMM_EUNSUPPORTED -4   /* shape outside what the requested kernel variant covers */
#define LUTAMM_EDEVICE      -5   /* a kernel reported a bounded wait that ran out          */
#define LUTAMM_ENOMEM       -6

/* flags for lutamm_amm / lutamm_pim_lut */
#define LUTAMM_FLAG_ASYNC         1u  /* return without waiting; input and output both device memory, or both
                                         host memory (pinned, for real overlap) that stays valid and untouched
                                         until lutamm_sync() */
#define LUTAMM_FLAG_PEER_STORE    4u  /* lutamm_amm_column_sharded only: the kernel stores this rank's slab into
                                         every rank's gathered buffer itself (see below) instead of an all-gather */
#define LUTAMM_FLAG_OUTPUT_TILED  2u  /* write the output in the reference's DPU-tiled layout
                                         [dpu][f_mtile][n_in_stile][f_in_mtile] (pim_lut_kernel.c:183,
                                         test_amm.cpp:193-202) instead of row-major [M][N]          */

/* kernel variants for step 2 */
#define LUTAMM_VARIANT_AUTO    0
#define LUTAMM_VARIANT_GATHER  1   /* TMA-staged shared-memory gather, CUDA cores          */
#define LUTAMM_VARIANT_UMMA    2   /* one-hot x LUT int8 contraction on tcgen05 / TMEM     */

/* index formats for lutamm_index_calculation */
#define LUTAMM_INDEX_U8_ROWMAJOR  0  /* uint8  idx[M][CB]                                   */
#define LUTAMM_INDEX_U16_TILED    1  /* uint16, the reference's [n_tile][cb_tile][n_in][cb_in]
                                        layout (index_calc_host.cpp:41-49)                  */

typedef struct lutamm_ctx lutamm_ctx;

/* Field-for-field the reference's IndexCalcParams (src/host/defines.h:12-24). */
typedef struct lutamm_index_params {
    uint32_t n;
    uint32_t input_feature_len;
    uint32_t sub_vec_len;
    uint32_t num_codebook;
    uint32_t num_centroid;
    uint32_t num_threads;     /* host threads in the reference; ignored here            */
    uint32_t n_stile_size;    /* only used by the tiled index / output compat layouts   */
    uint32_t cb_mtile_size;
} lutamm_index_params;

/* Field-for-field the reference's LUTParams (src/host/defines.h:26-50). */
typedef struct lutamm_lut_params {
    uint32_t n;
    uint32_t output_feature_len;
    uint32_t num_codebook;
    uint32_t num_centroid;
    float    scale;
    float    bias;            /* the per-tensor LUT bias; added CB times (pim_lut_host.cpp:201) */
    uint32_t num_threads;
    uint32_t dpu_num;         /* UPMEM mapping fields: accepted, used only by the compat layouts */
    uint32_t input_parallelism;
    uint32_t lut_parallelism;
    uint32_t feature_stile_size;
    uint32_t n_stile_size;
    uint32_t n_mtile_size;
    uint32_t feature_mtile_size;
    uint32_t cb_mtile_size;
    uint32_t lut_load_type;   /* enum LUTLoadType {STATIC, FINE_GRAIN, COARSE_GRAIN} */
    uint32_t feature_load_tile_size;
    uint32_t cb_load_tile_size;
} lutamm_lut_params;

/* GPU execution plan for one layer: what the reference's auto-tuner output
 * (kernel_params in the YAML, src/tuner/auto_tuner.cpp:46-82) becomes on a GPU.
 * The tcgen05 fields are requests: the launcher rounds ring depths down to even numbers, takes the
 * largest builder-group count not above umma_groups that divides the one-hot ring evenly, and builds one
 * slab per turn where two would let ring slots change hands - every combination computes the same
 * result. */
typedef struct lutamm_plan {
    uint32_t variant;         /* LUTAMM_VARIANT_*                                         */
    uint32_t ccs_tokens;      /* tokens each search thread walks (0 = default)            */
    uint32_t gather_cfg;      /* gather kernel tile configuration id (0 = default)        */
    uint32_t umma_n_tile;     /* tcgen05 N tile: 64, 128, 160, 192 or 256 (0 = default)   */
    uint32_t umma_split;      /* tcgen05 split of the codebook axis across CTAs (0 = auto) */
    uint32_t umma_stages;     /* tcgen05: LUT slabs in flight in shared memory (0 = as many as fit) */
    uint32_t umma_groups;     /* tcgen05 one-hot builder groups of 4 warps (0 = default)  */
    uint32_t umma_operand;    /* where the one-hot operand lives: 0 = default,
                                 1 = shared memory, 2 = tensor memory (TMEM)             */
    uint32_t umma_sps;        /* tcgen05: 128-byte slabs of the codebook axis a one-hot builder
                                 group takes per turn, 1 or 2 (0 = default; 4 is read as 2)  */
    uint32_t umma_epilogue;   /* tcgen05: how a finished tile leaves the SM.  LUTAMM_EPILOGUE_TRANSPOSE: through a
                                 shared-memory transpose and row-contiguous 16-byte stores.  LUTAMM_EPILOGUE_COPY_ENGINE:
                                 dequantised in the layout tensor memory delivers, staged swizzled and written by tiled
                                 bulk stores - a third of the instructions, which a CTA with several tiles takes from the
                                 main loop it runs beside.  0 = the copy engine wherever the launch admits it: launches
                                 with split tiles, tiled output, peer stores, 64- / 160- / 256-wide tiles or the
                                 int32 copy of lutamm_amm_debug always take the transposing form.            */
} lutamm_plan;
#define LUTAMM_EPILOGUE_AUTO        0u
#define LUTAMM_EPILOGUE_TRANSPOSE   1u
#define LUTAMM_EPILOGUE_COPY_ENGINE 2u

/* Device times of the last timed call, milliseconds (CUDA events on the context's stream).
 * Mirrors the reference's amm_time accumulators (src/host/utils.h:14-20). */
typedef struct lutamm_timings {
    float index_calc_ms;      /* amm_profiles.index_calc_latency                          */
    float lut_kernel_ms;      /* amm_profiles.kernel_latency                              */
    float data_transfer_ms;   /* amm_profiles.data_transfer_latency (host<->device copies) */
    float total_ms;
} lutamm_timings;

/* ---- context --------------------------------------------------------------------- */

/* Replaces allocate_dpu()/allocate_rank() (src/host/dpu_common.h:11-33): binds a context
 * to one CUDA device and creates its stream. */
int lutamm_create(lutamm_ctx** out, int device);

/* Replaces free_dpu_set() (src/host/dpu_common.h:35-38). Frees weights and scratch. */
int lutamm_destroy(lutamm_ctx* ctx);

/* Run on a caller-owned CUDA stream (a cudaStream_t passed as void*); NULL restores the
 * context's own stream.  No counterpart in the reference (dpu_launch is synchronous,
 * pim_lut_host.cpp:163). */
int lutamm_set_stream(lutamm_ctx* ctx, void* cuda_stream);

/* Block until everything queued on the context's stream has finished
 * (dpu_sync, pim_lut_host.cpp:22,36,117,181). */
int lutamm_sync(lutamm_ctx* ctx);

const char* lutamm_last_error(const lutamm_ctx* ctx);

/* Library identification; also the symbol CPU-only tests call to prove the library loads. */
const char* lutamm_version(void);

/* ---- weights --------------------------------------------------------------------- */

/* Upload one linear layer's centroids, LUT and bias once and keep them resident.
 * Replaces load_binary() before every AMM (src/host/dpu_common.h:40-54,
 * transformer_layer.cpp:300,430,499,555) and the per-call LUT push prepare_lut_table()
 * (src/host/pim_lut_host.cpp:26-37).  Validates what parse_amm_configs() asserts
 * (src/host/parser.cpp:56-69) plus K == CB*v, CT <= 256, N % 16 == 0. */
int lutamm_load_weights(lutamm_ctx* ctx, int layer_id,
                        const float* centroid, const int8_t* lut, const float* bias,
                        const lutamm_index_params* index_params,
                        const lutamm_lut_params* lut_params);

/* The same with the LUT in a stated layout.  LUTAMM_LUT_DPU_TILED is the table exactly as the
 * reference's callers hold it after reorder_pim_lut() (inference-engine/test/test_amm.cpp:71-121;
 * the layer tests re-tile the same way): re-tiled along the output features with tile width
 * feature_stile_size (lut_load_type STATIC) or feature_load_tile_size (FINE / COARSE_GRAIN), which
 * must divide output_feature_len.  It is un-tiled on the device at load time. */
#define LUTAMM_LUT_CANONICAL 0u
#define LUTAMM_LUT_DPU_TILED 1u
int lutamm_load_weights_layout(lutamm_ctx* ctx, int layer_id,
                               const float* centroid, const int8_t* lut, const float* bias,
                               const lutamm_index_params* index_params,
                               const lutamm_lut_params* lut_params, uint32_t lut_layout);

int lutamm_unload_weights(lutamm_ctx* ctx, int layer_id);

/* Build one linear layer's int8 lookup table from its centroids and its dense weight on the GPU.
 * Replaces the table construction of the reference's weight converter
 * (model-calibration/pim_weight_converter.py:21-36 lut_quant, :83-91 bmm + view):
 *   lut_f[cb][ct][n] = sum_d centroid[cb][ct][d] * weight[cb*v + d][n]   fp32, d ascending, unfused
 *   scale = max|lut_f| / 127 (zero point 0),  lut = int8(rint(clamp(lut_f / scale, -128, 127))),
 *   lut_bias = -scale * 0.
 * centroid [CB][CT][v] fp32, weight [CB*v][N] fp32 row-major (the checkpoint's layout), lut_out
 * [CB][CT][N] int8: each may be host or device memory; scale_out and lut_bias_out are host floats.
 * N must be a multiple of 4.  Synchronous.  The reference's bmm runs in whatever order its
 * BLAS picks, so against it the table agrees to one int8 step at rounding boundaries; against the
 * stated order it is exact. */
int lutamm_build_lut(lutamm_ctx* ctx, const float* centroid, const float* weight,
                     uint32_t num_codebook, uint32_t num_centroid, uint32_t sub_vec_len,
                     uint32_t output_feature_len, int8_t* lut_out, float* scale_out, float* lut_bias_out);

/* ---- the operator ---------------------------------------------------------------- */

/* Replaces amm_host() (src/host/amm_host.cpp:10-30; declared amm_host.h:8-10):
 * search + gather + dequantise for n_tokens rows. */
int lutamm_amm(lutamm_ctx* ctx, int layer_id, const float* input, float* output,
               uint32_t n_tokens, uint32_t flags);

/* lutamm_amm plus the two intermediate results, for parity checks: idx_out uint8
 * [n_tokens][CB], acc_out int32 [n_tokens][N]; either may be NULL.  Stands in for the
 * reference's amm_cpu()/check_dpu_result() verification hook (test_amm.cpp:126-213). */
int lutamm_amm_debug(lutamm_ctx* ctx, int layer_id, const float* input, float* output,
                     uint32_t n_tokens, uint8_t* idx_out, int32_t* acc_out, uint32_t flags);

/* Replaces index_calculation() (src/host/index_calc_host.cpp:8-53). */
int lutamm_index_calculation(lutamm_ctx* ctx, int layer_id, const float* input, void* index_out,
                             uint32_t n_tokens, uint32_t index_format);

/* Replaces pim_lut() (src/host/pim_lut_host.cpp:121-222) with prepare_input_index()
 * (:40-118) folded into the kernel's address arithmetic: index is uint8 [n_tokens][CB].
 * An index >= num_centroid selects no table row: that codebook contributes 0 to every
 * accumulator of the token (both kernel variants), and nothing outside the table is read. */
int lutamm_pim_lut(lutamm_ctx* ctx, int layer_id, const uint8_t* index, float* output,
                   uint32_t n_tokens, uint32_t flags);

/* ---- one AMM across the GPUs of a box ---------------------------------------------- */

/* The reference spreads one AMM over an input_parallelism x lut_parallelism grid of DPUs
 * (src/host/parser.cpp:41-42): token slabs (index slabs, pim_lut_host.cpp:109-117) times output-column
 * slabs (LUT slabs, pim_lut_host.cpp:26-37).  Here a rank is one process with one context on one GPU;
 * the two axes are two calls.  NCCL carries the exchanges (all-gathers on the context's stream); it is
 * loaded at run time, so a machine without it gets LUTAMM_EUNSUPPORTED from these calls only.
 *
 * lutamm_shard_unique_id: rank 0 makes the 128-byte id (ncclGetUniqueId) and hands it to the other ranks
 * by whatever channel the launcher has; lutamm_shard_init joins the context to the communicator
 * (collective: every rank calls it).  Both stand where the reference's allocate_dpu()/allocate_rank()
 * sized the DPU grid (src/host/dpu_common.h:11-33). */
#define LUTAMM_SHARD_ID_BYTES 128
int lutamm_shard_unique_id(char* id /* [LUTAMM_SHARD_ID_BYTES] */);
int lutamm_shard_init(lutamm_ctx* ctx, int rank, int world, const char* id);
int lutamm_shard_finalize(lutamm_ctx* ctx);

/* Sharding by output columns (the reference's lut_parallelism axis).  The layer was loaded on this rank
 * with ITS slab of the table and the bias: columns [rank*N/G, (rank+1)*N/G), output_feature_len = N/G (a
 * multiple of 16).  `input` holds all n_tokens rows on every rank.  `gathered` is [G][n_tokens][N/G] fp32
 * on every rank: this rank's kernel writes block `rank` in place and one all-gather fills the others.
 * That buffer IS the reference's DPU-tiled output (pim_lut_kernel.c:183, test_amm.cpp:193-202) for
 * lut_parallelism = G, n_stile_size = n_tokens, feature_stile_size = feature_mtile_size = N/G, so a caller
 * that takes the reference's layout needs no re-layout pass.
 * search_mode: every rank searches all tokens, or each rank searches n_tokens/G of them and the uint8
 * indices are all-gathered (n_tokens*CB bytes on the wire instead of G-fold search work; falls back to
 * the replicated search when n_tokens % G != 0).  Device buffers only. */
#define LUTAMM_SHARD_SEARCH_REPLICATED 0u
#define LUTAMM_SHARD_SEARCH_SPLIT      1u
int lutamm_amm_column_sharded(lutamm_ctx* ctx, int layer_id, const float* input, float* gathered,
                              uint32_t n_tokens, uint32_t search_mode, uint32_t flags);

/* The same with the exchange fused into the kernel (LUTAMM_FLAG_PEER_STORE): `gathered` must come from
 * lutamm_shard_alloc_gathered, which allocates it on every rank (a collective call) and maps every rank's copy
 * into every other rank through CUDA IPC.  The tcgen05 kernel's epilogue then stores each finished tile of this
 * rank's slab into block `rank` of EVERY rank's buffer - plain stores over NVLink, no TMA, no multicast - so
 * the transfer overlaps the contraction tile by tile; two small all-gathers order the ranks around it (nobody
 * stores before everybody is done with the previous contents, nobody reads before everybody's kernel is done).
 * Plans the fused kernel is not built for (CUDA-core gather, 64- or 256-wide tiles) fall back to the kernel
 * plus all-gather.  A rank whose allocation fails still takes part in the handle exchange, so every rank
 * returns LUTAMM_ENOMEM together instead of some waiting for it.  The reference's counterpart is the per-DPU
 * read-back of output slabs into one host tensor (src/host/pim_lut_host.cpp:173-203). */
int lutamm_shard_alloc_gathered(lutamm_ctx* ctx, size_t bytes, void** device_ptr);
int lutamm_shard_free_gathered(lutamm_ctx* ctx, void* device_ptr);

/* Sharding by tokens (the reference's input_parallelism axis): weights replicated, the ranks own
 * contiguous near-equal row blocks - n/G rows each, the first n % G ranks one more (C4's 12608 tokens on any
 * G; a rank left without rows returns at once) - and nothing is exchanged.  `input_rows` holds this rank's
 * rows.  gather == 0: `output` is this rank's block.  gather != 0 (needs n_tokens_total % G == 0): `output`
 * is the full [n_tokens_total][N] on every rank, written in place by one all-gather - or, with
 * LUTAMM_FLAG_PEER_STORE and a buffer from lutamm_shard_alloc_gathered, by the kernel's own stores as above.
 * Device buffers only. */
int lutamm_amm_token_sharded(lutamm_ctx* ctx, int layer_id, const float* input_rows, float* output,
                             uint32_t n_tokens_total, uint32_t gather, uint32_t flags);

/* Which sharding of ONE operator is fastest on this group of GPUs (the reference's auto-tuner ranks
 * input_parallelism x lut_parallelism splits of an AMM by a latency model, src/tuner/auto_tuner.cpp:368-549; here
 * the candidates are timed).  A collective call: every rank passes the same n_tokens_total (a multiple of the
 * world size) and the same reps.  `layer_all_columns` holds the operator with all N output columns (token
 * sharding), `layer_my_columns` this rank's N/G columns of it (column sharding); either may be negative to
 * leave its candidates out.  The call allocates its own operands (input n_tokens_total x K, one gathered buffer of
 * n_tokens_total x N floats through lutamm_shard_alloc_gathered), times `reps` calls of each candidate with CUDA events
 * after two warm-up calls, and reports the slowest rank's time per call in ms[], -1 for a candidate that was
 * left out or that this build has no kernel for.  `best` is the fastest candidate that leaves the whole output on
 * every rank (LUTAMM_SHARDING_TOKENS_LOCAL, which gathers nothing, is reported for comparison only). */
#define LUTAMM_SHARDING_TOKENS_LOCAL     0u  /* lutamm_amm_token_sharded, gather = 0                     */
#define LUTAMM_SHARDING_TOKENS_GATHERED  1u  /* ... gather = 1: rows all-gathered                         */
#define LUTAMM_SHARDING_TOKENS_FUSED     2u  /* ... gather = 1 with LUTAMM_FLAG_PEER_STORE                 */
#define LUTAMM_SHARDING_COLUMNS          3u  /* lutamm_amm_column_sharded, LUTAMM_SHARD_SEARCH_REPLICATED  */
#define LUTAMM_SHARDING_COLUMNS_SPLIT    4u  /* ... LUTAMM_SHARD_SEARCH_SPLIT                             */
#define LUTAMM_SHARDING_COLUMNS_FUSED    5u  /* ... LUTAMM_SHARD_SEARCH_SPLIT with LUTAMM_FLAG_PEER_STORE  */
#define LUTAMM_SHARDING_MODES            6
typedef struct {
    uint32_t best;
    uint32_t world;
    float ms[LUTAMM_SHARDING_MODES];
} lutamm_sharding_report;
int lutamm_tune_sharding(lutamm_ctx* ctx, int layer_all_columns, int layer_my_columns, uint32_t n_tokens_total,
                         uint32_t reps, lutamm_sharding_report* report);

/* ---- plans, tuning, timing ------------------------------------------------------- */

int lutamm_set_plan(lutamm_ctx* ctx, int layer_id, const lutamm_plan* plan);
int lutamm_get_plan(lutamm_ctx* ctx, int layer_id, lutamm_plan* plan);

/* Activation applied to every output element after the dequantisation, inside the LUT kernel's
 * epilogue (the int32 accumulators lutamm_amm_debug returns are not affected).  In the reference the
 * FFN1 operator is followed by a separate in-place GELU pass over its output
 * (src/host/transformer_layer.cpp:503, ggml_gelu_inplace); fused here it costs no memory traffic.
 *   LUTAMM_ACT_GELU_TANH       0.5 x (1 + tanh(u)), u = sqrt(2/pi) x (1 + 0.044715 x^2), in fp32, evaluated in the
 *                              cancellation-free form x / (1 + exp(-2u)); relative error below 1e-6
 *   LUTAMM_ACT_GELU_TANH_F16   the same with x rounded to fp16 first and the result rounded to fp16, the
 *                              precision of ggml's table-driven GELU (one table entry per fp16 value)
 * The default after lutamm_load_weights is LUTAMM_ACT_NONE. */
#define LUTAMM_ACT_NONE           0u
#define LUTAMM_ACT_GELU_TANH      1u
#define LUTAMM_ACT_GELU_TANH_F16  2u
int lutamm_set_activation(lutamm_ctx* ctx, int layer_id, uint32_t activation);

/* Replaces the auto-tuner's mapping search (src/tuner/auto_tuner.cpp:368-603): times the
 * candidate kernel variants and tile configurations for n_tokens rows with CUDA events
 * and installs the fastest.  best may be NULL. */
int lutamm_tune(lutamm_ctx* ctx, int layer_id, uint32_t n_tokens, lutamm_plan* best);

/* Plans found by lutamm_tune are remembered in the context by shape - (n_tokens, K, N, CB, CT, SM count) -
 * and a later lutamm_tune for a shape it knows installs the remembered plan without measuring.  These two
 * calls keep that table in a text file beside the configuration, so that a new process does not re-tune
 * (the reference's tuner writes its result into the YAML, src/tuner/auto_tuner.cpp:552-603; so does the
 * tuner here, and this file is the shape-keyed form of the same thing). */
int lutamm_plan_cache_save(lutamm_ctx* ctx, const char* path);
int lutamm_plan_cache_load(lutamm_ctx* ctx, const char* path);

/* Turn per-stage CUDA-event timing on (non-zero) or off; the reference's AMM_BREAKDOWN
 * compile-time switch (amm_host.cpp:14-26, pim_lut_host.cpp:124-212) as a runtime flag. */
int lutamm_enable_timing(lutamm_ctx* ctx, int on);
int lutamm_get_timings(lutamm_ctx* ctx, lutamm_timings* out);

/* The int8 tensor rate of this GPU, measured: every SM issues nothing but tcgen05.mma kind::i8
 * (128 x 256 x 32 per instruction, both operands on chip) for a few milliseconds.  The denominator for
 * the tensor-side roofline of the tcgen05 LUT kernel; the reference has no counterpart (its auto-tuner
 * uses fitted DPU constants, src/tuner/auto_tuner.cpp:121-166).
 *   tops            10^12 int8 operations (2 per multiply-add) per second, by CUDA events
 *   mac_per_clk_sm  multiply-adds per SM clock per SM, by one CTA's own cycle counter
 *   sm_mhz          the SM clock those two figures imply
 * Any pointer may be NULL. */
int lutamm_measure_int8_peak(lutamm_ctx* ctx, double* tops, double* mac_per_clk_sm, double* sm_mhz);

/* Self-test of the failure path every kernel of this library shares.  A one-CTA kernel sets up tensor
 * memory and an mbarrier, then waits - with the library's bounded wait, cut to `polls` probes - for a barrier
 * that nobody arrives at; the wait gives up, the kernel reports through the context's device error word, frees
 * its tensor memory and returns.  The call therefore returns LUTAMM_EDEVICE, and the context must be fully
 * usable afterwards (error word cleared, split-tile counters re-armed).  The reference has no counterpart: a
 * DPU fault aborts its process (DPU_ASSERT, src/host/dpu_common.h:13). */
int lutamm_selftest_bounded_wait(lutamm_ctx* ctx, uint32_t polls);

/* Kernels of this library launched on this context since creation. */
uint64_t lutamm_launch_count(const lutamm_ctx* ctx);

/* ---- for callers that must not allocate -------------------------------------------- */

/* Device bytes of index scratch compiled into the library for lutamm_amm_static_scratch();
 * every GPU that loads the library holds them (plus 256) until the process exits. */
#define LUTAMM_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)

/* The whole AMM (search + gather-accumulate + dequantise, CUDA-core gather variant) without
 * any allocation: no cudaMalloc/cudaFree, no pooled allocator, no context.  It has no
 * counterpart in the reference.  It is for hosts that fix their device-memory layout at
 * start-up and forbid allocation afterwards (serving processes with pre-sized arenas,
 * latency-critical loops, plug-in hosts that pass a fixed set of buffers).
 * All five buffers are DEVICE memory of `device`, laid out as for lutamm_load_weights /
 * lutamm_amm; n_tokens = index_params->n.  The index buffer between the two kernels lives in
 * a fixed __device__ array: n * num_codebook > LUTAMM_STATIC_SCRATCH_BYTES is rejected with
 * LUTAMM_EINVAL.  The call is synchronous on `cuda_stream` (a cudaStream_t, NULL = default
 * stream).  All calls in a process share the array on a device, so calls that overlap on the
 * GPU race: serialise them.  The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress) and should therefore come before any stream capture.
 * Error text: lutamm_static_scratch_last_error() (per thread). */
int lutamm_amm_static_scratch(int device, void* cuda_stream,
                              const float* input, const float* centroid, const int8_t* lut,
                              const float* bias, float* output,
                              const lutamm_index_params* index_params,
                              const lutamm_lut_params* lut_params);
const char* lutamm_static_scratch_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* LUTAMM_H */
