// Parameter blocks of the AMM operator, C++ host side.
//
// Same names, order and meaning as the reference's inference-engine/src/host/defines.h:5-56,
// so code written against that header compiles against this one.  The two blocks are
// layout-identical to lutamm_index_params / lutamm_lut_params of the C ABI (include/lutamm.h)
// and are passed across it by pointer cast.  The UPMEM mapping fields (dpu_num,
// *_parallelism, *_stile/mtile/load_tile_size, lut_load_type) are carried for the tiled
// compatibility layouts only; the GPU execution plan lives in GpuPlan.
#pragma once
#include <stdint.h>

#include <string>

#include "lutamm.h"

typedef int8_t lut_data_type;      // LUT entries
typedef uint16_t index_data_type;  // reference index type; the GPU path stores uint8
typedef int32_t output_data_type;  // accumulators

enum LUTLoadType { STATIC = 0, FINE_GRAIN = 1, COARSE_GRAIN = 2 };

struct IndexCalcParams {
    uint32_t n;                  // tokens
    uint32_t input_feature_len;  // K
    uint32_t sub_vec_len;        // v = K / num_codebook
    uint32_t num_codebook;       // CB
    uint32_t num_centroid;       // CT
    uint32_t num_threads;        // host threads of the reference; unused here
    uint32_t n_stile_size;       // tiled index layout only
    uint32_t cb_mtile_size;
};
static_assert(sizeof(IndexCalcParams) == sizeof(lutamm_index_params), "must match the C ABI block");

struct LUTParams {
    uint32_t n;
    uint32_t output_feature_len;  // N
    uint32_t num_codebook;
    uint32_t num_centroid;
    float scale;
    float bias;                   // per-tensor LUT bias, added num_codebook times
    uint32_t num_threads;
    uint32_t dpu_num;
    uint32_t input_parallelism;
    uint32_t lut_parallelism;
    uint32_t feature_stile_size;
    uint32_t n_stile_size;
    uint32_t n_mtile_size;
    uint32_t feature_mtile_size;
    uint32_t cb_mtile_size;
    LUTLoadType lut_load_type;
    uint32_t feature_load_tile_size;
    uint32_t cb_load_tile_size;
};
static_assert(sizeof(LUTParams) == sizeof(lutamm_lut_params), "must match the C ABI block");

// What the auto-tuner decides on a GPU (kernel_params.gpu_* keys of the YAML).
typedef lutamm_plan GpuPlan;

struct AMMParams {
    IndexCalcParams index_params;
    LUTParams lut_params;
    GpuPlan gpu_plan;    // all zero = library defaults
    uint32_t gpu_device; // system_params.gpu_device, default 0
};

// The encoder layer's parameter blocks, as in the reference (src/host/defines.h:58-95).
struct AttentionParams {
    uint32_t seq_len;
    uint32_t batch_size;
    uint32_t n;  // seq_len * batch_size
    uint32_t head_num;
    uint32_t head_dim;
    uint32_t token_dim;
    uint32_t dpu_num;            // UPMEM mapping of the QKV operator: carried, unused on the GPU
    uint32_t input_parallelism;
    uint32_t lut_parallelism;
    uint32_t n_tile_size;
    uint32_t token_tile_size;
    uint32_t num_threads;
};

// amm_param_list: 0 QKV (token_dim -> 3 token_dim), 1 attention output, 2 FFN1, 3 FFN2 (ffn_hidden_dim ->
// token_dim), 4-6 the separate Q / K / V operators (token_dim -> token_dim), which the reference fills from
// the attention-output keys (src/host/parser.cpp:235-322).
struct TransformerParams {
    std::string pim_binary_list[4];  // *_lut_pim_binary: DPU kernel images, kept so a file round-trips
    AMMParams amm_param_list[7];
    AttentionParams attention_params;
    uint32_t ffn_hidden_dim;
    uint32_t layer_num;
    uint32_t num_threads;
    uint32_t gpu_device;
};
