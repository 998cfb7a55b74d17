// YAML -> AMMParams, the counterpart of parse_amm_configs() in the reference
// (inference-engine/src/host/parser.cpp:8-86; schema: configs/single_kernel_output_example.yaml).
// Differences: a malformed file or a violated invariant is an error return with a message
// (the reference prints and carries on, or asserts); kernel_params is optional - without it
// the tile sizes default to one tile (canonical row-major layouts) - and may carry the GPU
// plan as gpu_* keys written by the tuner; system_params.dpu_num / nr_tasklets are accepted
// and only used for the reference's divisibility checks when kernel_params is present.
#pragma once
#include <string>

#include "defines.h"

bool parse_amm_configs(AMMParams& amm_params, const std::string& yaml_path, std::string* error, bool verbose = true);

// YAML -> TransformerParams, the counterpart of parse_transformer_configs() in the reference
// (inference-engine/src/host/parser.cpp:89-413; schema: configs/transformer_output_example.yaml).
// Per linear <p> in {qkv, o, ffn1, ffn2}: <p>_num_codebook and <p>_num_centroid are required; <p>_scale,
// <p>_bias default to 0.01 / 0; the UPMEM mapping keys (<p>_input_parallelism, <p>_lut_parallelism,
// <p>_n_mtile_size, <p>_feature_mtile_size, <p>_cb_mtile_size, <p>_lut_load_type,
// <p>_feature_load_tile_size, <p>_cb_load_tile_size) are optional as a group: absent means one tile.
// When present, the divisibility rules the reference asserts for a single AMM (parser.cpp:56-69) are
// checked per linear and reported as errors.  <p>_gpu_* keys carry the GPU plan the tuner wrote.
bool parse_transformer_configs(TransformerParams& transformer_params, const std::string& yaml_path, std::string* error,
                               bool verbose = true);
