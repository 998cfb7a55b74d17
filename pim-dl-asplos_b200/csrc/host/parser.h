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
