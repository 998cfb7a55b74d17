// The AMM operator with the reference's own argument list
// (inference-engine/src/host/amm_host.h:8-10), a lutamm context standing where the
// dpu_set_t* stood, so callers written like transformer_layer.cpp keep their shape:
//
//     amm_host(ctx, input, centroid, lut, bias, output, index_params, lut_params);
//
// The reference pushes the whole LUT to the DPUs on every call (pim_lut_host.cpp:143).
// Here the weights named by (centroid, lut, bias) are uploaded the first time they are seen
// and stay resident; later calls with the same three pointers AND the same parameter blocks
// (everything but n and the host-thread counts) only run the kernels, a call with the same
// pointers but other parameters reloads.  The association is by address, not by content: a
// caller that refills the same buffers with other weights calls amm_host_forget() first.
// Pointers may be host or device addresses.  Returns 0 or a negative LUTAMM_E* code (the reference
// returns void and aborts on error).
#pragma once
#include "defines.h"

int amm_host(lutamm_ctx* ctx, float* input_tensor, float* centroid_tensor, lut_data_type* lut_table,
             float* bias_tensor, float* output_tensor, IndexCalcParams index_params, LUTParams lut_params);

// The same operator with the reference's DATA contract as well: `lut_table` is the table after
// reorder_pim_lut() (test/test_amm.cpp:71-121, re-tiled per lut_params.lut_load_type and tile sizes)
// and `output_tensor` receives the DPU-tiled layout the reference returns
// (pim_lut_host.cpp:173-203, read back through test/test_amm.cpp:193-202).  A caller written
// against the reference passes its buffers unchanged.
int amm_host_dpu_layout(lutamm_ctx* ctx, float* input_tensor, float* centroid_tensor, lut_data_type* dpu_lut_table,
                        float* bias_tensor, float* output_tensor, IndexCalcParams index_params, LUTParams lut_params);

// The two halves, as in index_calc_host.h:5 and pim_lut_host.h:14-15.  `layer_id` names
// weights loaded with lutamm_load_weights(); the index buffer is uint8 [n][num_codebook].
int index_calculation(lutamm_ctx* ctx, int layer_id, float* input_tensor, uint8_t* lut_input_index, uint32_t n);
int pim_lut(lutamm_ctx* ctx, int layer_id, uint8_t* input_index, float* output_tensor, uint32_t n);

// Forget the pointer -> layer association kept by amm_host() for this context (frees the
// device copies).  Call before the weight buffers are reused for other contents.
void amm_host_forget(lutamm_ctx* ctx);
