/* Builds the reference's DPU kernel (inference-engine/src/dpu/pim_lut_kernel.c) UNMODIFIED
 * into a host shared object: the source is pulled in by #include from where it lies, its
 * main() is renamed on the command line (-Dmain=dpu_main), and the sizes of its MRAM
 * symbols are exported so the host shim knows how much to move.
 * TEST INFRASTRUCTURE ONLY (see dpu.h). */
#include <stddef.h>
#include <stdint.h>
__thread uint32_t shim_tasklet_id;
void shim_set_tasklet(uint32_t id) { shim_tasklet_id = id; }

#include "pim_lut_kernel.c" /* found through -I <reference>/inference-engine/src/dpu */

const size_t shim_sizeof_lut_table = sizeof(lut_table);
const size_t shim_sizeof_input_index = sizeof(input_index);
const size_t shim_sizeof_output_data = sizeof(output_data);
const size_t shim_sizeof_dpu_arguments = sizeof(dpu_arguments);
const unsigned shim_nr_tasklets = NR_TASKLETS;
