// C-linkage door onto the reference's own CPU statement of the whole operator, amm_cpu()
// (inference-engine/test/test_amm.cpp:126-183), compiled from that file unmodified with its main()
// renamed on the command line.  TEST INFRASTRUCTURE ONLY: the checker's second opinion and the
// timed CPU baseline ("the reference's CPU AMM time", test_amm.cpp:305).
#include <string>

#include "defines.h" /* the reference's header, found through -I */

void amm_cpu(float* input_tensor, float* centroid_tensor, lut_data_type* lut_table, float* bias_tensor,
             float* output_tensor, IndexCalcParams index_params, LUTParams lut_params);

// test_amm.cpp's main() calls the YAML parser (parser.cpp needs yaml-cpp, absent); main() is never run.
void parse_amm_configs(AMMParams&, std::string) {}

extern "C" void ref_amm_cpu(float* input, float* centroid, int8_t* lut_canonical, float* bias, float* output,
                            const IndexCalcParams* ip, const LUTParams* lp) {
    amm_cpu(input, centroid, lut_canonical, bias, output, *ip, *lp);
}
