/* Stand-in for <yaml-cpp/yaml.h> (an absent submodule of the reference): the reference's
 * test/test_amm.cpp includes it through parser.h but uses nothing of it outside main().
 * TEST INFRASTRUCTURE ONLY (see ../dpu.h). */
#ifndef LUTAMM_SHIM_YAML_H
#define LUTAMM_SHIM_YAML_H
namespace YAML {}
#endif
