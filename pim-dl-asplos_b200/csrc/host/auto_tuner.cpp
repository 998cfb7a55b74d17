// GPU re-targeting of the reference's auto-tuner (inference-engine/src/tuner/auto_tuner.cpp).
//
//     tuner 0 in.yaml out.yaml      tune one AMM (amm_shape_params), like tune_single_kernel (:552)
//
// The reference enumerates DPU mappings (input x lut parallelism, micro-tile factors, load
// type, loop order) and ranks them with an analytic latency model fitted to UPMEM hardware
// (:111-346, :368-549).  None of those constants mean anything on a GPU, so the search here
// is by measurement: lutamm_tune() times the candidate kernel variants / tile shapes / splits
// with CUDA events on the device and keeps the fastest.  The output YAML keeps the input's
// sections and adds the plan as kernel_params.gpu_* keys (read back by parse_amm_configs);
// the UPMEM kernel_params keys are written as "one tile" so the file also parses with tools
// that expect them.  Mode 1 (whole model: four linears) is handled by the Python launcher
// run_layer.py --tune, which knows the transformer schema.
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "parser.h"
#include "yaml_lite.h"

int main(int argc, char** argv) {
    if (argc != 4 || std::string(argv[1]) != "0") {
        std::printf("usage: %s 0 input_yaml_path output_yaml_path\n", argv[0]);
        return 2;
    }
    const std::string in = argv[2], out = argv[3];
    AMMParams prm;
    std::string err;
    if (!parse_amm_configs(prm, in, &err, /*verbose=*/false)) {
        std::cerr << "config error: " << err << std::endl;
        return 2;
    }
    const IndexCalcParams& ip = prm.index_params;
    const LUTParams& lp = prm.lut_params;
    std::vector<float> centroid((size_t)ip.num_codebook * ip.num_centroid * ip.sub_vec_len), bias(lp.output_feature_len);
    std::vector<int8_t> lut((size_t)lp.num_codebook * lp.num_centroid * lp.output_feature_len);
    std::mt19937 g(233);
    std::uniform_real_distribution<float> d_c(-10.f, 10.f);
    std::uniform_int_distribution<int> d_l(-128, 127);
    for (auto& v : centroid) v = d_c(g);
    for (auto& v : lut) v = (int8_t)d_l(g);
    for (auto& v : bias) v = d_c(g);

    lutamm_ctx* ctx = nullptr;
    if (lutamm_create(&ctx, (int)prm.gpu_device) != LUTAMM_OK) {
        std::cerr << "cannot create a GPU context: " << lutamm_last_error(nullptr) << std::endl;
        return 1;
    }
    if (lutamm_load_weights(ctx, 0, centroid.data(), lut.data(), bias.data(),
                            reinterpret_cast<const lutamm_index_params*>(&ip),
                            reinterpret_cast<const lutamm_lut_params*>(&lp)) != LUTAMM_OK) {
        std::cerr << "load failed: " << lutamm_last_error(ctx) << std::endl;
        return 1;
    }
    GpuPlan best{};
    if (lutamm_tune(ctx, 0, ip.n, &best) != LUTAMM_OK) {
        std::cerr << "tuning failed: " << lutamm_last_error(ctx) << std::endl;
        return 1;
    }
    std::cout << "best plan: variant " << best.variant << " (1 gather, 2 tcgen05), ccs tokens " << best.ccs_tokens
              << ", gather cfg " << best.gather_cfg << ", n tile " << best.umma_n_tile << ", split " << best.umma_split
              << ", operand " << best.umma_operand << std::endl;

    yaml_lite::Doc doc;
    if (!yaml_lite::load(in, &doc, &err)) { std::cerr << err << std::endl; return 2; }
    const char* K = "kernel_params";
    auto put = [&](const char* key, uint32_t v) { doc.set(K, key, std::to_string(v)); };
    if (!doc.find(K, "n_stile_size")) {  // UPMEM keys: one tile
        put("loop_order", 0); put("lut_load_type", 0);
        put("n_stile_size", lp.n); put("feature_stile_size", lp.output_feature_len);
        put("n_mtile_size", lp.n); put("feature_mtile_size", lp.output_feature_len); put("cb_mtile_size", lp.num_codebook);
        put("feature_load_tile_size", lp.output_feature_len); put("cb_load_tile_size", lp.num_codebook);
        doc.set("system_params", "dpu_num", "1");
        doc.set("system_params", "nr_tasklets", "1");
    }
    put("gpu_variant", best.variant); put("gpu_ccs_tokens", best.ccs_tokens); put("gpu_gather_cfg", best.gather_cfg);
    put("gpu_umma_n_tile", best.umma_n_tile); put("gpu_umma_split", best.umma_split); put("gpu_umma_stages", best.umma_stages);
    put("gpu_umma_groups", best.umma_groups); put("gpu_umma_operand", best.umma_operand); put("gpu_umma_sps", best.umma_sps);
    if (!yaml_lite::save(out, doc, &err)) { std::cerr << err << std::endl; return 1; }
    std::cout << "wrote " << out << std::endl;
    lutamm_destroy(ctx);
    return 0;
}
