// GPU re-targeting of the reference's auto-tuner (inference-engine/src/tuner/auto_tuner.cpp).
//
//     tuner 0 in.yaml out.yaml      tune one AMM (amm_shape_params), like tune_single_kernel (:552-603)
//     tuner 1 in.yaml out.yaml      tune the four linears of an encoder layer (network_params +
//                                   <p>_num_codebook / <p>_num_centroid), like tune_single_model (:745-790)
//
// The reference enumerates DPU mappings (input x lut parallelism, micro-tile factors, load
// type, loop order) and ranks them with an analytic latency model fitted to UPMEM hardware
// (:111-346, :368-549).  None of those constants mean anything on a GPU, so the search here
// is by measurement: lutamm_tune() times the candidate kernel variants / tile shapes / splits /
// ring depths with CUDA events on the device and keeps the fastest.  The output YAML keeps the
// input's sections and adds the plan as kernel_params.[<p>_]gpu_* keys (read back by the parsers);
// the UPMEM kernel_params keys are written as "one tile" where the input had none, so the file also
// parses with tools that expect them.  Plans are also kept by shape in <out.yaml>.plans (read if
// present, rewritten at the end), so a shape tuned once on this kind of GPU is not measured again.
//
// In mode 1 the reference builds its FFN2 problem as token_dim -> ffn_hidden_dim (:654-656), the
// transpose of the layer's real FFN2 (transformer_layer.cpp:555-556 runs ffn_hidden_dim -> token_dim);
// here FFN2 is tuned with its real shape.
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "parser.h"
#include "yaml_lite.h"

namespace {

int tune_one(lutamm_ctx* ctx, int layer_id, const AMMParams& prm, GpuPlan* best) {
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
    if (lutamm_load_weights(ctx, layer_id, centroid.data(), lut.data(), bias.data(), reinterpret_cast<const lutamm_index_params*>(&ip),
                            reinterpret_cast<const lutamm_lut_params*>(&lp)) != LUTAMM_OK) {
        std::cerr << "load failed: " << lutamm_last_error(ctx) << std::endl;
        return 1;
    }
    if (lutamm_tune(ctx, layer_id, ip.n, best) != LUTAMM_OK) {
        std::cerr << "tuning failed: " << lutamm_last_error(ctx) << std::endl;
        return 1;
    }
    lutamm_unload_weights(ctx, layer_id);
    return 0;
}

void put_plan(yaml_lite::Doc& doc, const std::string& pre, const GpuPlan& p) {
    auto put = [&](const char* key, uint32_t v) { doc.set("kernel_params", pre + key, std::to_string(v)); };
    put("gpu_variant", p.variant); put("gpu_ccs_tokens", p.ccs_tokens); put("gpu_gather_cfg", p.gather_cfg);
    put("gpu_umma_n_tile", p.umma_n_tile); put("gpu_umma_split", p.umma_split); put("gpu_umma_stages", p.umma_stages);
    put("gpu_umma_groups", p.umma_groups); put("gpu_umma_operand", p.umma_operand); put("gpu_umma_sps", p.umma_sps);
    put("gpu_umma_epilogue", p.umma_epilogue);
}

void print_plan(const char* what, const GpuPlan& best) {
    std::cout << what << ": variant " << best.variant << " (1 gather, 2 tcgen05), ccs tokens " << best.ccs_tokens << ", gather cfg "
              << best.gather_cfg << ", n tile " << best.umma_n_tile << ", split " << best.umma_split << ", stages " << best.umma_stages
              << ", groups " << best.umma_groups << ", operand " << best.umma_operand << std::endl;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 4 || (std::string(argv[1]) != "0" && std::string(argv[1]) != "1")) {
        std::printf("usage: %s type (0: single kernel, 1: single model) input_config_path output_config_path\n", argv[0]);
        return 2;
    }
    const bool model = std::string(argv[1]) == "1";
    const std::string in = argv[2], out = argv[3], cache = out + ".plans";
    std::string err;
    AMMParams one;
    TransformerParams tp;
    if (model ? !parse_transformer_configs(tp, in, &err, /*verbose=*/false) : !parse_amm_configs(one, in, &err, /*verbose=*/false)) {
        std::cerr << "config error: " << err << std::endl;
        return 2;
    }
    std::printf("start tuning\n");
    lutamm_ctx* ctx = nullptr;
    if (lutamm_create(&ctx, (int)(model ? tp.gpu_device : one.gpu_device)) != LUTAMM_OK) {
        std::cerr << "cannot create a GPU context: " << lutamm_last_error(nullptr) << std::endl;
        return 1;
    }
    if (FILE* f = std::fopen(cache.c_str(), "r")) {
        std::fclose(f);
        if (lutamm_plan_cache_load(ctx, cache.c_str()) != LUTAMM_OK) std::cerr << "ignoring " << cache << ": " << lutamm_last_error(ctx) << std::endl;
    }
    yaml_lite::Doc doc;
    if (!yaml_lite::load(in, &doc, &err)) { std::cerr << err << std::endl; return 2; }
    const char* K = "kernel_params";
    auto put = [&](const std::string& key, uint32_t v) { doc.set(K, key, std::to_string(v)); };
    if (!model) {
        GpuPlan best{};
        if (tune_one(ctx, 0, one, &best)) return 1;
        print_plan("best plan", best);
        const LUTParams& lp = one.lut_params;
        if (!doc.find(K, "n_stile_size")) {  // UPMEM keys: one tile
            put("loop_order", 0); put("lut_load_type", 0);
            put("n_stile_size", lp.n); put("feature_stile_size", lp.output_feature_len);
            put("n_mtile_size", lp.n); put("feature_mtile_size", lp.output_feature_len); put("cb_mtile_size", lp.num_codebook);
            put("feature_load_tile_size", lp.output_feature_len); put("cb_load_tile_size", lp.num_codebook);
            doc.set("system_params", "dpu_num", "1");
            doc.set("system_params", "nr_tasklets", "1");
        }
        put_plan(doc, "", best);
    } else {
        static const char* kPre[4] = {"qkv", "o", "ffn1", "ffn2"};
        for (int i = 0; i < 4; ++i) {
            GpuPlan best{};
            if (tune_one(ctx, i, tp.amm_param_list[i], &best)) return 1;
            print_plan(kPre[i], best);
            const std::string pre = std::string(kPre[i]) + "_";
            const LUTParams& lp = tp.amm_param_list[i].lut_params;
            if (!doc.find(K, pre + "input_parallelism")) {  // UPMEM keys: one tile
                put(pre + "input_parallelism", 1); put(pre + "lut_parallelism", 1); put(pre + "loop_order", 0); put(pre + "lut_load_type", 0);
                put(pre + "n_mtile_size", lp.n); put(pre + "feature_mtile_size", lp.output_feature_len); put(pre + "cb_mtile_size", lp.num_codebook);
                put(pre + "feature_load_tile_size", lp.output_feature_len); put(pre + "cb_load_tile_size", lp.num_codebook);
            }
            put_plan(doc, pre, best);
        }
        if (!doc.find("system_params", "dpu_num")) {
            doc.set("system_params", "dpu_num", "1");
            doc.set("system_params", "nr_tasklets", "1");
        }
    }
    if (!yaml_lite::save(out, doc, &err)) { std::cerr << err << std::endl; return 1; }
    if (lutamm_plan_cache_save(ctx, cache.c_str()) != LUTAMM_OK) std::cerr << "could not write " << cache << ": " << lutamm_last_error(ctx) << std::endl;
    std::cout << "wrote " << out << " and " << cache << std::endl;
    lutamm_destroy(ctx);
    std::printf("finish tuning\n");
    return 0;
}
