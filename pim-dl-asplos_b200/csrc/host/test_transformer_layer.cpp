// Encoder-layer driver, C++ side: the counterpart of the reference's
// inference-engine/test/test_transformer_layer.cpp (main at :266-390), restricted to what lives below
// the C ABI - the layer's LUT-AMM operators.
//
//     test_transformer_layer config.yaml [--separate]
//
// Parses the transformer YAML (parse_transformer_configs), builds seeded random operands for the
// layer's linears - QKV, attention output, FFN1, FFN2, or with --separate the three operators Q, K, V in
// place of QKV, which is how the reference's model driver is built (run_model.py:130, -DSEPARATE=1;
// transformer_layer.cpp:333-343) - and times 5 warm-up + 10 recorded rounds (the reference's cadence,
// test_transformer_layer.cpp:35-36) of those operators on host buffers: like the reference, whose operands
// live in host memory and cross to the DPUs on every call, each round pays its host<->device copies.  The dense
// parts of the layer (attention, LayerNorm, GELU: ggml on the host in the reference) are not in this
// binary; the Python launcher run_layer.py runs the whole layer.  Log lines keep the reference's wording.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "amm_host.h"
#include "parser.h"

#define WARMUP_ROUND 5
#define RECORD_ROUND 10

static double W_time() {
    using namespace std::chrono;
    return duration<double>(steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc < 2) {
        std::printf("usage: %s config_yaml_path [--separate]\n", argv[0]);
        return 2;
    }
    bool separate = false;
    for (int i = 2; i < argc; ++i)
        if (!std::strcmp(argv[i], "--separate")) separate = true;
    double time1 = W_time();
    TransformerParams tp;
    std::string err;
    if (!parse_transformer_configs(tp, argv[1], &err)) {
        std::cerr << "config error: " << err << std::endl;
        return 2;
    }
    double time2 = W_time();
    std::printf("parameter parsing time %.6f\n", time2 - time1);

    time1 = W_time();
    lutamm_ctx* ctx = nullptr;
    if (lutamm_create(&ctx, (int)tp.gpu_device) != LUTAMM_OK) {
        std::cerr << "cannot create a GPU context: " << lutamm_last_error(nullptr) << std::endl;
        return 1;
    }
    time2 = W_time();
    std::printf("dpu allocate time %.6f\n", time2 - time1);

    // which operators the layer runs, in order
    std::vector<int> ops = separate ? std::vector<int>{4, 5, 6, 1, 2, 3} : std::vector<int>{0, 1, 2, 3};
    static const char* kName[7] = {"qkv", "o", "ffn1", "ffn2", "q", "k", "v"};
    time1 = W_time();
    std::mt19937 g(233);
    std::uniform_real_distribution<float> d_c(-10.f, 10.f), d_x(-5.f, 5.f);
    std::uniform_int_distribution<int> d_l(-128, 127);
    std::vector<std::vector<float>> h_in(7), h_out(7);
    for (int id : ops) {
        const AMMParams& a = tp.amm_param_list[id];
        const IndexCalcParams& ip = a.index_params;
        const LUTParams& lp = a.lut_params;
        std::vector<float> centroid((size_t)ip.num_codebook * ip.num_centroid * ip.sub_vec_len), bias(lp.output_feature_len);
        std::vector<int8_t> lut((size_t)lp.num_codebook * lp.num_centroid * lp.output_feature_len);
        std::vector<float>& x = h_in[id];
        x.resize((size_t)ip.n * ip.input_feature_len);
        h_out[id].resize((size_t)lp.n * lp.output_feature_len);
        for (auto& v : centroid) v = d_c(g);
        for (auto& v : lut) v = (int8_t)d_l(g);
        for (auto& v : bias) v = d_c(g);
        for (auto& v : x) v = d_x(g);
        if (lutamm_load_weights(ctx, id, centroid.data(), lut.data(), bias.data(), reinterpret_cast<const lutamm_index_params*>(&ip),
                                reinterpret_cast<const lutamm_lut_params*>(&lp)) != LUTAMM_OK ||
            lutamm_set_plan(ctx, id, &a.gpu_plan) != LUTAMM_OK) {
            std::cerr << kName[id] << ": " << lutamm_last_error(ctx) << std::endl;
            return 1;
        }
    }
    time2 = W_time();
    std::printf("weight initialization time %.6f\n", time2 - time1);

    double total_time = 0;
    for (int i = 0; i < WARMUP_ROUND + RECORD_ROUND; ++i) {
        time1 = W_time();
        for (int id : ops)
            if (lutamm_amm(ctx, id, h_in[id].data(), h_out[id].data(), tp.amm_param_list[id].index_params.n, 0) != LUTAMM_OK) {
                std::cerr << kName[id] << ": " << lutamm_last_error(ctx) << std::endl;
                return 1;
            }
        time2 = W_time();
        std::printf("iteration %d, inference time %.6f\n", i, time2 - time1);
        if (i >= WARMUP_ROUND) total_time += time2 - time1;
    }
    std::cout << "--------------------------------------------\n";
    std::printf("%d rounds' average inference time %.6f  (the layer's %zu LUT-AMM operators%s)\n", RECORD_ROUND, total_time / RECORD_ROUND,
                ops.size(), separate ? ", separate Q / K / V" : "");
    lutamm_destroy(ctx);
    return 0;
}
