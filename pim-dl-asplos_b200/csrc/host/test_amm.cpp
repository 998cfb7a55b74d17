// Single-AMM benchmark driver: the counterpart of the reference's
// inference-engine/test/test_amm.cpp (main at :241-320).
//
//     test_amm kernel_config.yaml [ignored: the reference's DPU binary path] [--breakdown]
//
// Parses the YAML, fills the operand tensors with seeded random data in the reference's
// ranges (test_amm.cpp:30,40,50-53,63; one generator per tensor instead of one generator
// raced over by OpenMP threads), then runs 10 warm-up and 20 timed rounds of amm_host()
// (test_amm.cpp:21-22) with host buffers, i.e. every round pays its host<->device copies
// like the reference pays its host<->DPU transfers.  The lines "PIM AMM time" /
// "PIM AVG AMM time" keep the reference's wording so its log scrapers keep working.
// Values are not checked here: parity against the CPU oracle lives in the test-suite.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "amm_host.h"
#include "parser.h"

#define WARMUP_ROUND 10
#define RECORD_ROUND 20

static double W_time() {
    using namespace std::chrono;
    return duration<double>(steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc < 2) {
        std::printf("usage: %s kernel_config_yaml_path [dpu_binary_path (ignored)] [--breakdown]\n", argv[0]);
        return 2;
    }
    bool breakdown = false;
    for (int i = 2; i < argc; ++i)
        if (!std::strcmp(argv[i], "--breakdown")) breakdown = true;

    AMMParams prm;
    std::string err;
    if (!parse_amm_configs(prm, argv[1], &err)) {
        std::cerr << "config error: " << err << std::endl;
        return 2;
    }
    const IndexCalcParams& ip = prm.index_params;
    const LUTParams& lp = prm.lut_params;
    const size_t n_in = (size_t)ip.n * ip.input_feature_len;
    const size_t n_cent = (size_t)ip.num_codebook * ip.num_centroid * ip.sub_vec_len;
    const size_t n_lut = (size_t)lp.num_codebook * lp.num_centroid * lp.output_feature_len;
    const size_t n_out = (size_t)lp.n * lp.output_feature_len;

    // The device first: without one the driver stops here instead of after filling gigabytes of operands.
    double t1 = W_time();
    lutamm_ctx* ctx = nullptr;
    if (lutamm_create(&ctx, (int)prm.gpu_device) != LUTAMM_OK) {
        std::cerr << "cannot create a GPU context: " << lutamm_last_error(nullptr) << std::endl;
        return 1;
    }
    std::cout << "gpu context create time is " << W_time() - t1 << std::endl;

    std::vector<float> input(n_in), centroid(n_cent), bias(lp.output_feature_len), output(n_out);
    std::vector<lut_data_type> lut(n_lut);
    {
        std::mt19937 g_in(233), g_cent(234), g_lut(235), g_bias(236);
        std::uniform_real_distribution<float> d_in(-5.f, 5.f), d_c(-10.f, 10.f);
        std::uniform_int_distribution<int> d_l(-128, 127);
        for (auto& v : input) v = d_in(g_in);
        for (auto& v : centroid) v = d_c(g_cent);
        for (auto& v : lut) v = (lut_data_type)d_l(g_lut);
        for (auto& v : bias) v = d_c(g_bias);
    }
    std::cout << "data generation finished" << std::endl;

    // first call uploads the weights (the reference's load_binary + LUT push)
    t1 = W_time();
    int rc = amm_host(ctx, input.data(), centroid.data(), lut.data(), bias.data(), output.data(), ip, lp);
    if (rc != LUTAMM_OK) {
        std::cerr << "amm_host failed: " << lutamm_last_error(ctx) << std::endl;
        return 1;
    }
    std::cout << "weight load + first call time is " << W_time() - t1 << std::endl;
    // the plan from the YAML, if any; weights loaded by amm_host() get ids from 1 << 20 upwards
    const GpuPlan zero{};
    if (std::memcmp(&prm.gpu_plan, &zero, sizeof zero) != 0 && lutamm_set_plan(ctx, 1 << 20, &prm.gpu_plan) != LUTAMM_OK)
        std::cerr << "plan from the config not applied: " << lutamm_last_error(ctx) << std::endl;
    if (breakdown) lutamm_enable_timing(ctx, 1);

    double total = 0.0;
    lutamm_timings acc{};
    for (uint32_t round = 0; round < WARMUP_ROUND + RECORD_ROUND; ++round) {
        std::cout << "---------- ROUND " << round << " ----------" << std::endl;
        t1 = W_time();
        rc = amm_host(ctx, input.data(), centroid.data(), lut.data(), bias.data(), output.data(), ip, lp);
        const double t = W_time() - t1;
        if (rc != LUTAMM_OK) {
            std::cerr << "amm_host failed: " << lutamm_last_error(ctx) << std::endl;
            return 1;
        }
        std::cout << "PIM AMM time " << t << std::endl;
        if (round >= WARMUP_ROUND) {
            total += t;
            lutamm_timings tm;
            if (breakdown && lutamm_get_timings(ctx, &tm) == LUTAMM_OK) {
                acc.index_calc_ms += tm.index_calc_ms;
                acc.lut_kernel_ms += tm.lut_kernel_ms;
                acc.data_transfer_ms += tm.data_transfer_ms;
                // the reference's AMM_BREAKDOWN lines (amm_host.cpp:25, pim_lut_host.cpp:210)
                std::printf("index calculation time %.6f\n", acc.index_calc_ms * 1e-3);
                std::printf("other latency %.6f, data transfer latency %.6f, pim kernel latency %.6f\n", 0.0,
                            acc.data_transfer_ms * 1e-3, acc.lut_kernel_ms * 1e-3);
            }
        }
    }
    std::cout << "warm up rounds " << WARMUP_ROUND << ", record rounds " << RECORD_ROUND << std::endl;
    std::cout << "PIM AVG AMM time " << total / RECORD_ROUND << std::endl;
    std::cout << "tokens per second " << ip.n / (total / RECORD_ROUND) << std::endl;
    double checksum = 0;
    for (size_t i = 0; i < n_out; i += 997) checksum += output[i];
    std::cout << "output checksum " << checksum << std::endl;
    amm_host_forget(ctx);
    lutamm_destroy(ctx);
    return 0;
}
