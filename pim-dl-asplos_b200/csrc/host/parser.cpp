#include "parser.h"

#include <cstdlib>
#include <iostream>

#include "yaml_lite.h"

namespace {

struct Reader {
    const yaml_lite::Doc& doc;
    std::string err;
    bool u32(const char* sec, const char* key, uint32_t* out, bool required, uint32_t dflt = 0) {
        const std::string* v = doc.find(sec, key);
        if (!v) {
            if (required) { err = std::string("missing ") + sec + "." + key; return false; }
            *out = dflt;
            return true;
        }
        char* end = nullptr;
        unsigned long x = std::strtoul(v->c_str(), &end, 10);
        if (end == v->c_str() || *end != 0) { err = std::string(sec) + "." + key + ": not an unsigned integer: " + *v; return false; }
        *out = static_cast<uint32_t>(x);
        return true;
    }
    bool f32(const char* sec, const char* key, float* out, bool required, float dflt = 0.f) {
        const std::string* v = doc.find(sec, key);
        if (!v) {
            if (required) { err = std::string("missing ") + sec + "." + key; return false; }
            *out = dflt;
            return true;
        }
        char* end = nullptr;
        float x = std::strtof(v->c_str(), &end);
        if (end == v->c_str() || *end != 0) { err = std::string(sec) + "." + key + ": not a number: " + *v; return false; }
        *out = x;
        return true;
    }
};

}  // namespace

bool parse_amm_configs(AMMParams& p, const std::string& yaml_path, std::string* error, bool verbose) {
    yaml_lite::Doc doc;
    if (!yaml_lite::load(yaml_path, &doc, error)) return false;
    Reader r{doc, {}};
    p = AMMParams{};
    IndexCalcParams& ip = p.index_params;
    LUTParams& lp = p.lut_params;
    const char* S = "system_params";
    const char* A = "amm_shape_params";
    const char* K = "kernel_params";

    uint32_t nr_tasklets = 0, lut_load_type = 0, loop_order = 0;
    bool ok = r.u32(A, "n", &ip.n, true) && r.u32(A, "input_feature_len", &ip.input_feature_len, true) &&
              r.u32(A, "num_codebook", &ip.num_codebook, true) && r.u32(A, "num_centroid", &ip.num_centroid, true) &&
              r.u32(A, "output_feature_len", &lp.output_feature_len, true) && r.f32(A, "scale", &lp.scale, true) &&
              r.f32(A, "bias", &lp.bias, false, 0.f) && r.u32(S, "num_threads", &ip.num_threads, false, 1) &&
              r.u32(S, "dpu_num", &lp.dpu_num, false, 0) && r.u32(S, "nr_tasklets", &nr_tasklets, false, 0) &&
              r.u32(S, "gpu_device", &p.gpu_device, false, 0);
    if (!ok) { *error = yaml_path + ": " + r.err; return false; }
    if (!ip.n || !ip.input_feature_len || !ip.num_codebook || !ip.num_centroid || !lp.output_feature_len) {
        *error = yaml_path + ": amm_shape_params must all be positive";
        return false;
    }
    if (ip.input_feature_len % ip.num_codebook) {  // parser.cpp:57
        *error = yaml_path + ": input_feature_len is not a multiple of num_codebook";
        return false;
    }
    ip.sub_vec_len = ip.input_feature_len / ip.num_codebook;  // parser.cpp:26
    lp.n = ip.n;
    lp.num_codebook = ip.num_codebook;
    lp.num_centroid = ip.num_centroid;
    lp.num_threads = ip.num_threads;

    const bool have_kernel = doc.find(K, "n_stile_size") != nullptr;
    if (have_kernel) {
        ok = r.u32(K, "n_stile_size", &lp.n_stile_size, true) && r.u32(K, "feature_stile_size", &lp.feature_stile_size, true) &&
             r.u32(K, "n_mtile_size", &lp.n_mtile_size, true) && r.u32(K, "feature_mtile_size", &lp.feature_mtile_size, true) &&
             r.u32(K, "cb_mtile_size", &lp.cb_mtile_size, true) &&
             r.u32(K, "feature_load_tile_size", &lp.feature_load_tile_size, true) &&
             r.u32(K, "cb_load_tile_size", &lp.cb_load_tile_size, true) && r.u32(K, "lut_load_type", &lut_load_type, true) &&
             r.u32(K, "loop_order", &loop_order, false, 0);
        if (!ok) { *error = yaml_path + ": " + r.err; return false; }
        if (!lp.n_stile_size || !lp.feature_stile_size || !lp.n_mtile_size || !lp.feature_mtile_size || !lp.cb_mtile_size ||
            !lp.feature_load_tile_size || !lp.cb_load_tile_size || lut_load_type > 2) {
            *error = yaml_path + ": kernel_params tile sizes must be positive and lut_load_type in 0..2";
            return false;
        }
        lp.lut_load_type = static_cast<LUTLoadType>(lut_load_type);
        lp.input_parallelism = lp.n / lp.n_stile_size;                             // parser.cpp:41
        lp.lut_parallelism = lp.output_feature_len / lp.feature_stile_size;        // parser.cpp:42
        // the reference's asserts (parser.cpp:59-69), as errors
        struct { bool bad; const char* what; } checks[] = {
            {lp.dpu_num && lp.input_parallelism * lp.lut_parallelism != lp.dpu_num, "input_parallelism * lut_parallelism != dpu_num"},
            {lp.n != lp.n_stile_size * lp.input_parallelism, "n is not a multiple of n_stile_size"},
            {lp.output_feature_len != lp.feature_stile_size * lp.lut_parallelism, "output_feature_len is not a multiple of feature_stile_size"},
            {lp.n_stile_size % lp.n_mtile_size != 0, "n_stile_size % n_mtile_size != 0"},
            {lp.feature_stile_size % lp.feature_mtile_size != 0, "feature_stile_size % feature_mtile_size != 0"},
            {lp.num_codebook % lp.cb_mtile_size != 0, "num_codebook % cb_mtile_size != 0"},
            {lp.feature_mtile_size % lp.feature_load_tile_size != 0, "feature_mtile_size % feature_load_tile_size != 0"},
            {lp.cb_mtile_size % lp.cb_load_tile_size != 0, "cb_mtile_size % cb_load_tile_size != 0"},
            {nr_tasklets && lp.n_mtile_size % nr_tasklets != 0, "n_mtile_size % nr_tasklets != 0"},
        };
        for (const auto& c : checks)
            if (c.bad) { *error = yaml_path + ": " + c.what; return false; }
    } else {
        // one tile: canonical row-major index and output layouts
        lp.n_stile_size = lp.n_mtile_size = lp.n;
        lp.feature_stile_size = lp.feature_mtile_size = lp.feature_load_tile_size = lp.output_feature_len;
        lp.cb_mtile_size = lp.cb_load_tile_size = lp.num_codebook;
        lp.input_parallelism = lp.lut_parallelism = 1;
        lp.lut_load_type = STATIC;
    }
    ip.n_stile_size = lp.n_stile_size;
    ip.cb_mtile_size = lp.cb_mtile_size;

    GpuPlan& g = p.gpu_plan;
    ok = r.u32(K, "gpu_variant", &g.variant, false) && r.u32(K, "gpu_ccs_tokens", &g.ccs_tokens, false) &&
         r.u32(K, "gpu_gather_cfg", &g.gather_cfg, false) && r.u32(K, "gpu_umma_n_tile", &g.umma_n_tile, false) &&
         r.u32(K, "gpu_umma_split", &g.umma_split, false) && r.u32(K, "gpu_umma_stages", &g.umma_stages, false) &&
         r.u32(K, "gpu_umma_groups", &g.umma_groups, false) && r.u32(K, "gpu_umma_operand", &g.umma_operand, false) &&
         r.u32(K, "gpu_umma_sps", &g.umma_sps, false) && r.u32(K, "gpu_umma_epilogue", &g.umma_epilogue, false);
    if (!ok) { *error = yaml_path + ": " + r.err; return false; }

    if (verbose) {
        std::cout << "------ system params ------\n"
                  << "gpu device " << p.gpu_device << " (dpu num " << lp.dpu_num << ", num tasklets " << nr_tasklets
                  << ", num threads " << ip.num_threads << ": UPMEM/host settings, not used on the GPU)\n"
                  << "------ amm shape params ------\n"
                  << "num codebook " << ip.num_codebook << ", num centroid " << ip.num_centroid << "\n"
                  << "n " << ip.n << ", input feature len " << ip.input_feature_len << ", output feature len "
                  << lp.output_feature_len << "\n"
                  << "scale " << lp.scale << ", bias " << lp.bias << "\n"
                  << "------ kernel params ------\n"
                  << "n stile size " << lp.n_stile_size << ", feature stile size " << lp.feature_stile_size << "\n"
                  << "n mtile size " << lp.n_mtile_size << ", feature mtile size " << lp.feature_mtile_size
                  << ", cb mtile size " << lp.cb_mtile_size << "\n"
                  << "gpu plan: variant " << g.variant << " (0 auto, 1 gather, 2 tcgen05), n tile " << g.umma_n_tile
                  << ", split " << g.umma_split << ", operand " << g.umma_operand << ", gather cfg " << g.gather_cfg << "\n"
                  << "------ calculated params ------\n"
                  << "sub vec len " << ip.sub_vec_len << ", input parallelism " << lp.input_parallelism
                  << ", lut parallelism " << lp.lut_parallelism << std::endl;
    }
    return true;
}

namespace {

bool parse_linear(Reader& r, const yaml_lite::Doc& doc, const std::string& pre, uint32_t n, uint32_t K, uint32_t N,
                  uint32_t num_threads, uint32_t dpu_num, uint32_t nr_tasklets, AMMParams* out, std::string* why) {
    const char* Kp = "kernel_params";
    AMMParams p{};
    IndexCalcParams& ip = p.index_params;
    LUTParams& lp = p.lut_params;
    auto key = [&](const char* k) { return pre + "_" + k; };
    ip.n = lp.n = n;
    ip.input_feature_len = K;
    lp.output_feature_len = N;
    ip.num_threads = lp.num_threads = num_threads;
    lp.dpu_num = dpu_num;
    if (!(r.u32(Kp, key("num_codebook").c_str(), &ip.num_codebook, true) && r.u32(Kp, key("num_centroid").c_str(), &ip.num_centroid, true) &&
          r.f32(Kp, key("scale").c_str(), &lp.scale, false, 0.01f) && r.f32(Kp, key("bias").c_str(), &lp.bias, false, 0.f))) {
        *why = r.err;
        return false;
    }
    if (!ip.num_codebook || !ip.num_centroid) { *why = pre + ": num_codebook and num_centroid must be positive"; return false; }
    if (K % ip.num_codebook) { *why = pre + ": input feature length is not a multiple of num_codebook"; return false; }  // parser.cpp:395-410
    ip.sub_vec_len = K / ip.num_codebook;
    lp.num_codebook = ip.num_codebook;
    lp.num_centroid = ip.num_centroid;
    if (doc.find(Kp, key("input_parallelism"))) {
        uint32_t load_type = 0;
        if (!(r.u32(Kp, key("input_parallelism").c_str(), &lp.input_parallelism, true) && r.u32(Kp, key("lut_parallelism").c_str(), &lp.lut_parallelism, true) &&
              r.u32(Kp, key("n_mtile_size").c_str(), &lp.n_mtile_size, true) && r.u32(Kp, key("feature_mtile_size").c_str(), &lp.feature_mtile_size, true) &&
              r.u32(Kp, key("cb_mtile_size").c_str(), &lp.cb_mtile_size, true) && r.u32(Kp, key("lut_load_type").c_str(), &load_type, true) &&
              r.u32(Kp, key("feature_load_tile_size").c_str(), &lp.feature_load_tile_size, true) &&
              r.u32(Kp, key("cb_load_tile_size").c_str(), &lp.cb_load_tile_size, true))) {
            *why = r.err;
            return false;
        }
        if (!lp.input_parallelism || !lp.lut_parallelism || !lp.n_mtile_size || !lp.feature_mtile_size || !lp.cb_mtile_size ||
            !lp.feature_load_tile_size || !lp.cb_load_tile_size || load_type > 2) {
            *why = pre + ": mapping parameters must be positive and lut_load_type in 0..2";
            return false;
        }
        lp.lut_load_type = static_cast<LUTLoadType>(load_type);
        lp.feature_stile_size = N / lp.lut_parallelism;  // parser.cpp:128-129
        lp.n_stile_size = n / lp.input_parallelism;
        struct { bool bad; const char* what; } checks[] = {
            {dpu_num && lp.input_parallelism * lp.lut_parallelism != dpu_num, "input_parallelism * lut_parallelism != dpu_num"},
            {n != lp.n_stile_size * lp.input_parallelism, "n is not a multiple of input_parallelism"},
            {N != lp.feature_stile_size * lp.lut_parallelism, "output feature length is not a multiple of lut_parallelism"},
            {lp.n_stile_size % lp.n_mtile_size != 0, "n_stile_size % n_mtile_size != 0"},
            {lp.feature_stile_size % lp.feature_mtile_size != 0, "feature_stile_size % feature_mtile_size != 0"},
            {lp.num_codebook % lp.cb_mtile_size != 0, "num_codebook % cb_mtile_size != 0"},
            {lp.feature_mtile_size % lp.feature_load_tile_size != 0, "feature_mtile_size % feature_load_tile_size != 0"},
            {lp.cb_mtile_size % lp.cb_load_tile_size != 0, "cb_mtile_size % cb_load_tile_size != 0"},
            {nr_tasklets && lp.n_mtile_size % nr_tasklets != 0, "n_mtile_size % nr_tasklets != 0"},
        };
        for (const auto& c : checks)
            if (c.bad) { *why = pre + ": " + c.what; return false; }
    } else {
        lp.input_parallelism = lp.lut_parallelism = 1;
        lp.n_stile_size = lp.n_mtile_size = n;
        lp.feature_stile_size = lp.feature_mtile_size = lp.feature_load_tile_size = N;
        lp.cb_mtile_size = lp.cb_load_tile_size = lp.num_codebook;
        lp.lut_load_type = STATIC;
    }
    ip.n_stile_size = lp.n_stile_size;
    ip.cb_mtile_size = lp.cb_mtile_size;
    GpuPlan& g = p.gpu_plan;
    if (!(r.u32(Kp, key("gpu_variant").c_str(), &g.variant, false) && r.u32(Kp, key("gpu_ccs_tokens").c_str(), &g.ccs_tokens, false) &&
          r.u32(Kp, key("gpu_gather_cfg").c_str(), &g.gather_cfg, false) && r.u32(Kp, key("gpu_umma_n_tile").c_str(), &g.umma_n_tile, false) &&
          r.u32(Kp, key("gpu_umma_split").c_str(), &g.umma_split, false) && r.u32(Kp, key("gpu_umma_stages").c_str(), &g.umma_stages, false) &&
          r.u32(Kp, key("gpu_umma_groups").c_str(), &g.umma_groups, false) && r.u32(Kp, key("gpu_umma_operand").c_str(), &g.umma_operand, false) &&
          r.u32(Kp, key("gpu_umma_sps").c_str(), &g.umma_sps, false) &&
          r.u32(Kp, key("gpu_umma_epilogue").c_str(), &g.umma_epilogue, false))) {
        *why = r.err;
        return false;
    }
    *out = p;
    return true;
}

}  // namespace

bool parse_transformer_configs(TransformerParams& tp, const std::string& yaml_path, std::string* error, bool verbose) {
    yaml_lite::Doc doc;
    if (!yaml_lite::load(yaml_path, &doc, error)) return false;
    Reader r{doc, {}};
    tp = TransformerParams{};
    const char* S = "system_params";
    const char* Nw = "network_params";
    AttentionParams& at = tp.attention_params;
    uint32_t dpu_num = 0, nr_tasklets = 0;
    bool ok = r.u32(Nw, "seq_len", &at.seq_len, true) && r.u32(Nw, "batch_size", &at.batch_size, true) &&
              r.u32(Nw, "head_num", &at.head_num, true) && r.u32(Nw, "token_dim", &at.token_dim, true) &&
              r.u32(Nw, "head_dim", &at.head_dim, false, 0) && r.u32(Nw, "ffn_hidden_dim", &tp.ffn_hidden_dim, true) &&
              r.u32(Nw, "layer_num", &tp.layer_num, false, 1) && r.u32(S, "num_threads", &tp.num_threads, false, 1) &&
              r.u32(S, "dpu_num", &dpu_num, false, 0) && r.u32(S, "nr_tasklets", &nr_tasklets, false, 0) &&
              r.u32(S, "gpu_device", &tp.gpu_device, false, 0);
    if (!ok) { *error = yaml_path + ": " + r.err; return false; }
    if (!at.seq_len || !at.batch_size || !at.head_num || !at.token_dim || !tp.ffn_hidden_dim || !tp.layer_num) {
        *error = yaml_path + ": network_params must all be positive";
        return false;
    }
    if (!at.head_dim) at.head_dim = at.token_dim / at.head_num;
    if (at.head_dim * at.head_num != at.token_dim) { *error = yaml_path + ": head_dim * head_num != token_dim"; return false; }
    at.n = at.seq_len * at.batch_size;
    at.num_threads = tp.num_threads;
    at.dpu_num = dpu_num;
    static const char* kBin[4] = {"qkv_lut_pim_binary", "o_lut_pim_binary", "ffn1_lut_pim_binary", "ffn2_lut_pim_binary"};
    for (int i = 0; i < 4; ++i)
        if (const std::string* v = doc.find(S, kBin[i])) tp.pim_binary_list[i] = *v;
    const uint32_t n = at.n, D = at.token_dim, F = tp.ffn_hidden_dim;
    struct { const char* pre; uint32_t K, N; } lin[7] = {{"qkv", D, 3 * D}, {"o", D, D}, {"ffn1", D, F}, {"ffn2", F, D},
                                                         {"o", D, D}, {"o", D, D}, {"o", D, D}};  // 4-6: Q, K, V (parser.cpp:235-322)
    for (int i = 0; i < 7; ++i) {
        std::string why;
        if (!parse_linear(r, doc, lin[i].pre, n, lin[i].K, lin[i].N, tp.num_threads, dpu_num, nr_tasklets, &tp.amm_param_list[i], &why)) {
            *error = yaml_path + ": " + why;
            return false;
        }
        tp.amm_param_list[i].gpu_device = tp.gpu_device;
    }
    const LUTParams& q = tp.amm_param_list[0].lut_params;
    at.input_parallelism = q.input_parallelism;
    at.lut_parallelism = q.lut_parallelism;
    at.n_tile_size = q.n_stile_size;                   // parser.cpp:335-336
    at.token_tile_size = q.feature_stile_size / 3;
    if (verbose) {
        std::cout << "----------Transformer Params----------\n"
                  << "thread num " << tp.num_threads << "\nlayer num " << tp.layer_num << "\n";
        static const char* kName[4] = {"QKV", "O", "FFN1", "FFN2"};
        for (int i = 0; i < 4; ++i) {
            const AMMParams& a = tp.amm_param_list[i];
            std::cout << "----------" << kName[i] << " LUT Params----------\n"
                      << "n " << a.index_params.n << ", input feature len " << a.index_params.input_feature_len << ", output feature len "
                      << a.lut_params.output_feature_len << "\nnum codebook " << a.index_params.num_codebook << ", num centroid "
                      << a.index_params.num_centroid << ", sub vec len " << a.index_params.sub_vec_len << "\nscale " << a.lut_params.scale
                      << ", bias " << a.lut_params.bias << "\n";
        }
        std::cout << "----------Attention Params----------\n"
                  << "seq len " << at.seq_len << ", batch size " << at.batch_size << ", n " << at.n << "\nhead num " << at.head_num
                  << ", head dim " << at.head_dim << ", token dim " << at.token_dim << "\n-----------------------------------" << std::endl;
    }
    return true;
}
