#include "amm_host.h"

#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

namespace {

struct Key {
    lutamm_ctx* ctx;
    const void* centroid;
    const void* lut;
    const void* bias;
    bool operator<(const Key& o) const {
        return std::tie(ctx, centroid, lut, bias) < std::tie(o.ctx, o.centroid, o.lut, o.bias);
    }
};

// What the resident copy was loaded with: a later call that names the same three buffers but other
// parameter blocks (scale, LUT bias, shape, tile sizes, table layout) must not be served by it.
struct Resident {
    int id;
    IndexCalcParams ip;
    LUTParams lp;
    uint32_t lut_layout;
};

// Everything except `n` (the token count of the call, which the kernels take per call) and the
// host-thread counts decides what is resident or how the output is addressed.
bool same_params(const Resident& r, const IndexCalcParams& ip, const LUTParams& lp, uint32_t lut_layout) {
    IndexCalcParams a = r.ip, b = ip;
    LUTParams c = r.lp, d = lp;
    a.n = b.n = 0; a.num_threads = b.num_threads = 0;
    c.n = d.n = 0; c.num_threads = d.num_threads = 0;
    return r.lut_layout == lut_layout && std::memcmp(&a, &b, sizeof a) == 0 && std::memcmp(&c, &d, sizeof c) == 0;
}

std::mutex g_mu;
std::map<Key, Resident> g_layers;      // weights already resident -> layer id and what it was loaded with
std::map<lutamm_ctx*, int> g_next_id;  // ids handed out by amm_host() start high, away from user ids
constexpr int kFirstAutoId = 1 << 20;

}  // namespace

namespace {
int amm_host_impl(lutamm_ctx* ctx, float* input_tensor, float* centroid_tensor, lut_data_type* lut_table,
                  float* bias_tensor, float* output_tensor, IndexCalcParams index_params, LUTParams lut_params,
                  uint32_t lut_layout, uint32_t flags);
}

int amm_host(lutamm_ctx* ctx, float* input_tensor, float* centroid_tensor, lut_data_type* lut_table,
             float* bias_tensor, float* output_tensor, IndexCalcParams index_params, LUTParams lut_params) {
    return amm_host_impl(ctx, input_tensor, centroid_tensor, lut_table, bias_tensor, output_tensor, index_params,
                         lut_params, LUTAMM_LUT_CANONICAL, 0);
}

int amm_host_dpu_layout(lutamm_ctx* ctx, float* input_tensor, float* centroid_tensor, lut_data_type* dpu_lut_table,
                        float* bias_tensor, float* output_tensor, IndexCalcParams index_params, LUTParams lut_params) {
    return amm_host_impl(ctx, input_tensor, centroid_tensor, dpu_lut_table, bias_tensor, output_tensor, index_params,
                         lut_params, LUTAMM_LUT_DPU_TILED, LUTAMM_FLAG_OUTPUT_TILED);
}

namespace {
int amm_host_impl(lutamm_ctx* ctx, float* input_tensor, float* centroid_tensor, lut_data_type* lut_table,
                  float* bias_tensor, float* output_tensor, IndexCalcParams index_params, LUTParams lut_params,
                  uint32_t lut_layout, uint32_t flags) {
    int id;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        const Key k{ctx, centroid_tensor, lut_table, bias_tensor};
        auto it = g_layers.find(k);
        if (it != g_layers.end() && !same_params(it->second, index_params, lut_params, lut_layout)) {
            // same buffers, different operator: the resident copy is stale
            lutamm_unload_weights(ctx, it->second.id);
            g_layers.erase(it);
            it = g_layers.end();
        }
        if (it == g_layers.end()) {
            int& next = g_next_id[ctx];
            if (next < kFirstAutoId) next = kFirstAutoId;
            id = next++;
            const int rc = lutamm_load_weights_layout(ctx, id, centroid_tensor, lut_table, bias_tensor,
                                                      reinterpret_cast<const lutamm_index_params*>(&index_params),
                                                      reinterpret_cast<const lutamm_lut_params*>(&lut_params), lut_layout);
            if (rc != LUTAMM_OK) return rc;
            g_layers.emplace(k, Resident{id, index_params, lut_params, lut_layout});
        } else {
            id = it->second.id;
        }
    }
    return lutamm_amm(ctx, id, input_tensor, output_tensor, index_params.n, flags);
}
}  // namespace

int index_calculation(lutamm_ctx* ctx, int layer_id, float* input_tensor, uint8_t* lut_input_index, uint32_t n) {
    return lutamm_index_calculation(ctx, layer_id, input_tensor, lut_input_index, n, LUTAMM_INDEX_U8_ROWMAJOR);
}

int pim_lut(lutamm_ctx* ctx, int layer_id, uint8_t* input_index, float* output_tensor, uint32_t n) {
    return lutamm_pim_lut(ctx, layer_id, input_index, output_tensor, n, 0);
}

void amm_host_forget(lutamm_ctx* ctx) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto it = g_layers.begin(); it != g_layers.end();) {
        if (it->first.ctx == ctx) {
            lutamm_unload_weights(ctx, it->second.id);
            it = g_layers.erase(it);
        } else {
            ++it;
        }
    }
    g_next_id.erase(ctx);
}
