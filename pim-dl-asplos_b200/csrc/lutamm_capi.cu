// C ABI of the library (declared in include/lutamm.h): context, resident weights, the AMM
// operator and its two halves, plans, tuning and timing.  Everything below this file is
// CUDA for sm_100a; there is no CPU implementation of the operator in the library, so a
// machine without a usable device gets an error from lutamm_create, never a slow answer.
#include "../../include/lutamm.h"
#include "kernels.h"
#include "nccl_shard.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <vector>

using namespace lutamm;

namespace lutamm {

EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

}  // namespace lutamm

namespace {

constexpr int kNumUmmaTiles = 5;  // 64, 128, 160, 192, 256
inline int umma_tile_slot(uint32_t n_tile) { return n_tile == 64 ? 0 : n_tile == 128 ? 1 : n_tile == 160 ? 2 : n_tile == 192 ? 3 : 4; }

struct Layer {
    lutamm_index_params ip{};
    lutamm_lut_params lp{};
    uint32_t K = 0, v = 0, CB = 0, CT = 0, N = 0;
    float* d_centroid = nullptr;
    int8_t* d_lut = nullptr;    // canonical [CB][CT][N]
    int8_t* d_lut_t = nullptr;  // [N][CB*CT], made on first use of the tcgen05 variant
    float* d_bias = nullptr;
    lutamm_plan plan{};
    uint32_t act = LUTAMM_ACT_NONE;
    std::vector<CUtensorMap> gather_maps;
    std::vector<char> gather_map_ok;
    CUtensorMap umma_maps[kNumUmmaTiles];
    bool umma_map_ok[kNumUmmaTiles] = {false, false, false, false, false};
};

struct Buf {
    void* p = nullptr;
    size_t cap = 0;
};

}  // namespace

// Staging slots of the host-buffer pipeline.  With two, a slab's kernels wait for the copy-out of the slab before
// last, and copy-outs of very different sizes (3 to 12 MB per linear of a BERT-base layer) leave the link idle in
// between; a third decouples them (that layer's step through host buffers 0.69-0.74 -> 0.64 ms, BERT-large 6.6 ->
// 6.2 ms on the same box); a fourth adds nothing.
constexpr int kHostSlots = 3;

struct lutamm_ctx {
    int device = 0;
    int sm_count = 148;
    uint64_t unfused_exchanges = 0;  // sharded calls that asked for peer stores and got the kernel + all-gather
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    std::map<int, Layer> layers;
    Buf d_in, d_out, d_idx, d_idx16, d_acc_dbg, d_acc_scratch, d_counters, d_build;
    // host-buffer pipeline: copy-in and copy-out streams, kHostSlots staging slots
    cudaStream_t s_in = nullptr, s_out = nullptr;
    Buf p_in[kHostSlots], p_out[kHostSlots];
    cudaEvent_t ev_in[kHostSlots] = {}, ev_comp[kHostSlots] = {}, ev_out[kHostSlots] = {};
    uint32_t slot = 0;
    uint32_t* d_err = nullptr;
    uint32_t* h_err = nullptr;  // pinned
    bool timing = false;
    cudaEvent_t ev[6] = {};
    lutamm_timings last{};
    bool last_valid = false;
    uint64_t launches = 0;
    std::string err;
    // plans found by lutamm_tune, by shape: (n_tokens, K, N, CB, CT, SM count) -> plan
    std::map<std::vector<uint32_t>, lutamm_plan> plan_cache;
    // sharding across the GPUs of a box (lutamm_shard_init)
    lutamm::NcclComm comm = nullptr;
    int rank = 0, world = 1;
    // gathered-output buffers that every rank of the communicator can store into (lutamm_shard_alloc_gathered):
    // local base -> this buffer as mapped here on each rank (entry [rank] is the local base itself)
    std::map<void*, std::vector<void*>> peer_bufs;
    Buf d_sync;  // a few words for the small all-gathers that order ranks around the peer stores
};

namespace {

thread_local std::string g_noctx_err;

int fail(lutamm_ctx* c, int code, const std::string& msg) {
    if (c) c->err = msg; else g_noctx_err = msg;
    return code;
}

#define CU_TRY(c, expr)                                                                              \
    do {                                                                                             \
        cudaError_t e__ = (expr);                                                                    \
        if (e__ != cudaSuccess)                                                                      \
            return fail((c), LUTAMM_ECUDA, std::string(#expr) + ": " + cudaGetErrorString(e__));      \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
    }
    ~DeviceGuard() {
        if (ok && prev >= 0) cudaSetDevice(prev);
    }
};

// grow-only device buffer; `zero` clears newly allocated memory
int ensure(lutamm_ctx* c, Buf& b, size_t bytes, bool zero = false) {
    if (bytes <= b.cap) return LUTAMM_OK;
    // Stream order: everything queued so far may still use the old block.
    if (c->s_in) CU_TRY(c, cudaStreamSynchronize(c->s_in));
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    if (c->s_out) CU_TRY(c, cudaStreamSynchronize(c->s_out));
    if (b.p) CU_TRY(c, cudaFree(b.p));
    b.p = nullptr;
    b.cap = 0;
    size_t want = bytes + bytes / 4 + 256;
    cudaError_t e = cudaMalloc(&b.p, want);
    if (e != cudaSuccess) {
        want = bytes;
        e = cudaMalloc(&b.p, want);
    }
    if (e != cudaSuccess) return fail(c, LUTAMM_ENOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
    b.cap = want;
    if (zero) CU_TRY(c, cudaMemsetAsync(b.p, 0, want, c->stream));
    return LUTAMM_OK;
}

bool is_device_ptr(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

Layer* find_layer(lutamm_ctx* c, int id) {
    auto it = c->layers.find(id);
    return it == c->layers.end() ? nullptr : &it->second;
}

void free_layer(Layer& L) {
    cudaFree(L.d_centroid);
    cudaFree(L.d_lut);
    cudaFree(L.d_lut_t);
    cudaFree(L.d_bias);
    L = Layer{};
}

uint32_t resolve_variant(const lutamm_ctx* c, const Layer& L) {
    (void)c;
    uint32_t v = L.plan.variant;
    if (v == LUTAMM_VARIANT_AUTO) v = umma_supported(L.CB, L.CT, L.N) ? LUTAMM_VARIANT_UMMA : LUTAMM_VARIANT_GATHER;
    return v;
}

OutLayout make_layout(const Layer& L, uint32_t flags) {
    OutLayout o{};
    if (flags & LUTAMM_FLAG_OUTPUT_TILED) {
        o.tiled = 1;
        o.n_stile = L.lp.n_stile_size;
        o.f_stile = L.lp.feature_stile_size;
        o.f_mtile = L.lp.feature_mtile_size;
        o.lut_par = L.lp.lut_parallelism ? L.lp.lut_parallelism : (L.lp.feature_stile_size ? L.N / L.lp.feature_stile_size : 1);
    }
    return o;
}

int check_tiled(lutamm_ctx* c, const Layer& L, uint32_t M) {
    const lutamm_lut_params& p = L.lp;
    if (!p.n_stile_size || !p.feature_stile_size || !p.feature_mtile_size || M % p.n_stile_size ||
        L.N % p.feature_stile_size || p.feature_stile_size % p.feature_mtile_size)
        return fail(c, LUTAMM_EINVAL,
                    "tiled output needs n % n_stile_size == 0, output_feature_len % feature_stile_size == 0 and "
                    "feature_stile_size % feature_mtile_size == 0 (parser.cpp:61-63)");
    return LUTAMM_OK;
}

// step 2+3 on device buffers
int run_lut(lutamm_ctx* c, Layer& L, const uint8_t* d_idx, float* d_out, int32_t* d_acc_out, uint32_t M,
            uint32_t flags, const lutamm_plan& plan, float* const* peer_out = nullptr, uint32_t n_peers = 0) {
    LutArgs a{};
    if (peer_out && n_peers && n_peers <= kMaxPeers) {
        a.n_peers = n_peers;
        for (uint32_t g = 0; g < n_peers; ++g) a.peer_out[g] = peer_out[g];
    }
    a.idx = d_idx;
    a.bias = L.d_bias;
    a.out = d_out;
    a.acc_out = d_acc_out;
    a.M = M; a.CB = L.CB; a.CT = L.CT; a.N = L.N;
    a.scale = L.lp.scale;
    a.lut_bias = L.lp.bias;
    a.layout = make_layout(L, flags);
    a.act = L.act;
    const char* why = nullptr;
    uint32_t variant = plan.variant;
    if (variant == LUTAMM_VARIANT_AUTO) variant = resolve_variant(c, L);
    if (variant == LUTAMM_VARIANT_UMMA) {
        if (!umma_supported(L.CB, L.CT, L.N))
            return fail(c, LUTAMM_EUNSUPPORTED, "tcgen05 variant does not cover this shape (num_centroid a power of two in 8..256, num_codebook % 16 == 0)");
        UmmaPlan up;
        umma_default_plan(M, L.CB, L.CT, L.N, c->sm_count, plan.umma_operand, plan.umma_n_tile, plan.umma_sps, &up);
        const bool a_tmem = up.a_tmem != 0;
        if (plan.umma_split) up.split = plan.umma_split;
        up.stages = plan.umma_stages;
        up.groups = plan.umma_groups;
        if (plan.umma_sps) up.sps = plan.umma_sps;
        up.epilogue = plan.umma_epilogue;
        if (!umma_tile_ok(up.n_tile, a_tmem))
            return fail(c, LUTAMM_EINVAL, "umma_n_tile must be 64, 128 or 256 with the one-hot operand in shared memory, "
                                          "64, 128, 160 or 192 with it in tensor memory");
        if (!L.d_lut_t) {
            // First tcgen05 call for this layer: make the K-major copy of the table.  The kernel that
            // follows is a programmatic dependent launch whose TMA producer does not wait for the
            // preceding grid, so the copy has to be complete - not merely queued - before it starts.
            const size_t bytes = (size_t)L.CB * L.CT * L.N;
            CU_TRY(c, cudaMalloc(&L.d_lut_t, bytes));
            cudaError_t te = launch_transpose_lut(L.d_lut, L.d_lut_t, L.CB * L.CT, L.N, c->stream);
            if (te == cudaSuccess) te = cudaStreamSynchronize(c->stream);
            if (te != cudaSuccess) {
                cudaFree(L.d_lut_t);
                L.d_lut_t = nullptr;
                return fail(c, LUTAMM_ECUDA, std::string("LUT transpose: ") + cudaGetErrorString(te));
            }
            ++c->launches;
        }
        const int slot = umma_tile_slot(up.n_tile);
        if (!L.umma_map_ok[slot]) {
            cudaError_t e = umma_make_tmap(&L.umma_maps[slot], L.d_lut_t, L.CB, L.CT, L.N, up.n_tile, &why);
            if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, why ? why : cudaGetErrorString(e));
            L.umma_map_ok[slot] = true;
        }
        if (up.split > 1) {
            const uint32_t tiles = ((M + 127) / 128) * ((L.N + up.n_tile - 1) / up.n_tile);
            int r = ensure(c, c->d_acc_scratch, (size_t)up.split * M * L.N * sizeof(int32_t), false);
            if (r) return r;
            r = ensure(c, c->d_counters, (size_t)tiles * 2 * sizeof(uint32_t), true);  // arrived / done per tile
            if (r) return r;
        }
        cudaError_t e = launch_umma(a, L.umma_maps[slot], up, static_cast<int32_t*>(c->d_acc_scratch.p),
                                    static_cast<uint32_t*>(c->d_counters.p), c->d_err, c->stream, &why);
        if (e == cudaErrorNotSupported && a.n_peers) return fail(c, LUTAMM_EUNSUPPORTED, why ? why : "peer stores not built for this plan");
        if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, why ? why : (std::string("tcgen05 launch: ") + cudaGetErrorString(e)));
        ++c->launches;
        return LUTAMM_OK;
    }
    if (a.n_peers) return fail(c, LUTAMM_EUNSUPPORTED, "peer stores exist in the tcgen05 kernel only");
    if (variant != LUTAMM_VARIANT_GATHER) return fail(c, LUTAMM_EINVAL, "unknown kernel variant");
    uint32_t cfg = plan.gather_cfg;
    if (cfg >= gather_num_cfgs()) return fail(c, LUTAMM_EINVAL, "unknown gather tile configuration");
    if (L.gather_maps.size() != gather_num_cfgs()) {
        L.gather_maps.resize(gather_num_cfgs());
        L.gather_map_ok.assign(gather_num_cfgs(), 0);
    }
    if (!L.gather_map_ok[cfg]) {
        cudaError_t e = gather_make_tmap(&L.gather_maps[cfg], L.d_lut, L.CB, L.CT, L.N, cfg, &why);
        if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, why ? why : cudaGetErrorString(e));
        L.gather_map_ok[cfg] = 1;
    }
    cudaError_t e = launch_gather(a, L.gather_maps[cfg], cfg, c->d_err, c->stream, &why);
    if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, why ? why : (std::string("gather launch: ") + cudaGetErrorString(e)));
    ++c->launches;
    return LUTAMM_OK;
}

int run_ccs(lutamm_ctx* c, Layer& L, const float* d_x, void* d_idx, uint32_t M, uint32_t format, int ccs_tokens = -1) {
    CcsArgs a{};
    a.x = d_x;
    a.centroid = L.d_centroid;
    a.idx_out = d_idx;
    a.M = M; a.K = L.K; a.v = L.v; a.CB = L.CB; a.CT = L.CT;
    a.format = format;
    a.n_stile = L.ip.n_stile_size;
    a.cb_mtile = L.ip.cb_mtile_size;
    a.tokens_per_thread = ccs_tokens >= 0 ? (uint32_t)ccs_tokens : L.plan.ccs_tokens;
    const char* why = nullptr;
    cudaError_t e = launch_ccs(a, c->stream, &why);
    if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, why ? why : (std::string("search launch: ") + cudaGetErrorString(e)));
    ++c->launches;
    return LUTAMM_OK;
}

// read back the device error word after a synchronisation
int check_dev_err(lutamm_ctx* c) {
    if (c->s_in) CU_TRY(c, cudaStreamSynchronize(c->s_in));
    CU_TRY(c, cudaMemcpyAsync(c->h_err, c->d_err, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    if (c->s_out) CU_TRY(c, cudaStreamSynchronize(c->s_out));
    if (*c->h_err) {
        const uint32_t code = *c->h_err;
        cudaMemsetAsync(c->d_err, 0, sizeof(uint32_t), c->stream);
        // a kernel that gave up may have left split-K tile counters half counted
        if (c->d_counters.p) cudaMemsetAsync(c->d_counters.p, 0, c->d_counters.cap, c->stream);
        return fail(c, LUTAMM_EDEVICE, "a kernel gave up on a bounded wait (code " + std::to_string(code) + "); output is not valid");
    }
    return LUTAMM_OK;
}

// Host buffers on both sides: a three-stream pipeline.  Rows go through in chunks; chunk j is
// copied in on s_in, computed on the context's stream and copied out on s_out, each stage
// ordered by events, with three staging slots so that the copy-in of the next chunk (or of the
// next call, with LUTAMM_FLAG_ASYNC), the kernels and the copy-out of the previous one overlap
// and both directions of the host link are busy at once.  The reference's counterpart are the
// serial host<->DPU transfers around dpu_launch (pim_lut_host.cpp:143-181).
int amm_host_pipelined(lutamm_ctx* c, Layer& L, const float* input, float* output, uint32_t M, uint32_t flags) {
    // Token slabs of at least 512 rows, at most four per call: a call's first copy-in and last copy-out overlap
    // nothing, so halving them pays (BERT-base at 1024 tokens: 0.80 -> 0.73 ms per four-linear step through host
    // buffers), while slabs of 256 rows or more than four slabs cost more in small copies and launches than they hide.
    uint32_t chunks = M >= 1024 ? M / 512 : 1;
    if (chunks > 4) chunks = 4;
    uint32_t rows = ((M + chunks - 1) / chunks + 127) / 128 * 128;
    if ((flags & LUTAMM_FLAG_OUTPUT_TILED) || rows >= M) { rows = M; }
    int r;
    if ((r = ensure(c, c->d_idx, (size_t)rows * L.CB))) return r;
    constexpr uint32_t n_slots = kHostSlots;
    for (uint32_t k = 0; k < n_slots; ++k) {
        if ((r = ensure(c, c->p_in[k], (size_t)rows * L.K * sizeof(float)))) return r;
        if ((r = ensure(c, c->p_out[k], (size_t)rows * L.N * sizeof(float)))) return r;
    }
    for (uint32_t m0 = 0; m0 < M; m0 += rows) {
        const uint32_t m = std::min(rows, M - m0);
        const uint32_t k = c->slot++ % n_slots;
        float* d_x = static_cast<float*>(c->p_in[k].p);
        float* d_y = static_cast<float*>(c->p_out[k].p);
        CU_TRY(c, cudaStreamWaitEvent(c->s_in, c->ev_comp[k], 0));   // kernels that read this slot are done
        CU_TRY(c, cudaMemcpyAsync(d_x, input + (size_t)m0 * L.K, (size_t)m * L.K * sizeof(float), cudaMemcpyHostToDevice, c->s_in));
        CU_TRY(c, cudaEventRecord(c->ev_in[k], c->s_in));
        CU_TRY(c, cudaStreamWaitEvent(c->stream, c->ev_in[k], 0));
        CU_TRY(c, cudaStreamWaitEvent(c->stream, c->ev_out[k], 0));  // the slot's previous result has left
        if ((r = run_ccs(c, L, d_x, c->d_idx.p, m, LUTAMM_INDEX_U8_ROWMAJOR))) return r;
        if ((r = run_lut(c, L, static_cast<const uint8_t*>(c->d_idx.p), d_y, nullptr, m, flags, L.plan))) return r;
        CU_TRY(c, cudaEventRecord(c->ev_comp[k], c->stream));
        CU_TRY(c, cudaStreamWaitEvent(c->s_out, c->ev_comp[k], 0));
        CU_TRY(c, cudaMemcpyAsync(output + (size_t)m0 * L.N, d_y, (size_t)m * L.N * sizeof(float), cudaMemcpyDeviceToHost, c->s_out));
        CU_TRY(c, cudaEventRecord(c->ev_out[k], c->s_out));
    }
    if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
    return check_dev_err(c);
}

int amm_impl(lutamm_ctx* c, int layer_id, const float* input, float* output, uint32_t M, uint8_t* idx_out,
             int32_t* acc_out, uint32_t flags) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (M == 0) return LUTAMM_OK;
    if (!input || !output) return fail(c, LUTAMM_EINVAL, "null input or output");
    if ((flags & LUTAMM_FLAG_OUTPUT_TILED)) {
        int r = check_tiled(c, *L, M);
        if (r) return r;
    }
    const bool in_dev = is_device_ptr(input), out_dev = is_device_ptr(output);
    const bool both_host = !in_dev && !out_dev;
    if ((flags & LUTAMM_FLAG_ASYNC) && !(((in_dev && out_dev) || both_host) && !idx_out && !acc_out))
        return fail(c, LUTAMM_EINVAL, "LUTAMM_FLAG_ASYNC needs input and output both in device memory or both in host memory, and no debug outputs");
    if (both_host && !idx_out && !acc_out && !c->timing) return amm_host_pipelined(c, *L, input, output, M, flags);
    if (in_dev && (reinterpret_cast<uintptr_t>(input) & 3u)) return fail(c, LUTAMM_EINVAL, "input is not 4-byte aligned");
    if (out_dev && (reinterpret_cast<uintptr_t>(output) & 15u)) return fail(c, LUTAMM_EINVAL, "device output must be 16-byte aligned");

    const size_t in_bytes = (size_t)M * L->K * sizeof(float), out_bytes = (size_t)M * L->N * sizeof(float);
    int r;
    const float* d_x = input;
    float* d_y = output;
    const bool t = c->timing;
    if (t) CU_TRY(c, cudaEventRecord(c->ev[0], c->stream));
    if (!in_dev) {
        if ((r = ensure(c, c->d_in, in_bytes))) return r;
        CU_TRY(c, cudaMemcpyAsync(c->d_in.p, input, in_bytes, cudaMemcpyHostToDevice, c->stream));
        d_x = static_cast<const float*>(c->d_in.p);
    }
    if (!out_dev) {
        if ((r = ensure(c, c->d_out, out_bytes))) return r;
        d_y = static_cast<float*>(c->d_out.p);
    }
    if ((r = ensure(c, c->d_idx, (size_t)M * L->CB))) return r;
    int32_t* d_acc = nullptr;
    if (acc_out) {
        if ((r = ensure(c, c->d_acc_dbg, (size_t)M * L->N * sizeof(int32_t)))) return r;
        d_acc = static_cast<int32_t*>(c->d_acc_dbg.p);
    }
    if (t) CU_TRY(c, cudaEventRecord(c->ev[1], c->stream));
    if ((r = run_ccs(c, *L, d_x, c->d_idx.p, M, LUTAMM_INDEX_U8_ROWMAJOR))) return r;
    if (t) CU_TRY(c, cudaEventRecord(c->ev[2], c->stream));
    if ((r = run_lut(c, *L, static_cast<const uint8_t*>(c->d_idx.p), d_y, d_acc, M, flags, L->plan))) return r;
    if (t) CU_TRY(c, cudaEventRecord(c->ev[3], c->stream));
    if (!out_dev) CU_TRY(c, cudaMemcpyAsync(output, d_y, out_bytes, cudaMemcpyDeviceToHost, c->stream));
    if (idx_out)
        CU_TRY(c, cudaMemcpyAsync(idx_out, c->d_idx.p, (size_t)M * L->CB, cudaMemcpyDefault, c->stream));
    if (acc_out)
        CU_TRY(c, cudaMemcpyAsync(acc_out, d_acc, (size_t)M * L->N * sizeof(int32_t), cudaMemcpyDefault, c->stream));
    if (t) CU_TRY(c, cudaEventRecord(c->ev[4], c->stream));
    if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
    if ((r = check_dev_err(c))) return r;
    if (t) {
        float a01 = 0, a12 = 0, a23 = 0, a34 = 0;
        cudaEventElapsedTime(&a01, c->ev[0], c->ev[1]);
        cudaEventElapsedTime(&a12, c->ev[1], c->ev[2]);
        cudaEventElapsedTime(&a23, c->ev[2], c->ev[3]);
        cudaEventElapsedTime(&a34, c->ev[3], c->ev[4]);
        c->last.data_transfer_ms = a01 + a34;
        c->last.index_calc_ms = a12;
        c->last.lut_kernel_ms = a23;
        c->last.total_ms = a01 + a12 + a23 + a34;
        c->last_valid = true;
    }
    return LUTAMM_OK;
}

}  // namespace

// =========================================================================== C ABI
extern "C" {

const char* lutamm_version(void) { return "lutamm-b200 0.1 (sm_100a)"; }

int lutamm_create(lutamm_ctx** out, int device) {
    if (!out) return fail(nullptr, LUTAMM_EINVAL, "null out pointer");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(nullptr, LUTAMM_ECUDA, std::string("no usable CUDA device: ") + cudaGetErrorString(e));
    if (device < 0 || device >= n) return fail(nullptr, LUTAMM_EINVAL, "device ordinal out of range");
    cudaDeviceProp prop;
    CU_TRY(nullptr, cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(nullptr, LUTAMM_EUNSUPPORTED, "this library is built for sm_100a (B200) only; found sm_" +
                                                       std::to_string(prop.major) + std::to_string(prop.minor));
    lutamm_ctx* c = new (std::nothrow) lutamm_ctx();
    if (!c) return fail(nullptr, LUTAMM_ENOMEM, "out of host memory");
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    DeviceGuard g(device);
    if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&c->d_err, sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(c->d_err, 0, sizeof(uint32_t)) != cudaSuccess ||
        cudaMallocHost(&c->h_err, sizeof(uint32_t)) != cudaSuccess) {
        std::string m = std::string("context set-up failed: ") + cudaGetErrorString(cudaGetLastError());
        delete c;
        return fail(nullptr, LUTAMM_ECUDA, m);
    }
    *c->h_err = 0;
    c->stream = c->own_stream;
    for (auto& ev : c->ev) cudaEventCreate(&ev);
    cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking);
    cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking);
    for (int k = 0; k < kHostSlots; ++k) {
        cudaEventCreateWithFlags(&c->ev_in[k], cudaEventDisableTiming);
        cudaEventCreateWithFlags(&c->ev_comp[k], cudaEventDisableTiming);
        cudaEventCreateWithFlags(&c->ev_out[k], cudaEventDisableTiming);
    }
    *out = c;
    return LUTAMM_OK;
}

int lutamm_destroy(lutamm_ctx* c) {
    if (!c) return LUTAMM_OK;
    DeviceGuard g(c->device);
    if (c->s_in) cudaStreamSynchronize(c->s_in);
    cudaStreamSynchronize(c->stream);
    if (c->s_out) cudaStreamSynchronize(c->s_out);
    for (auto& kv : c->peer_bufs) {
        for (size_t g = 0; g < kv.second.size(); ++g)
            if ((int)g != c->rank && kv.second[g]) cudaIpcCloseMemHandle(kv.second[g]);
        cudaFree(kv.first);
    }
    c->peer_bufs.clear();
    cudaFree(c->d_sync.p);
    if (c->comm && nccl_api().ok) nccl_api().comm_destroy(c->comm);
    c->comm = nullptr;
    for (auto& kv : c->layers) free_layer(kv.second);
    for (int k = 0; k < kHostSlots; ++k) {
        cudaFree(c->p_in[k].p); cudaFree(c->p_out[k].p);
        if (c->ev_in[k]) cudaEventDestroy(c->ev_in[k]);
        if (c->ev_comp[k]) cudaEventDestroy(c->ev_comp[k]);
        if (c->ev_out[k]) cudaEventDestroy(c->ev_out[k]);
    }
    if (c->s_in) cudaStreamDestroy(c->s_in);
    if (c->s_out) cudaStreamDestroy(c->s_out);
    for (Buf* b : {&c->d_in, &c->d_out, &c->d_idx, &c->d_idx16, &c->d_acc_dbg, &c->d_acc_scratch, &c->d_counters,
                   &c->d_build})
        cudaFree(b->p);
    cudaFree(c->d_err);
    cudaFreeHost(c->h_err);
    for (auto& ev : c->ev)
        if (ev) cudaEventDestroy(ev);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
    return LUTAMM_OK;
}

int lutamm_set_stream(lutamm_ctx* c, void* cuda_stream) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    c->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : c->own_stream;
    return LUTAMM_OK;
}

int lutamm_sync(lutamm_ctx* c) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    return check_dev_err(c);
}

const char* lutamm_last_error(const lutamm_ctx* c) { return c ? c->err.c_str() : g_noctx_err.c_str(); }

int lutamm_load_weights(lutamm_ctx* c, int layer_id, const float* centroid, const int8_t* lut, const float* bias,
                        const lutamm_index_params* ip, const lutamm_lut_params* lp) {
    return lutamm_load_weights_layout(c, layer_id, centroid, lut, bias, ip, lp, LUTAMM_LUT_CANONICAL);
}

int lutamm_load_weights_layout(lutamm_ctx* c, int layer_id, const float* centroid, const int8_t* lut, const float* bias,
                               const lutamm_index_params* ip, const lutamm_lut_params* lp, uint32_t lut_layout) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!centroid || !lut || !bias || !ip || !lp) return fail(c, LUTAMM_EINVAL, "null argument");
    const uint32_t K = ip->input_feature_len, CB = ip->num_codebook, CT = ip->num_centroid, N = lp->output_feature_len;
    if (!K || !CB || !CT || !N) return fail(c, LUTAMM_EINVAL, "zero-sized shape parameter");
    if (K % CB) return fail(c, LUTAMM_EINVAL, "input_feature_len % num_codebook != 0 (parser.cpp:57)");
    const uint32_t v = K / CB;
    if (ip->sub_vec_len && ip->sub_vec_len != v)
        return fail(c, LUTAMM_EINVAL, "sub_vec_len != input_feature_len / num_codebook (parser.cpp:26)");
    if (lp->num_codebook != CB || lp->num_centroid != CT)
        return fail(c, LUTAMM_EINVAL, "index and LUT parameter blocks disagree on num_codebook / num_centroid");
    if (lut_layout != LUTAMM_LUT_CANONICAL && lut_layout != LUTAMM_LUT_DPU_TILED) return fail(c, LUTAMM_EINVAL, "unknown LUT layout");
    if (CT > 256) return fail(c, LUTAMM_EINVAL, "num_centroid > 256 does not fit the uint8 index");
    if (N % 16) return fail(c, LUTAMM_EINVAL, "output_feature_len must be a multiple of 16");
    if ((uint64_t)CB * CT * N >= (1ull << 40)) return fail(c, LUTAMM_EINVAL, "LUT too large");
    DeviceGuard g(c->device);
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    Layer* old = find_layer(c, layer_id);
    if (old) free_layer(*old);
    Layer& L = c->layers[layer_id];
    L.ip = *ip; L.lp = *lp;
    L.K = K; L.v = v; L.CB = CB; L.CT = CT; L.N = N;
    const size_t cb = (size_t)CB * CT * v * sizeof(float), lb = (size_t)CB * CT * N, bb = (size_t)N * sizeof(float);
    cudaError_t e;
    if ((e = cudaMalloc(&L.d_centroid, cb)) != cudaSuccess || (e = cudaMalloc(&L.d_lut, lb)) != cudaSuccess ||
        (e = cudaMalloc(&L.d_bias, bb)) != cudaSuccess) {
        free_layer(L);
        c->layers.erase(layer_id);
        return fail(c, LUTAMM_ENOMEM, std::string("cudaMalloc for weights: ") + cudaGetErrorString(e));
    }
    CU_TRY(c, cudaMemcpyAsync(L.d_centroid, centroid, cb, cudaMemcpyDefault, c->stream));
    if (lut_layout == LUTAMM_LUT_DPU_TILED) {
        // the table as the reference sends it to the DPUs: stage it, then un-tile on the device
        const uint32_t T = lp->lut_load_type == 0 ? lp->feature_stile_size : lp->feature_load_tile_size;
        int r = ensure(c, c->d_build, lb);
        if (r) { free_layer(L); c->layers.erase(layer_id); return r; }
        CU_TRY(c, cudaMemcpyAsync(c->d_build.p, lut, lb, cudaMemcpyDefault, c->stream));
        const char* why = nullptr;
        cudaError_t ue = launch_lut_untile(static_cast<const int8_t*>(c->d_build.p), L.d_lut, CB * CT, N, T, c->stream, &why);
        if (ue != cudaSuccess) {
            free_layer(L);
            c->layers.erase(layer_id);
            return fail(c, why ? LUTAMM_EINVAL : LUTAMM_ECUDA, why ? std::string(why) : std::string("LUT un-tiling: ") + cudaGetErrorString(ue));
        }
        c->launches += 1;
    } else {
        CU_TRY(c, cudaMemcpyAsync(L.d_lut, lut, lb, cudaMemcpyDefault, c->stream));
    }
    CU_TRY(c, cudaMemcpyAsync(L.d_bias, bias, bb, cudaMemcpyDefault, c->stream));
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    L.plan = lutamm_plan{};
    return LUTAMM_OK;
}

int lutamm_build_lut(lutamm_ctx* c, const float* centroid, const float* weight, uint32_t CB, uint32_t CT, uint32_t v,
                     uint32_t N, int8_t* lut_out, float* scale_out, float* lut_bias_out) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!centroid || !weight || !lut_out || !scale_out || !lut_bias_out) return fail(c, LUTAMM_EINVAL, "null argument");
    if (!CB || !CT || !v || !N) return fail(c, LUTAMM_EINVAL, "zero-sized shape parameter");
    if (N % 4) return fail(c, LUTAMM_EINVAL, "output_feature_len must be a multiple of 4");
    DeviceGuard g(c->device);
    const size_t cen_b = (size_t)CB * CT * v * sizeof(float), w_b = (size_t)CB * v * N * sizeof(float),
                 lut_b = (size_t)CB * CT * N;
    // staging for whichever of the three tensors lives in host memory; [0..255] holds the scalars
    const bool cen_dev = is_device_ptr(centroid), w_dev = is_device_ptr(weight), lut_dev = is_device_ptr(lut_out);
    const size_t off_cen = 256, off_w = off_cen + (cen_dev ? 0 : (cen_b + 255) / 256 * 256),
                 off_lut = off_w + (w_dev ? 0 : (w_b + 255) / 256 * 256), total = off_lut + (lut_dev ? 0 : lut_b);
    if (int rc = ensure(c, c->d_build, total)) return rc;
    char* base = static_cast<char*>(c->d_build.p);
    const float* d_cen = centroid;
    const float* d_w = weight;
    int8_t* d_lut = lut_out;
    if (!cen_dev) {
        CU_TRY(c, cudaMemcpyAsync(base + off_cen, centroid, cen_b, cudaMemcpyHostToDevice, c->stream));
        d_cen = reinterpret_cast<const float*>(base + off_cen);
    }
    if (!w_dev) {
        CU_TRY(c, cudaMemcpyAsync(base + off_w, weight, w_b, cudaMemcpyHostToDevice, c->stream));
        d_w = reinterpret_cast<const float*>(base + off_w);
    }
    if (!lut_dev) d_lut = reinterpret_cast<int8_t*>(base + off_lut);
    LutBuildArgs a{d_cen, d_w, d_lut, reinterpret_cast<uint32_t*>(base), reinterpret_cast<float*>(base + 16),
                   reinterpret_cast<float*>(base + 32), CB, CT, v, N};
    const char* why = nullptr;
    cudaError_t e = launch_lut_build(a, c->stream, &why);
    if (e != cudaSuccess)
        return fail(c, why ? LUTAMM_EINVAL : LUTAMM_ECUDA, why ? std::string(why) : std::string("lut build: ") + cudaGetErrorString(e));
    c->launches += 3;
    if (!lut_dev) CU_TRY(c, cudaMemcpyAsync(lut_out, d_lut, lut_b, cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(c, cudaMemcpyAsync(scale_out, base + 16, sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(c, cudaMemcpyAsync(lut_bias_out, base + 32, sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    return LUTAMM_OK;
}

int lutamm_unload_weights(lutamm_ctx* c, int layer_id) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    free_layer(*L);
    c->layers.erase(layer_id);
    return LUTAMM_OK;
}

int lutamm_amm(lutamm_ctx* c, int layer_id, const float* input, float* output, uint32_t n_tokens, uint32_t flags) {
    return amm_impl(c, layer_id, input, output, n_tokens, nullptr, nullptr, flags);
}

int lutamm_amm_debug(lutamm_ctx* c, int layer_id, const float* input, float* output, uint32_t n_tokens,
                     uint8_t* idx_out, int32_t* acc_out, uint32_t flags) {
    return amm_impl(c, layer_id, input, output, n_tokens, idx_out, acc_out, flags & ~LUTAMM_FLAG_ASYNC);
}

int lutamm_index_calculation(lutamm_ctx* c, int layer_id, const float* input, void* index_out, uint32_t M,
                             uint32_t format) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (M == 0) return LUTAMM_OK;
    if (!input || !index_out) return fail(c, LUTAMM_EINVAL, "null input or output");
    if (format != LUTAMM_INDEX_U8_ROWMAJOR && format != LUTAMM_INDEX_U16_TILED)
        return fail(c, LUTAMM_EINVAL, "unknown index format");
    if (format == LUTAMM_INDEX_U16_TILED) {
        if (!L->ip.n_stile_size || !L->ip.cb_mtile_size || M % L->ip.n_stile_size || L->CB % L->ip.cb_mtile_size)
            return fail(c, LUTAMM_EINVAL, "tiled index layout needs n % n_stile_size == 0 and num_codebook % cb_mtile_size == 0");
    }
    int r;
    const float* d_x = input;
    if (!is_device_ptr(input)) {
        const size_t in_bytes = (size_t)M * L->K * sizeof(float);
        if ((r = ensure(c, c->d_in, in_bytes))) return r;
        CU_TRY(c, cudaMemcpyAsync(c->d_in.p, input, in_bytes, cudaMemcpyHostToDevice, c->stream));
        d_x = static_cast<const float*>(c->d_in.p);
    }
    const size_t esz = format == LUTAMM_INDEX_U16_TILED ? 2 : 1;
    const size_t obytes = (size_t)M * L->CB * esz;
    void* d_o = index_out;
    const bool out_dev = is_device_ptr(index_out);
    if (!out_dev) {
        Buf& b = esz == 2 ? c->d_idx16 : c->d_idx;
        if ((r = ensure(c, b, obytes))) return r;
        d_o = b.p;
    }
    if ((r = run_ccs(c, *L, d_x, d_o, M, format))) return r;
    if (!out_dev) CU_TRY(c, cudaMemcpyAsync(index_out, d_o, obytes, cudaMemcpyDeviceToHost, c->stream));
    return check_dev_err(c);
}

int lutamm_pim_lut(lutamm_ctx* c, int layer_id, const uint8_t* index, float* output, uint32_t M, uint32_t flags) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (M == 0) return LUTAMM_OK;
    if (!index || !output) return fail(c, LUTAMM_EINVAL, "null index or output");
    int r;
    if ((flags & LUTAMM_FLAG_OUTPUT_TILED) && (r = check_tiled(c, *L, M))) return r;
    const bool in_dev = is_device_ptr(index), out_dev = is_device_ptr(output);
    if ((flags & LUTAMM_FLAG_ASYNC) && !(in_dev && out_dev))
        return fail(c, LUTAMM_EINVAL, "LUTAMM_FLAG_ASYNC needs device buffers");
    const uint8_t* d_i = index;
    if (!in_dev) {
        if ((r = ensure(c, c->d_idx, (size_t)M * L->CB))) return r;
        CU_TRY(c, cudaMemcpyAsync(c->d_idx.p, index, (size_t)M * L->CB, cudaMemcpyHostToDevice, c->stream));
        d_i = static_cast<const uint8_t*>(c->d_idx.p);
    }
    float* d_y = output;
    const size_t out_bytes = (size_t)M * L->N * sizeof(float);
    if (!out_dev) {
        if ((r = ensure(c, c->d_out, out_bytes))) return r;
        d_y = static_cast<float*>(c->d_out.p);
    }
    if ((r = run_lut(c, *L, d_i, d_y, nullptr, M, flags, L->plan))) return r;
    if (!out_dev) CU_TRY(c, cudaMemcpyAsync(output, d_y, out_bytes, cudaMemcpyDeviceToHost, c->stream));
    if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
    return check_dev_err(c);
}

int lutamm_set_plan(lutamm_ctx* c, int layer_id, const lutamm_plan* plan) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (!plan) return fail(c, LUTAMM_EINVAL, "null plan");
    if (plan->variant > LUTAMM_VARIANT_UMMA) return fail(c, LUTAMM_EINVAL, "unknown kernel variant");
    if (plan->gather_cfg >= gather_num_cfgs()) return fail(c, LUTAMM_EINVAL, "unknown gather tile configuration");
    if (plan->umma_operand > 2) return fail(c, LUTAMM_EINVAL, "umma_operand must be 0, 1 (shared memory) or 2 (tensor memory)");
    if (plan->umma_n_tile && plan->umma_operand && !umma_tile_ok(plan->umma_n_tile, plan->umma_operand == 2))
        return fail(c, LUTAMM_EINVAL, "umma_n_tile must be 0, 64, 128 or 256 with the one-hot operand in shared memory, "
                                      "0, 64, 128, 160 or 192 with it in tensor memory");
    if (plan->umma_sps != 0 && plan->umma_sps != 1 && plan->umma_sps != 2 && plan->umma_sps != 4)
        return fail(c, LUTAMM_EINVAL, "umma_sps must be 0, 1, 2 or 4");
    if (plan->umma_epilogue > LUTAMM_EPILOGUE_COPY_ENGINE) return fail(c, LUTAMM_EINVAL, "unknown umma_epilogue");
    if (plan->variant == LUTAMM_VARIANT_UMMA && !umma_supported(L->CB, L->CT, L->N))
        return fail(c, LUTAMM_EUNSUPPORTED, "tcgen05 variant does not cover this shape");
    L->plan = *plan;
    return LUTAMM_OK;
}

int lutamm_set_activation(lutamm_ctx* c, int layer_id, uint32_t activation) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (activation > LUTAMM_ACT_GELU_TANH_F16) return fail(c, LUTAMM_EINVAL, "unknown activation");
    L->act = activation;
    return LUTAMM_OK;
}

int lutamm_get_plan(lutamm_ctx* c, int layer_id, lutamm_plan* plan) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (!plan) return fail(c, LUTAMM_EINVAL, "null plan");
    *plan = L->plan;
    return LUTAMM_OK;
}

int lutamm_tune(lutamm_ctx* c, int layer_id, uint32_t M, lutamm_plan* best_out) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (M == 0) return fail(c, LUTAMM_EINVAL, "cannot tune for zero tokens");
    // a shape tuned before on this kind of GPU (this process, or a cache file loaded into the context)
    const std::vector<uint32_t> key = {M, L->K, L->N, L->CB, L->CT, (uint32_t)c->sm_count};
    auto hit = c->plan_cache.find(key);
    if (hit != c->plan_cache.end()) {
        L->plan = hit->second;
        if (best_out) *best_out = hit->second;
        return LUTAMM_OK;
    }
    int r;
    // Inputs: zero activations give valid indices; the kernels' timing does not depend on values.
    if ((r = ensure(c, c->d_in, (size_t)M * L->K * sizeof(float)))) return r;
    if ((r = ensure(c, c->d_out, (size_t)M * L->N * sizeof(float)))) return r;
    if ((r = ensure(c, c->d_idx, (size_t)M * L->CB))) return r;
    CU_TRY(c, cudaMemsetAsync(c->d_in.p, 0, (size_t)M * L->K * sizeof(float), c->stream));

    // The search space: kernel variant; for the CUDA-core gather its tile configuration; for tcgen05 where
    // the one-hot operand lives, the tile width, the split of the codebook axis, the depth of the LUT ring
    // and the number of one-hot builder groups.  (What the reference's tuner enumerates instead - DPU grid,
    // micro-tile factors, load type, loop order, src/tuner/auto_tuner.cpp:368-549 - has no meaning here.)
    std::vector<lutamm_plan> cands;
    for (uint32_t cfg = 0; cfg < gather_num_cfgs(); ++cfg) {
        lutamm_plan p{};
        p.variant = LUTAMM_VARIANT_GATHER;
        p.gather_cfg = cfg;
        cands.push_back(p);
    }
    if (umma_supported(L->CB, L->CT, L->N)) {
        const uint32_t slabs = (uint32_t)(((uint64_t)L->CB * L->CT + 127) / 128);
        struct Cand { uint32_t operand, n_tile, sps; };
        for (const Cand& cd : {Cand{1, 256, 1}, Cand{2, 192, 1}, Cand{2, 160, 1}, Cand{2, 128, 2}, Cand{2, 128, 1}, Cand{1, 128, 1}, Cand{2, 64, 1}}) {
            if (cd.n_tile > 128 && L->N < cd.n_tile) continue;
            const uint32_t tiles = ((M + 127) / 128) * ((L->N + cd.n_tile - 1) / cd.n_tile);
            if (cd.n_tile == 64 && tiles > 4u * (uint32_t)c->sm_count) continue;  // narrow tiles only pay on small problems
            std::vector<uint32_t> splits = {1};
            uint32_t s_fill = tiles < (uint32_t)c->sm_count ? (uint32_t)c->sm_count / tiles : 1;
            for (uint32_t s : {s_fill, s_fill * 2, s_fill / 2})
                if (s > 1 && s <= slabs / 4 && s <= 32 && std::find(splits.begin(), splits.end(), s) == splits.end()) splits.push_back(s);
            for (uint32_t s : splits) {
                lutamm_plan p{};
                p.variant = LUTAMM_VARIANT_UMMA;
                p.umma_n_tile = cd.n_tile;
                p.umma_split = s;
                p.umma_operand = cd.operand;
                p.umma_sps = cd.sps;
                cands.push_back(p);
                if (s == 1 || s == s_fill) {  // ring depth and builder groups around the likely winners only
                    lutamm_plan q = p;
                    q.umma_stages = 6;
                    cands.push_back(q);
                    q = p;
                    q.umma_groups = 2;
                    cands.push_back(q);
                }
            }
        }
    }
    cudaEvent_t e0 = c->ev[0], e1 = c->ev[1];
    const std::string saved_err = c->err;
    auto time_lut = [&](const lutamm_plan& p, float* ms) -> int {
        int rr;
        for (int w = 0; w < 2; ++w)
            if ((rr = run_lut(c, *L, static_cast<const uint8_t*>(c->d_idx.p), static_cast<float*>(c->d_out.p), nullptr, M, 0, p))) return rr;
        CU_TRY(c, cudaEventRecord(e0, c->stream));
        const int reps = 5;
        for (int i = 0; i < reps; ++i)
            if ((rr = run_lut(c, *L, static_cast<const uint8_t*>(c->d_idx.p), static_cast<float*>(c->d_out.p), nullptr, M, 0, p))) return rr;
        CU_TRY(c, cudaEventRecord(e1, c->stream));
        if ((rr = check_dev_err(c))) return rr;
        float t = 0;
        CU_TRY(c, cudaEventElapsedTime(&t, e0, e1));
        *ms = t / reps;
        return LUTAMM_OK;
    };
    if ((r = run_ccs(c, *L, static_cast<const float*>(c->d_in.p), c->d_idx.p, M, LUTAMM_INDEX_U8_ROWMAJOR))) return r;
    // the layer's plan is replaced only when the whole search has succeeded
    lutamm_plan best = L->plan;
    float best_ms = 1e30f;
    for (const lutamm_plan& p : cands) {
        float ms = 0;
        r = time_lut(p, &ms);
        if (r == LUTAMM_EDEVICE) return r;
        if (r) { c->err = saved_err; continue; }  // a candidate the shape does not admit: not an error of the call
        if (ms < best_ms) { best_ms = ms; best = p; }
    }
    if (best_ms >= 1e30f) return fail(c, LUTAMM_EUNSUPPORTED, "no kernel candidate could run this shape");
    // search granularity of step 1
    float best_ccs = 1e30f;
    uint32_t best_tok = 0;
    for (uint32_t tok : {0u, 4u, 8u, 16u, 32u, 64u}) {
        for (int w = 0; w < 2; ++w)
            if ((r = run_ccs(c, *L, static_cast<const float*>(c->d_in.p), c->d_idx.p, M, LUTAMM_INDEX_U8_ROWMAJOR, (int)tok))) return r;
        CU_TRY(c, cudaEventRecord(e0, c->stream));
        for (int i = 0; i < 5; ++i)
            if ((r = run_ccs(c, *L, static_cast<const float*>(c->d_in.p), c->d_idx.p, M, LUTAMM_INDEX_U8_ROWMAJOR, (int)tok))) return r;
        CU_TRY(c, cudaEventRecord(e1, c->stream));
        CU_TRY(c, cudaStreamSynchronize(c->stream));
        float t = 0;
        CU_TRY(c, cudaEventElapsedTime(&t, e0, e1));
        if (t < best_ccs) { best_ccs = t; best_tok = tok; }
    }
    best.ccs_tokens = best_tok;
    L->plan = best;
    c->plan_cache[key] = best;
    if (best_out) *best_out = best;
    return LUTAMM_OK;
}

// Plan cache as a text file: one line per shape, "n K N CB CT SMs : variant ccs_tokens gather_cfg n_tile split
// stages groups operand sps".  A plan only applies to the GPU it was measured on, hence the SM count in the key.
int lutamm_plan_cache_save(lutamm_ctx* c, const char* path) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!path) return fail(c, LUTAMM_EINVAL, "null path");
    FILE* f = std::fopen(path, "w");
    if (!f) return fail(c, LUTAMM_EINVAL, std::string("cannot write ") + path);
    std::fprintf(f, "# lutamm plan cache: n K N CB CT SMs : variant ccs_tokens gather_cfg n_tile split stages groups operand sps\n");
    for (const auto& kv : c->plan_cache) {
        const lutamm_plan& p = kv.second;
        std::fprintf(f, "%u %u %u %u %u %u : %u %u %u %u %u %u %u %u %u\n", kv.first[0], kv.first[1], kv.first[2], kv.first[3], kv.first[4],
                     kv.first[5], p.variant, p.ccs_tokens, p.gather_cfg, p.umma_n_tile, p.umma_split, p.umma_stages, p.umma_groups,
                     p.umma_operand, p.umma_sps);
    }
    std::fclose(f);
    return LUTAMM_OK;
}

int lutamm_plan_cache_load(lutamm_ctx* c, const char* path) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!path) return fail(c, LUTAMM_EINVAL, "null path");
    FILE* f = std::fopen(path, "r");
    if (!f) return fail(c, LUTAMM_EINVAL, std::string("cannot read ") + path);
    char line[512];
    while (std::fgets(line, sizeof line, f)) {
        if (line[0] == '#' || line[0] == '\n') continue;
        unsigned k[6], v[9];
        if (std::sscanf(line, "%u %u %u %u %u %u : %u %u %u %u %u %u %u %u %u", &k[0], &k[1], &k[2], &k[3], &k[4], &k[5], &v[0], &v[1], &v[2],
                        &v[3], &v[4], &v[5], &v[6], &v[7], &v[8]) != 15) {
            std::fclose(f);
            return fail(c, LUTAMM_EINVAL, std::string("malformed plan cache line in ") + path);
        }
        lutamm_plan p{};
        p.variant = v[0]; p.ccs_tokens = v[1]; p.gather_cfg = v[2]; p.umma_n_tile = v[3]; p.umma_split = v[4];
        p.umma_stages = v[5]; p.umma_groups = v[6]; p.umma_operand = v[7]; p.umma_sps = v[8];
        if (p.variant > LUTAMM_VARIANT_UMMA || p.gather_cfg >= gather_num_cfgs() || p.umma_operand > 2) continue;  // not a plan of this build
        c->plan_cache[{k[0], k[1], k[2], k[3], k[4], k[5]}] = p;
    }
    std::fclose(f);
    return LUTAMM_OK;
}

int lutamm_enable_timing(lutamm_ctx* c, int on) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    c->timing = on != 0;
    c->last_valid = false;
    return LUTAMM_OK;
}

int lutamm_get_timings(lutamm_ctx* c, lutamm_timings* out) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!out) return fail(c, LUTAMM_EINVAL, "null out pointer");
    if (!c->last_valid) return fail(c, LUTAMM_EINVAL, "no timed call yet (lutamm_enable_timing, then a synchronous call)");
    *out = c->last;
    return LUTAMM_OK;
}


// ---- sharded forms -------------------------------------------------------------------------------
int lutamm_shard_unique_id(char* id) {
    if (!id) return fail(nullptr, LUTAMM_EINVAL, "null id buffer");
    const NcclApi& n = nccl_api();
    if (!n.ok) return fail(nullptr, LUTAMM_EUNSUPPORTED, n.why ? n.why : "NCCL unavailable");
    NcclUniqueId u;
    const int rc = n.get_unique_id(&u);
    if (rc != kNcclSuccess) return fail(nullptr, LUTAMM_ECUDA, std::string("ncclGetUniqueId: ") + n.get_error_string(rc));
    std::memcpy(id, u.internal, sizeof u.internal);
    return LUTAMM_OK;
}

int lutamm_shard_init(lutamm_ctx* c, int rank, int world, const char* id) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!id || world < 1 || rank < 0 || rank >= world) return fail(c, LUTAMM_EINVAL, "bad rank / world size / id");
    const NcclApi& n = nccl_api();
    if (!n.ok) return fail(c, LUTAMM_EUNSUPPORTED, n.why ? n.why : "NCCL unavailable");
    DeviceGuard g(c->device);
    if (c->comm) { n.comm_destroy(c->comm); c->comm = nullptr; }
    NcclUniqueId u;
    std::memcpy(u.internal, id, sizeof u.internal);
    const int rc = n.comm_init_rank(&c->comm, world, u, rank);
    if (rc != kNcclSuccess) { c->comm = nullptr; return fail(c, LUTAMM_ECUDA, std::string("ncclCommInitRank: ") + n.get_error_string(rc)); }
    c->rank = rank;
    c->world = world;
    return LUTAMM_OK;
}

int lutamm_shard_finalize(lutamm_ctx* c) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    if (c->comm) {
        CU_TRY(c, cudaStreamSynchronize(c->stream));
        if (nccl_api().ok) nccl_api().comm_destroy(c->comm);
        c->comm = nullptr;
    }
    c->rank = 0;
    c->world = 1;
    return LUTAMM_OK;
}

// A small all-gather on the context's stream: a rank passes it only after every rank has reached it in its own
// stream order.  Orders the ranks' kernels around stores into one another's memory.
static int rank_barrier(lutamm_ctx* c) {
    if (c->world <= 1) return LUTAMM_OK;
    const NcclApi& n = nccl_api();
    int rc;
    if ((rc = ensure(c, c->d_sync, 4 * (size_t)c->world, true))) return rc;
    uint32_t* w = static_cast<uint32_t*>(c->d_sync.p);
    const int e = n.all_gather(w + c->rank, w, 4, kNcclUint8, c->comm, c->stream);
    if (e != kNcclSuccess) return fail(c, LUTAMM_ECUDA, std::string("ncclAllGather(barrier): ") + n.get_error_string(e));
    return LUTAMM_OK;
}

int lutamm_shard_alloc_gathered(lutamm_ctx* c, size_t bytes, void** out) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!out || !bytes) return fail(c, LUTAMM_EINVAL, "null out pointer or zero size");
    *out = nullptr;
    DeviceGuard g(c->device);
    const int G = c->world, r = c->rank;
    if (G > (int)kMaxPeers) return fail(c, LUTAMM_EUNSUPPORTED, "at most 8 ranks");
    if (G > 1 && !c->comm) return fail(c, LUTAMM_EINVAL, "lutamm_shard_init has not been called on this context");
    void* p = nullptr;
    cudaError_t ce = cudaMalloc(&p, bytes);
    if (ce != cudaSuccess) {
        p = nullptr;
        cudaGetLastError();
        if (G == 1) return fail(c, LUTAMM_ENOMEM, std::string("cudaMalloc(gathered): ") + cudaGetErrorString(ce));
    }
    std::vector<void*> peers((size_t)G, nullptr);
    peers[(size_t)r] = p;
    if (G > 1) {
        // every rank's CUDA IPC handle to every rank, with a word that says whether the rank has a buffer at all
        // (a rank whose allocation failed still takes part, so that all ranks leave together): one all-gather
        const NcclApi& n = nccl_api();
        struct Slot { cudaIpcMemHandle_t handle; uint32_t valid; uint32_t pad[3]; };
        static_assert(sizeof(Slot) % 16 == 0, "slot size");
        constexpr size_t H = sizeof(Slot);
        Slot mine{};
        std::vector<Slot> all((size_t)G);
        int rc = ensure(c, c->d_build, H * (size_t)G + 256);
        bool ok = rc == LUTAMM_OK;   // (a failure here or in the exchange itself is not agreed on: the group is unusable)
        unsigned char* st = static_cast<unsigned char*>(c->d_build.p);
        cudaError_t he = cudaSuccess;
        if (p && (he = cudaIpcGetMemHandle(&mine.handle, p)) == cudaSuccess) mine.valid = 1;
        if (ok && (ce = cudaMemcpyAsync(st + H * r, &mine, H, cudaMemcpyHostToDevice, c->stream)) != cudaSuccess) { ok = false; rc = fail(c, LUTAMM_ECUDA, cudaGetErrorString(ce)); }
        if (ok) {
            const int e = n.all_gather(st + H * r, st, H, kNcclUint8, c->comm, c->stream);
            if (e != kNcclSuccess) { ok = false; rc = fail(c, LUTAMM_ECUDA, std::string("ncclAllGather(handles): ") + n.get_error_string(e)); }
        }
        if (ok && ((ce = cudaMemcpyAsync(all.data(), st, H * G, cudaMemcpyDeviceToHost, c->stream)) != cudaSuccess ||
                   (ce = cudaStreamSynchronize(c->stream)) != cudaSuccess)) { ok = false; rc = fail(c, LUTAMM_ECUDA, cudaGetErrorString(ce)); }
        for (int q = 0; ok && q < G; ++q)
            if (!all[(size_t)q].valid) {
                ok = false;
                rc = q == r ? fail(c, p ? LUTAMM_ECUDA : LUTAMM_ENOMEM, p ? std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(he)
                                                                          : std::string("cudaMalloc(gathered) failed on this rank"))
                            : fail(c, LUTAMM_ENOMEM, "rank " + std::to_string(q) + " could not allocate its gathered buffer");
            }
        for (int q = 0; ok && q < G; ++q) {
            if (q == r) continue;
            if ((ce = cudaIpcOpenMemHandle(&peers[(size_t)q], all[(size_t)q].handle, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess) {
                ok = false;
                rc = fail(c, LUTAMM_ECUDA, std::string("cudaIpcOpenMemHandle (is peer access between the GPUs available?): ") + cudaGetErrorString(ce));
            }
        }
        if (!ok) {
            for (int q = 0; q < G; ++q)
                if (q != r && peers[(size_t)q]) cudaIpcCloseMemHandle(peers[(size_t)q]);
            if (p) cudaFree(p);
            return rc;
        }
    }
    c->peer_bufs[p] = peers;
    *out = p;
    return LUTAMM_OK;
}

int lutamm_shard_free_gathered(lutamm_ctx* c, void* ptr) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    auto it = c->peer_bufs.find(ptr);
    if (it == c->peer_bufs.end()) return fail(c, LUTAMM_EINVAL, "not a buffer from lutamm_shard_alloc_gathered");
    int rc = rank_barrier(c);  // nobody stores into anybody's buffer any more
    if (rc) return rc;
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    for (size_t q = 0; q < it->second.size(); ++q)
        if ((int)q != c->rank && it->second[q]) cudaIpcCloseMemHandle(it->second[q]);
    if ((rc = rank_barrier(c))) return rc;   // every rank has unmapped before anybody frees
    CU_TRY(c, cudaStreamSynchronize(c->stream));
    cudaFree(ptr);
    c->peer_bufs.erase(it);
    return LUTAMM_OK;
}

int lutamm_amm_column_sharded(lutamm_ctx* c, int layer_id, const float* input, float* gathered, uint32_t M,
                              uint32_t search_mode, uint32_t flags) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (M == 0) return LUTAMM_OK;
    if (!input || !gathered) return fail(c, LUTAMM_EINVAL, "null input or output");
    if (!is_device_ptr(input) || !is_device_ptr(gathered)) return fail(c, LUTAMM_EINVAL, "the sharded entry points take device buffers");
    if (reinterpret_cast<uintptr_t>(gathered) & 15u) return fail(c, LUTAMM_EINVAL, "device output must be 16-byte aligned");
    if (search_mode != LUTAMM_SHARD_SEARCH_REPLICATED && search_mode != LUTAMM_SHARD_SEARCH_SPLIT)
        return fail(c, LUTAMM_EINVAL, "unknown search mode");
    if (flags & LUTAMM_FLAG_OUTPUT_TILED) return fail(c, LUTAMM_EINVAL, "the gathered buffer already is the reference's tiled layout with lut_parallelism = world size");
    const uint32_t G = (uint32_t)c->world, r = (uint32_t)c->rank;
    if (G > 1 && !c->comm) return fail(c, LUTAMM_EINVAL, "lutamm_shard_init has not been called on this context");
    const NcclApi& n = nccl_api();
    int rc;
    if ((rc = ensure(c, c->d_idx, (size_t)M * L->CB))) return rc;
    uint8_t* d_idx = static_cast<uint8_t*>(c->d_idx.p);
    if (search_mode == LUTAMM_SHARD_SEARCH_SPLIT && G > 1 && M % G == 0) {
        // each rank searches its M / G tokens, the uint8 indices are all-gathered in place: M*CB bytes
        // on the wire instead of G times the search
        const uint32_t m_loc = M / G;
        if ((rc = run_ccs(c, *L, input + (size_t)r * m_loc * L->K, d_idx + (size_t)r * m_loc * L->CB, m_loc, LUTAMM_INDEX_U8_ROWMAJOR))) return rc;
        const int e = n.all_gather(d_idx + (size_t)r * m_loc * L->CB, d_idx, (size_t)m_loc * L->CB, kNcclUint8, c->comm, c->stream);
        if (e != kNcclSuccess) return fail(c, LUTAMM_ECUDA, std::string("ncclAllGather(indices): ") + n.get_error_string(e));
    } else {
        if ((rc = run_ccs(c, *L, input, d_idx, M, LUTAMM_INDEX_U8_ROWMAJOR))) return rc;
    }
    const size_t slab = (size_t)M * L->N;
    if ((flags & LUTAMM_FLAG_PEER_STORE) && G > 1) {
        // The exchange fused into the kernel: the epilogue stores every finished tile of this rank's slab into
        // block r of EVERY rank's gathered buffer (plain stores over NVLink to memory mapped by CUDA IPC), so the
        // transfer overlaps the contraction tile by tile and no all-gather follows.  A rank may only start storing
        // once every rank is done with the buffer's previous contents, and may only read once every rank's kernel
        // has finished: one small all-gather before and one after.
        auto pb = c->peer_bufs.find(gathered);
        if (pb == c->peer_bufs.end()) return fail(c, LUTAMM_EINVAL, "LUTAMM_FLAG_PEER_STORE needs a buffer from lutamm_shard_alloc_gathered");
        float* peer_out[kMaxPeers] = {};
        for (uint32_t q = 0; q < G; ++q) peer_out[q] = static_cast<float*>(pb->second[q]) + (size_t)r * slab;
        if ((rc = rank_barrier(c))) return rc;
        rc = run_lut(c, *L, d_idx, gathered + (size_t)r * slab, nullptr, M, 0, L->plan, peer_out, G);
        if (rc == LUTAMM_OK) {
            if ((rc = rank_barrier(c))) return rc;
            if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
            return check_dev_err(c);
        }
        if (rc != LUTAMM_EUNSUPPORTED) return rc;
        ++c->unfused_exchanges;  // this plan has no fused form: the plain kernel and an all-gather, below
    }
    // this rank's [M][N_loc] slab straight into block r of the gathered buffer, then the blocks in place
    if ((rc = run_lut(c, *L, d_idx, gathered + (size_t)r * slab, nullptr, M, 0, L->plan))) return rc;
    if (G > 1) {
        const int e = n.all_gather(gathered + (size_t)r * slab, gathered, slab, kNcclFloat32, c->comm, c->stream);
        if (e != kNcclSuccess) return fail(c, LUTAMM_ECUDA, std::string("ncclAllGather(output slabs): ") + n.get_error_string(e));
    }
    if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
    return check_dev_err(c);
}

int lutamm_amm_token_sharded(lutamm_ctx* c, int layer_id, const float* input_rows, float* output, uint32_t M_total,
                             uint32_t gather, uint32_t flags) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    Layer* L = find_layer(c, layer_id);
    if (!L) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for layer " + std::to_string(layer_id));
    if (M_total == 0) return LUTAMM_OK;
    if (!input_rows || !output) return fail(c, LUTAMM_EINVAL, "null input or output");
    if (!is_device_ptr(input_rows) || !is_device_ptr(output)) return fail(c, LUTAMM_EINVAL, "the sharded entry points take device buffers");
    if (flags & LUTAMM_FLAG_OUTPUT_TILED) return fail(c, LUTAMM_EINVAL, "tiled output is not offered by the token-sharded call");
    const uint32_t G = (uint32_t)c->world, r = (uint32_t)c->rank;
    // near-equal contiguous row blocks: the first n % G ranks own one row more (an all-gather needs equal blocks)
    const uint32_t base = M_total / G, extra = M_total % G;
    if (extra && gather) return fail(c, LUTAMM_EINVAL, "gathering the rows needs n_tokens to be a multiple of the world size");
    if (G > 1 && gather && !c->comm) return fail(c, LUTAMM_EINVAL, "lutamm_shard_init has not been called on this context");
    const uint32_t m_loc = base + (r < extra ? 1u : 0u);
    if (m_loc == 0) return LUTAMM_OK;  // fewer tokens than ranks: nothing for this one
    int rc;
    if ((rc = ensure(c, c->d_idx, (size_t)m_loc * L->CB))) return rc;
    float* mine = gather ? output + (size_t)r * m_loc * L->N : output;
    if (reinterpret_cast<uintptr_t>(mine) & 15u) return fail(c, LUTAMM_EINVAL, "device output must be 16-byte aligned");
    if ((rc = run_ccs(c, *L, input_rows, c->d_idx.p, m_loc, LUTAMM_INDEX_U8_ROWMAJOR))) return rc;
    if (gather && G > 1 && (flags & LUTAMM_FLAG_PEER_STORE)) {
        // the row blocks exchanged by the kernel's own stores (see lutamm_amm_column_sharded)
        auto pb = c->peer_bufs.find(output);
        if (pb == c->peer_bufs.end()) return fail(c, LUTAMM_EINVAL, "LUTAMM_FLAG_PEER_STORE needs a buffer from lutamm_shard_alloc_gathered");
        float* peer_out[kMaxPeers] = {};
        for (uint32_t q = 0; q < G; ++q) peer_out[q] = static_cast<float*>(pb->second[q]) + (size_t)r * m_loc * L->N;
        if ((rc = rank_barrier(c))) return rc;
        rc = run_lut(c, *L, static_cast<const uint8_t*>(c->d_idx.p), mine, nullptr, m_loc, 0, L->plan, peer_out, G);
        if (rc == LUTAMM_OK) {
            if ((rc = rank_barrier(c))) return rc;
            if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
            return check_dev_err(c);
        }
        if (rc != LUTAMM_EUNSUPPORTED) return rc;
        ++c->unfused_exchanges;
    }
    if ((rc = run_lut(c, *L, static_cast<const uint8_t*>(c->d_idx.p), mine, nullptr, m_loc, 0, L->plan))) return rc;
    if (gather && G > 1) {
        const NcclApi& n = nccl_api();
        const int e = n.all_gather(mine, output, (size_t)m_loc * L->N, kNcclFloat32, c->comm, c->stream);
        if (e != kNcclSuccess) return fail(c, LUTAMM_ECUDA, std::string("ncclAllGather(rows): ") + n.get_error_string(e));
    }
    if (flags & LUTAMM_FLAG_ASYNC) return LUTAMM_OK;
    return check_dev_err(c);
}

int lutamm_tune_sharding(lutamm_ctx* c, int layer_all, int layer_cols, uint32_t M, uint32_t reps, lutamm_sharding_report* rep) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    if (!rep) return fail(c, LUTAMM_EINVAL, "null report");
    DeviceGuard g(c->device);
    const uint32_t G = (uint32_t)c->world;
    if (G > 1 && !c->comm) return fail(c, LUTAMM_EINVAL, "lutamm_shard_init has not been called on this context");
    if (M == 0 || M % G) return fail(c, LUTAMM_EINVAL, "n_tokens_total must be a positive multiple of the world size");
    if (reps == 0) reps = 3;
    Layer* LA = layer_all >= 0 ? find_layer(c, layer_all) : nullptr;
    Layer* LC = layer_cols >= 0 ? find_layer(c, layer_cols) : nullptr;
    if ((layer_all >= 0 && !LA) || (layer_cols >= 0 && !LC)) return fail(c, LUTAMM_ENOLAYER, "no weights loaded for one of the two layers");
    if (!LA && !LC) return fail(c, LUTAMM_EINVAL, "no candidate: both layers are negative");
    if (LA && LC && (LA->K != LC->K || LA->N != (size_t)LC->N * G))
        return fail(c, LUTAMM_EINVAL, "the column layer must hold N / world-size columns of the same operator");
    const uint32_t K = LA ? LA->K : LC->K;
    const size_t n_out = (size_t)M * (LA ? LA->N : (size_t)LC->N * G);
    rep->world = G;
    for (float& v : rep->ms) v = -1.f;

    // one collective allocation for both operands: the gathered output, then the input rows behind it (when a
    // rank cannot allocate, every rank learns it there and all leave together)
    float* d_x = nullptr;
    void* d_out = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = LUTAMM_OK;
    auto cleanup = [&]() {
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
        if (d_out) lutamm_shard_free_gathered(c, d_out);
    };
    if ((rc = lutamm_shard_alloc_gathered(c, (n_out + (size_t)M * K) * sizeof(float), &d_out))) return rc;
    d_x = static_cast<float*>(d_out) + n_out;
    if (cudaMemsetAsync(d_x, 0, (size_t)M * K * sizeof(float), c->stream) != cudaSuccess || cudaEventCreate(&e0) != cudaSuccess ||
        cudaEventCreate(&e1) != cudaSuccess) {
        cleanup();
        return fail(c, LUTAMM_ECUDA, "could not set up the timing run");
    }

    float* out = static_cast<float*>(d_out);
    const uint32_t m_loc = M / G;
    auto call = [&](uint32_t mode) -> int {
        const float* rows = d_x + (size_t)c->rank * m_loc * K;
        switch (mode) {
            case LUTAMM_SHARDING_TOKENS_LOCAL:    return lutamm_amm_token_sharded(c, layer_all, rows, out, M, 0, LUTAMM_FLAG_ASYNC);
            case LUTAMM_SHARDING_TOKENS_GATHERED: return lutamm_amm_token_sharded(c, layer_all, rows, out, M, 1, LUTAMM_FLAG_ASYNC);
            case LUTAMM_SHARDING_TOKENS_FUSED:    return lutamm_amm_token_sharded(c, layer_all, rows, out, M, 1, LUTAMM_FLAG_ASYNC | LUTAMM_FLAG_PEER_STORE);
            case LUTAMM_SHARDING_COLUMNS:         return lutamm_amm_column_sharded(c, layer_cols, d_x, out, M, LUTAMM_SHARD_SEARCH_REPLICATED, LUTAMM_FLAG_ASYNC);
            case LUTAMM_SHARDING_COLUMNS_SPLIT:   return lutamm_amm_column_sharded(c, layer_cols, d_x, out, M, LUTAMM_SHARD_SEARCH_SPLIT, LUTAMM_FLAG_ASYNC);
            default:                              return lutamm_amm_column_sharded(c, layer_cols, d_x, out, M, LUTAMM_SHARD_SEARCH_SPLIT, LUTAMM_FLAG_ASYNC | LUTAMM_FLAG_PEER_STORE);
        }
    };
    float mine[LUTAMM_SHARDING_MODES];
    for (uint32_t mode = 0; mode < LUTAMM_SHARDING_MODES; ++mode) {
        mine[mode] = -1.f;
        const bool tokens = mode <= LUTAMM_SHARDING_TOKENS_FUSED;
        if (tokens ? !LA : !LC) continue;
        if (G == 1 && (mode == LUTAMM_SHARDING_TOKENS_FUSED || mode == LUTAMM_SHARDING_COLUMNS_FUSED)) continue;  // nothing to fuse
        const uint64_t unfused_before = c->unfused_exchanges;
        for (int w = 0; w < 2 && rc == LUTAMM_OK; ++w) rc = call(mode);
        if (rc == LUTAMM_OK) rc = rank_barrier(c);
        if (rc != LUTAMM_OK) break;
        // a plan without a fused kernel ran as kernel + all-gather (on every rank alike: same plan, same shape):
        // that is the candidate before this one, not a new one
        if (c->unfused_exchanges != unfused_before) continue;
        cudaEventRecord(e0, c->stream);
        for (uint32_t i = 0; i < reps && rc == LUTAMM_OK; ++i) rc = call(mode);
        cudaEventRecord(e1, c->stream);
        if (rc != LUTAMM_OK) break;
        if (cudaStreamSynchronize(c->stream) != cudaSuccess) { rc = fail(c, LUTAMM_ECUDA, "synchronize failed while timing"); break; }
        if ((rc = check_dev_err(c))) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        mine[mode] = ms / (float)reps;
    }
    if (rc != LUTAMM_OK) { cleanup(); return rc; }
    // the slowest rank's time per candidate
    std::vector<float> all((size_t)G * LUTAMM_SHARDING_MODES, -1.f);
    if (G > 1) {
        constexpr size_t B = sizeof mine;
        if ((rc = ensure(c, c->d_build, B * G + 256))) { cleanup(); return rc; }
        unsigned char* st = static_cast<unsigned char*>(c->d_build.p);
        cudaMemcpyAsync(st + B * c->rank, mine, B, cudaMemcpyHostToDevice, c->stream);
        const int e = nccl_api().all_gather(st + B * c->rank, st, B, kNcclUint8, c->comm, c->stream);
        if (e != kNcclSuccess) { cleanup(); return fail(c, LUTAMM_ECUDA, std::string("ncclAllGather(timings): ") + nccl_api().get_error_string(e)); }
        if (cudaMemcpyAsync(all.data(), st, B * G, cudaMemcpyDeviceToHost, c->stream) != cudaSuccess || cudaStreamSynchronize(c->stream) != cudaSuccess) {
            cleanup();
            return fail(c, LUTAMM_ECUDA, "timing read-back failed");
        }
    } else {
        std::memcpy(all.data(), mine, sizeof mine);
    }
    float best_ms = -1.f;
    rep->best = LUTAMM_SHARDING_TOKENS_GATHERED;
    for (uint32_t mode = 0; mode < LUTAMM_SHARDING_MODES; ++mode) {
        float worst = 0.f;
        for (uint32_t q = 0; q < G; ++q) {
            const float v = all[(size_t)q * LUTAMM_SHARDING_MODES + mode];
            if (v < 0.f) { worst = -1.f; break; }
            worst = std::max(worst, v);
        }
        rep->ms[mode] = worst;
        if (mode != LUTAMM_SHARDING_TOKENS_LOCAL && worst >= 0.f && (best_ms < 0.f || worst < best_ms)) { best_ms = worst; rep->best = mode; }
    }
    cleanup();
    return LUTAMM_OK;
}

int lutamm_measure_int8_peak(lutamm_ctx* c, double* tops, double* mac_per_clk_sm, double* sm_mhz) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    const uint32_t n_tile = 256, slabs = 8192, grid = (uint32_t)c->sm_count;
    int r;
    if ((r = ensure(c, c->d_build, 256))) return r;
    unsigned long long* d_cycles = static_cast<unsigned long long*>(c->d_build.p);
    const char* why = nullptr;
    float best_ms = 1e30f;
    unsigned long long cycles = 0;
    for (int rep = 0; rep < 4; ++rep) {  // the first repetition warms up; the best of the rest counts
        CU_TRY(c, cudaEventRecord(c->ev[0], c->stream));
        cudaError_t e = launch_int8_peak(n_tile, slabs, grid, d_cycles, c->d_err, c->stream, &why);
        if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, why ? why : (std::string("int8 peak launch: ") + cudaGetErrorString(e)));
        ++c->launches;
        CU_TRY(c, cudaEventRecord(c->ev[1], c->stream));
        if ((r = check_dev_err(c))) return r;
        float ms = 0;
        CU_TRY(c, cudaEventElapsedTime(&ms, c->ev[0], c->ev[1]));
        if (rep > 0 && ms < best_ms) {
            best_ms = ms;
            CU_TRY(c, cudaMemcpy(&cycles, d_cycles, sizeof cycles, cudaMemcpyDeviceToHost));
        }
    }
    const double macs_per_cta = (double)slabs * 128.0 * n_tile * 128.0;
    if (tops) *tops = 2.0 * macs_per_cta * grid / (best_ms * 1e-3) / 1e12;
    if (mac_per_clk_sm) *mac_per_clk_sm = cycles ? macs_per_cta / (double)cycles : 0.0;
    // event time covers launch and tear-down too, so this slightly understates the clock
    if (sm_mhz) *sm_mhz = cycles ? (double)cycles / (best_ms * 1e-3) / 1e6 : 0.0;
    return LUTAMM_OK;
}

int lutamm_selftest_bounded_wait(lutamm_ctx* c, uint32_t polls) {
    if (!c) return fail(nullptr, LUTAMM_EINVAL, "null context");
    DeviceGuard g(c->device);
    if (polls == 0 || polls > (1u << 20)) return fail(c, LUTAMM_EINVAL, "polls must be in 1 .. 2^20");
    cudaError_t e = launch_stalled_wait(polls, c->d_err, c->stream);
    if (e != cudaSuccess) return fail(c, LUTAMM_ECUDA, std::string("self-test launch: ") + cudaGetErrorString(e));
    ++c->launches;
    return check_dev_err(c);   // LUTAMM_EDEVICE is the expected answer
}

uint64_t lutamm_launch_count(const lutamm_ctx* c) { return c ? c->launches : 0; }

}  // extern "C"
