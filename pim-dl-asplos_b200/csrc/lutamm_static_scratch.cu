// lutamm_amm_static_scratch(): the AMM for callers that must not allocate device memory.
//
// Who that is.  Some hosts hand this library a GPU whose memory they have already carved
// up: an inference server that sizes its arenas at start-up and treats any later
// cudaMalloc as a bug (it synchronises the whole device and can fail once memory is
// fragmented), a latency-critical loop that may not block on the allocator, or an embedding
// application that gives a plug-in a fixed set of buffers and nothing else.  The regular
// entry points keep a grow-only scratch arena per context, so their first call at a new
// size allocates.  This one never does: not cudaMalloc/cudaFree, not a pooled or library
// allocator.
//
// How.  The only intermediate of the operator is the closest-centroid index buffer,
// uint8 [n_tokens][num_codebook], written by the search kernel and read by the
// gather-accumulate kernel.  Here it lives in a file-scope __device__ array of fixed size
// (plus one error word).  Every GPU that loads this library therefore holds
// LUTAMM_STATIC_SCRATCH_BYTES + 256 bytes of device memory from module load until the
// process exits, whether or not the entry point is ever called.
//
// Rules that follow from one shared array:
//   * n_tokens * num_codebook must not exceed LUTAMM_STATIC_SCRATCH_BYTES; larger problems
//     are rejected with LUTAMM_EINVAL (split the batch);
//   * the array keeps whatever the previous call left in it; the one word that has to
//     start at zero (the kernels' error flag) is cleared at the start of every call, and
//     the index region is fully rewritten by the search kernel before it is read;
//   * two calls that overlap on the GPU (different streams, different threads, different
//     contexts of one process on one device) race on the array.  Serialise them.
//
// Set-up.  A __device__ array's name is only a host-side handle; the device address comes
// from cudaGetSymbolAddress, per device, with that device current.  The first call on a
// device does this (and sets the kernels' shared-memory attribute); make that first call
// before any stream capture begins, because these set-up calls are not stream operations.
//
// No counterpart in the reference, whose amm_host() allocates (and leaks) its index buffer
// on every call (inference-engine/src/host/amm_host.cpp:19).
#include <mutex>
#include <string>

#include "../../include/lutamm.h"
#include "kernels.h"

namespace {

constexpr size_t kHeaderBytes = 256;  // error word, padded so the index region stays 256-byte aligned
static __device__ __align__(256) unsigned char g_static_scratch[kHeaderBytes + LUTAMM_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device
thread_local std::string g_err;

int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}

bool on_device(const void* p, int device) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) && at.device == device;
}

}  // namespace

extern "C" const char* lutamm_static_scratch_last_error(void) { return g_err.c_str(); }

extern "C" int lutamm_amm_static_scratch(int device, void* cuda_stream, const float* input, const float* centroid,
                                         const int8_t* lut, const float* bias, float* output,
                                         const lutamm_index_params* ip, const lutamm_lut_params* lp) {
    using namespace lutamm;
    if (!input || !centroid || !lut || !bias || !output || !ip || !lp) return fail(LUTAMM_EINVAL, "null argument");
    if (device < 0 || device >= kMaxDevices) return fail(LUTAMM_EINVAL, "device ordinal out of range");
    const uint32_t M = ip->n, K = ip->input_feature_len, CB = ip->num_codebook, CT = ip->num_centroid;
    const uint32_t N = lp->output_feature_len;
    if (!K || !CB || !CT || !N || K % CB) return fail(LUTAMM_EINVAL, "bad shape: need input_feature_len % num_codebook == 0 and positive sizes");
    if (ip->sub_vec_len && ip->sub_vec_len != K / CB)
        return fail(LUTAMM_EINVAL, "sub_vec_len != input_feature_len / num_codebook");
    if (lp->num_codebook != CB || lp->num_centroid != CT || lp->n != M)
        return fail(LUTAMM_EINVAL, "index and LUT parameter blocks disagree");
    if (CT > 256) return fail(LUTAMM_EINVAL, "num_centroid > 256 does not fit the uint8 index");
    if (N % 16) return fail(LUTAMM_EINVAL, "output_feature_len must be a multiple of 16");
    if (M == 0) return LUTAMM_OK;
    if ((uint64_t)M * CB > (uint64_t)LUTAMM_STATIC_SCRATCH_BYTES)
        return fail(LUTAMM_EINVAL, "n * num_codebook = " + std::to_string((uint64_t)M * CB) +
                                       " index bytes exceed the static scratch of " +
                                       std::to_string((uint64_t)LUTAMM_STATIC_SCRATCH_BYTES) +
                                       " bytes; split the batch or use lutamm_amm()");

    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(device) != cudaSuccess)
        return fail(LUTAMM_ECUDA, std::string("cannot select device: ") + cudaGetErrorString(cudaGetLastError()));
    struct Restore {
        int d;
        ~Restore() { if (d >= 0) cudaSetDevice(d); }
    } restore{prev};

    for (const void* p : {(const void*)input, (const void*)centroid, (const void*)lut, (const void*)bias, (const void*)output})
        if (!on_device(p, device))
            return fail(LUTAMM_EINVAL, "every buffer must be device memory of the selected GPU: this entry point stages nothing");
    if ((reinterpret_cast<uintptr_t>(output) & 15u) || (reinterpret_cast<uintptr_t>(input) & 3u))
        return fail(LUTAMM_EINVAL, "output must be 16-byte aligned, input 4-byte aligned");

    unsigned char* scratch;
    {
        // once per device, with that device current: the symbol's device address
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_scratch_ptr[device]) {
            void* p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p)
                return fail(LUTAMM_ECUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
            g_scratch_ptr[device] = static_cast<unsigned char*>(p);
        }
        scratch = g_scratch_ptr[device];
    }
    uint32_t* d_err = reinterpret_cast<uint32_t*>(scratch);
    uint8_t* d_idx = scratch + kHeaderBytes;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);

    // the one word that must start at zero
    cudaError_t e = cudaMemsetAsync(d_err, 0, sizeof(uint32_t), s);
    if (e != cudaSuccess) return fail(LUTAMM_ECUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));

    const char* why = nullptr;
    CcsArgs ca{};
    ca.x = input; ca.centroid = centroid; ca.idx_out = d_idx;
    ca.M = M; ca.K = K; ca.v = K / CB; ca.CB = CB; ca.CT = CT;
    ca.format = LUTAMM_INDEX_U8_ROWMAJOR;
    e = launch_ccs(ca, s, &why);
    if (e != cudaSuccess) return fail(LUTAMM_ECUDA, why ? why : (std::string("search launch: ") + cudaGetErrorString(e)));

    // The gather-accumulate kernel reads the LUT in its canonical layout through a tensor map
    // encoded on the host (no device memory involved) and the indices from the static array.
    const uint32_t cfg = 0;
    CUtensorMap map;
    e = gather_make_tmap(&map, lut, CB, CT, N, cfg, &why);
    if (e != cudaSuccess) return fail(LUTAMM_ECUDA, why ? why : cudaGetErrorString(e));
    LutArgs la{};
    la.idx = d_idx; la.bias = bias; la.out = output; la.acc_out = nullptr;
    la.M = M; la.CB = CB; la.CT = CT; la.N = N;
    la.scale = lp->scale; la.lut_bias = lp->bias;
    e = launch_gather(la, map, cfg, d_err, s, &why);
    if (e != cudaSuccess) return fail(LUTAMM_ECUDA, why ? why : (std::string("gather launch: ") + cudaGetErrorString(e)));

    // The error word comes back on the caller's stream, behind the kernels; the legacy default stream
    // (which would serialise against every blocking stream of the process) is not touched.
    uint32_t h_err = 0;
    e = cudaMemcpyAsync(&h_err, d_err, sizeof h_err, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return fail(LUTAMM_ECUDA, std::string("cudaMemcpyAsync(error word): ") + cudaGetErrorString(e));
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(LUTAMM_ECUDA, std::string("cudaStreamSynchronize: ") + cudaGetErrorString(e));
    if (h_err) return fail(LUTAMM_EDEVICE, "a kernel gave up on a bounded wait; output is not valid");
    return LUTAMM_OK;
}
