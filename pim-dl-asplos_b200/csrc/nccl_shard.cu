// NCCL for the sharded forms of the operator (one process per GPU, the GPUs of one box).
//
// The reference spreads one AMM over an input_parallelism x lut_parallelism grid of DPUs
// (inference-engine/src/host/parser.cpp:41-42; LUT column slabs pim_lut_host.cpp:26-37, index slabs
// :109-117) and moves the slabs with host<->DPU transfers.  Here the two exchanges that sharding by
// output columns needs - the column slabs of the result, and optionally the uint8 indices when the
// search is split by tokens - are NCCL all-gathers over NVLink, issued on the context's stream between
// the kernels.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, which inside a PyTorch process is the copy
// torch already loaded), so the library keeps no link-time dependency on it and still loads on a
// machine without NCCL or without a GPU; the sharded entry points then report an error.
#include "nccl_shard.h"

#include <dlfcn.h>

#include <mutex>

namespace lutamm {

namespace {

NcclApi g_api;
std::once_flag g_once;

void resolve() {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        g_api.why = "libnccl.so.2 could not be loaded";
        return;
    }
    g_api.get_unique_id = reinterpret_cast<decltype(g_api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
    g_api.comm_init_rank = reinterpret_cast<decltype(g_api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
    g_api.comm_destroy = reinterpret_cast<decltype(g_api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
    g_api.all_gather = reinterpret_cast<decltype(g_api.all_gather)>(dlsym(h, "ncclAllGather"));
    g_api.get_error_string = reinterpret_cast<decltype(g_api.get_error_string)>(dlsym(h, "ncclGetErrorString"));
    g_api.get_version = reinterpret_cast<decltype(g_api.get_version)>(dlsym(h, "ncclGetVersion"));
    if (!g_api.get_unique_id || !g_api.comm_init_rank || !g_api.comm_destroy || !g_api.all_gather || !g_api.get_error_string) {
        g_api.why = "libnccl.so.2 lacks one of ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy / ncclAllGather";
        return;
    }
    g_api.ok = true;
}

}  // namespace

const NcclApi& nccl_api() {
    std::call_once(g_once, resolve);
    return g_api;
}

}  // namespace lutamm
