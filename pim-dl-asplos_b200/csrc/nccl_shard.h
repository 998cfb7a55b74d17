// The handful of NCCL entry points the sharded operator uses, resolved with dlopen at first use.
// Types are restated (NCCL's public ABI: an opaque communicator pointer, a 128-byte unique id passed by
// value, int enums) so that building the library does not need nccl.h.
#pragma once
#include <cstddef>
#include <cuda_runtime.h>

namespace lutamm {

struct NcclUniqueId {
    char internal[128];
};
typedef struct ncclComm* NcclComm;
constexpr int kNcclSuccess = 0;
constexpr int kNcclUint8 = 1;    // ncclUint8
constexpr int kNcclFloat32 = 7;  // ncclFloat32

struct NcclApi {
    bool ok = false;
    const char* why = nullptr;
    int (*get_unique_id)(NcclUniqueId*) = nullptr;
    int (*comm_init_rank)(NcclComm*, int nranks, NcclUniqueId id, int rank) = nullptr;
    int (*comm_destroy)(NcclComm) = nullptr;
    int (*all_gather)(const void* send, void* recv, size_t sendcount, int datatype, NcclComm, cudaStream_t) = nullptr;
    const char* (*get_error_string)(int) = nullptr;
    int (*get_version)(int*) = nullptr;
};

const NcclApi& nccl_api();

}  // namespace lutamm
