// NCCL entry points resolved at run time (dlopen of libnccl.so.2) instead of at link time, so the
// library has no load-time dependency on one particular NCCL: inside a Python process it shares
// the NCCL that torch already loaded, in the C++ programs it loads the system's.
#pragma once

#include <nccl.h>

namespace efa {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    const char*  (*GetErrorString)(ncclResult_t);
};

// nullptr (with the error recorded) when NCCL cannot be loaded.
const NcclApi* nccl_api();

}  // namespace efa
