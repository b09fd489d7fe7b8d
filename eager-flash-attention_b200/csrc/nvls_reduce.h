// Sum AllReduce of fp16 partial sums through an NVLink multicast object (NVSwitch reduces in the
// switch, fp32 accumulation, one rounding): the third way to do allreduce() of eager-flash-attention
// (run_drivers.cu:26-30) beside NCCL and the fused peer-memory kernel.
#pragma once

#include "runtime.h"

namespace efa {

// 1 when this path can run the problem on this machine; otherwise 0 and *why says what is in the way.
// Collective when it has to ask the devices (every rank gets the same answer).
int nvls_supported(efa_ctx* c, const efa_params& p, const char** why);

// Symmetric memory for S*d partial sums (room for fp32) and S*d fp16 results, bound to a multicast object over all
// ranks of the context. Collective; a no-op when the region in place is large enough.
int nvls_prepare(efa_ctx* c, const efa_params& p);

// Where the projection writes this rank's partial sums ([S][d] fp16, local memory), and where the reduced
// rows appear on every rank.
void* nvls_send_buf(efa_ctx* c);
void* nvls_result_buf(efa_ctx* c);
void* nvls_pull_send_buf(efa_ctx* c);      // [S][d] fp32, plain device memory mapped by every rank (EFA_REDUCE_PULL)

// Reduce elements [first, first + n) of the partial sums (fp32 when wire_f32, else fp16; the element index is the
// same either way) over all ranks into the same elements of the fp16 result buffer of EVERY rank. One kernel on `stream`; `slot` (< EFA_MAX_COMM) names the stream's barrier flags, so
// calls on different streams may overlap as long as they use different slots. Collective: every rank makes
// the same sequence of calls per slot.
// pull: the partial sums are the fp32 ones at nvls_pull_send_buf (EFA_REDUCE_PULL): every rank fetches its share of all ranks'
// partial sums over peer mappings, adds them itself and multicasts the result.
int nvls_allreduce(efa_ctx* c, int slot, size_t first, size_t n, bool wire_f32, bool pull, cudaStream_t stream);

// One file descriptor from rank 0 to every other rank of one host (Unix-domain socket, SCM_RIGHTS): rank 0 passes
// fd_root and gets it back in *fd_out, the others receive a descriptor of their own for the same open file.
// Host only. Returns 0 on this rank's success.
int share_fd(const efa_world& w, int fd_root, int* fd_out);

// Unmaps and unbinds (collective when the region exists). Called by efa_destroy_ctx.
void nvls_destroy(efa_ctx* c);

}  // namespace efa
