// Reduction of the per-tile partial sums over peer-mapped memory (NVLink), fused behind the
// projection: the alternative to one NCCL AllReduce per tile (allreduce(), run_drivers.cu:26-30).
#pragma once

#include "runtime.h"

namespace efa {

// Exchange IPC handles of the staging buffers for this shape (collective; cached in the context).
int p2p_prepare(efa_ctx* c, const efa_params& p, void* output);
// Enqueue projection + reduction of tile t on the projection stream.
int p2p_tile(efa_ctx* c, const efa_params& p, const efa_weights& w, const void* O_tile, int t, int* launches);
// Enqueue the final hand-shake that makes every rank's output complete.
int p2p_finish(efa_ctx* c, const efa_params& p);
void p2p_destroy(efa_ctx* c);

}  // namespace efa
