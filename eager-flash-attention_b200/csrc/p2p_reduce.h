// Reduction of the per-tile partial sums over peer-mapped memory (NVLink), fused behind the
// projection: the alternative to one NCCL AllReduce per tile (allreduce(), run_drivers.cu:26-30).
#pragma once

#include "runtime.h"

namespace efa {

// 1 when the fused path can run this problem; otherwise 0 and *why says what is in the way.
int p2p_supported(const efa_params& p, const char** why);
// Tile counters the attention kernel must signal into for the fused path (never reset: targets grow per run).
int* p2p_counters(efa_ctx* c);

// Exchange IPC handles of the staging buffers for this shape (collective; cached in the context).
int p2p_prepare(efa_ctx* c, const efa_params& p, void* output);
// Launch the persistent projection + reduction kernel of this run on the projection stream.
// O_all: fp16 [S][d_local].
int p2p_launch(efa_ctx* c, const efa_params& p, const efa_weights& w, const void* O_all, int* launches);
void p2p_destroy(efa_ctx* c);

}  // namespace efa
