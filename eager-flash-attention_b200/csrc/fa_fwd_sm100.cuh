// Internal C++ interface of the attention kernels (the C ABI in efa_b200.h forwards to these).
#pragma once

#include <cuda_runtime.h>
#include "../../include/efa_b200.h"

namespace efa {

const char* fa_check_params(const efa_flash_params& p, int q_rows);

int fa_forward(const void* Q, const void* K, const void* V, void* O, int o_dtype,
               const efa_flash_partials* part, int q_start, int q_rows,
               const efa_flash_params& p, cudaStream_t stream, int* tile_counters, int tile_rows,
               int reserve_sms = 0,    // > 0 (d_h 64/128 only): persistent grid that leaves that many SMs free
               int band_rows = 0,      // d_h 64/128 with counters: rows may complete in bands of this many rows
                                       // (better K/V reuse in L2); 0 = strict row order. Without counters the
                                       // order is free and whole heads are processed one after another.
               int heavy_first = -1,  // d_h 64/128: 1 = take the row blocks (or bands) from the last to the first, 0 = from
                                       // the first; -1 = last first exactly when there are no counters and the mask is causal
               const short* order_tab = nullptr);  // d_h 64/128, band_rows == 0: the order of the 256-row blocks (device memory)

// Split-KV attention + merge with the partials in a fixed device array (no allocation anywhere).
int fa_forward_noalloc(const void* Q, const void* K, const void* V, void* O, int o_dtype,
                       int q_start, int q_rows, const efa_flash_params& p, cudaStream_t stream);

// {code, block, site, 0} written by a kernel of fa_forward_noalloc whose bounded wait ran out; reset != 0 clears it.
int noalloc_status(int* out4, int reset);

int fa_combine(const efa_flash_partials& part, void* O, int o_dtype, int row0, int rows,
               const efa_flash_params& p, cudaStream_t stream);

int convert_f32_to_f16_dev(const float* in, void* out, size_t n, cudaStream_t stream);

// out[rows][d] = A[rows][d_local] * W[d_local][d]; fp16 in, fp32 accumulate, fp16 (EFA_F16) or fp32 (EFA_F32) out.
int project_f16(const void* A, const void* W, void* out, int rows, int d_local, int d, cudaStream_t stream,
                int out_dtype = EFA_F16);

}  // namespace efa
