// Kernel arguments shared by the attention kernels.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace efa {

struct FaArgs {
    float*  O32;
    __half* O16;
    float*  O_part;
    float*  m_part;
    float*  l_part;
    int     part_rows;
    int     q_start, q_rows, S, H_local, nsplit, kv_len, causal;
    float   scale_log2e;
    int*    tile_counters;
    int     tile_rows;
    int*    status;
    int     band_blocks;    // two-tile kernel: 256-row blocks per band of the work order (0 or 1 = strict row order)
    int     counters_sys;   // the tile counters live in host memory: order the rows before the count at system scope
    const short* order_tab; // two-tile kernel, strict-order launches only: order_tab[k] = the 256-row block taken k-th
                            // (device memory, one entry per block); nullptr = first to last (or last to first, below)
    int     heavy_first;    // two-tile kernel: take the row blocks (or bands) from the last to the first; with a causal
                            // mask the last rows sweep the most keys, so the longest items start first
};

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Warp-specialised two-tile kernel (fa_fwd_ws_sm100.cu), d_h = 64 or 128.
// reserve_sms > 0: persistent grid that leaves that many SMs without an attention CTA.
// K and V maps for it have boxes of fa_ws_kv_box_rows() rows (its stage length); Q maps 128 rows.
int fa_ws_kv_box_rows();
int fa_ws_preload();    // loads the code of every instantiation of the two-tile kernel on the current device
int fa_forward_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaArgs& a,
                  int d_h, bool out_f16, int reserve_sms, cudaStream_t stream);

}  // namespace efa
