// Drop-in replacement for flash_attn_tc.cu of eager-flash-attention: the four functions that
// flash_attn_tc.cuh declares (flash_attn_tc.cuh:45-62), defined over the C ABI of libefa_b200.so.
//
// Use: compile this file in place of flash_attn_tc.cu, with the reference's own headers on the
// include path, and link libefa_b200.so. Nothing else of the reference changes: its drivers, tests and
// benchmark then launch the sm_100a tcgen05 kernels through the interface they already use.
//
// Behaviour kept: asynchronous on `stream`; rows relative to the launch and keys absolute; with
// split > 1 the partials go to `part` and O is untouched until the combine; one count per finished
// 64-row block per (head, split) is added to tile_counters[(row within launch) / tile_rows] once the
// rows are visible device-wide. Failures that the reference turns into an abort abort here too, after
// printing the library's message.
#include "flash_attn_tc.cuh"

#include "../../../include/efa_b200.h"

#include <cstdio>
#include <cstdlib>

namespace {

void must(int rc, const char* what)
{
    if (rc != 0) {
        std::fprintf(stderr, "%s: %s\n", what, efa_last_error());
        std::abort();
    }
}

efa_flash_params convert(const FlashAttnTCParams& p)
{
    efa_flash_params e;
    e.S = p.S; e.d_h = p.d_h; e.H_local = p.H_local; e.split = p.split; e.causal = p.causal; e.scale = p.scale;
    return e;
}

efa_flash_partials convert(const FlashAttnTCPartials& w)
{
    efa_flash_partials e;
    e.O_part = w.O_part; e.m_part = w.m_part; e.l_part = w.l_part; e.rows = w.rows;
    return e;
}

}  // namespace

void flash_attn_tc_forward(const half* Q, const half* K, const half* V, float* O, const FlashAttnTCPartials& part,
                           int q_start, int q_rows, const FlashAttnTCParams& p, cudaStream_t stream,
                           int* tile_counters, int tile_rows)
{
    const efa_flash_params ep = convert(p);
    const efa_flash_partials ew = convert(part);
    must(efa_flash_attn_tc_forward(Q, K, V, O, EFA_F32, &ew, q_start, q_rows, &ep, stream, tile_counters, tile_rows),
         "flash_attn_tc_forward");
}

void flash_attn_tc_combine(const FlashAttnTCPartials& part, float* O, int row0, int rows, const FlashAttnTCParams& p,
                           cudaStream_t stream)
{
    const efa_flash_params ep = convert(p);
    const efa_flash_partials ew = convert(part);
    must(efa_flash_attn_tc_combine(&ew, O, EFA_F32, row0, rows, &ep, stream), "flash_attn_tc_combine");
}

const char* flash_attn_tc_check_params(const FlashAttnTCParams& p, int q_rows)
{
    const efa_flash_params ep = convert(p);
    return efa_flash_attn_tc_check_params(&ep, q_rows);
}

void convert_f32_to_f16(const float* in, half* out, size_t n, cudaStream_t stream)
{
    must(efa_convert_f32_to_f16(in, out, n, stream), "convert_f32_to_f16");
}
