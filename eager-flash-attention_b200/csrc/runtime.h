// Host runtime of one rank: problem description, streams and communicators, scratch memory.
// Counterpart of attn_main.cu / attn_defs.cuh of eager-flash-attention for the fp16 data path.
#pragma once

#include <cuda_runtime.h>
#include <nccl.h>
#include <vector>

#include "../../include/efa_b200.h"

#define EFA_MAX_COMM 8   /* MAX_COMM, attn_defs.cuh:90 */

struct P2PState;   // peer-mapped staging of the fused reduction (p2p_reduce.cu)
struct NvlsState;  // symmetric memory bound to an NVLink multicast object (nvls_reduce.cu)

struct efa_ctx {
    efa_world    world;
    cudaStream_t compute_stream = nullptr;
    cudaStream_t proj_stream = nullptr;
    cudaStream_t comm_streams[EFA_MAX_COMM] = {};
    ncclComm_t   nccls[EFA_MAX_COMM] = {};
    int          ncomm = 0;

    // Scratch, grown on demand and reused across run_mode calls (freed by efa_destroy_ctx).
    void*  O_all = nullptr;     size_t O_all_bytes = 0;      // fp16 [S][d_local]
    void*  send_buf = nullptr;  size_t send_bytes = 0;       // fp16 [S][d]
    int*   counters = nullptr;  size_t counters_n = 0;
    float* ws_O = nullptr; float* ws_m = nullptr; float* ws_l = nullptr;
    size_t ws_O_n = 0, ws_ml_n = 0;
    std::vector<cudaEvent_t> events;                        // disable-timing events, one per tile + a few
    cudaEvent_t ev_t0 = nullptr, ev_t1 = nullptr, ev_t2 = nullptr, ev_t3 = nullptr;   // timing events
    std::vector<cudaEvent_t> trace_events;                  // timing events of the EFA_TRACE timeline (stream mode)

    // Device staging of efa_run_mode_host.
    void* h_Q = nullptr; void* h_K = nullptr; void* h_V = nullptr; void* h_W = nullptr; void* h_out = nullptr;
    size_t h_qkv_bytes = 0, h_w_bytes = 0, h_out_bytes = 0;

    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;   // copies of the pipelined host-buffer path
    cudaStream_t rescue_stream = nullptr;                      // carries nothing but the store that releases pending counter waits

    short* order_tab = nullptr; size_t order_tab_n = 0;        // device copy of the row-block order of the last mixed-order run
    std::vector<short> order_tab_host;

    P2PState* p2p = nullptr;
    NvlsState* nvls = nullptr;
    int nvls_ctas = 16;                                        // thread blocks of one multicast reduction (fixed per context)

    // Limit of every device-side wait on another kernel or another rank (tile counters, arrival flags, barrier
    // flags), and of the host's wait for a stream; efa_ctx_set_wait_limit_ms changes both.
    unsigned long long wait_limit_ns = 10000000000ull;         // 10 s
    double             host_wait_limit_ms = 120000.0;          // 120 s
};

namespace efa {

int world_barrier(const efa_world& w);
int world_max(const efa_world& w, double* v);

// Grow-only scratch helpers; return 0 on success.
int ensure_bytes(void** ptr, size_t* have, size_t want);
int ensure_events(efa_ctx* c, size_t n);
int ensure_trace_events(efa_ctx* c, size_t n);

// residual (optional, fp16 [S][d]): added to every reduced group of rows right after its reduction.
int run_mode_impl(efa_ctx* c, int mode, const efa_weights& w, void* output, const efa_params& p, efa_run_stats* stats,
                  const void* residual = nullptr);

// Stream mode on HOST buffers as a pipeline over row chunks (causal): the copy-in of chunk c+1, the attention /
// projection / reduction of chunk c and the copy-out of chunk c-1 overlap. `dev` holds the device staging of Q, K, V,
// W_O; `dev_out` the device output. host_out receives rows [out_row0, out_row0 + out_rows) of the result (nothing when
// out_rows == 0). Returns 0 and fills stats->wall_ms (max over ranks).
int run_stream_host_pipelined(efa_ctx* c, const uint16_t* Qh, const uint16_t* Kh, const uint16_t* Vh, const uint16_t* W_O,
                              uint16_t* host_out, int out_row0, int out_rows, const efa_weights& dev, void* dev_out,
                              const efa_params& p, efa_run_stats* stats);

}  // namespace efa
