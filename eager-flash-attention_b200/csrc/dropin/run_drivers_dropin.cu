// Drop-in replacement for the three functions of run_drivers.cuh of eager-flash-attention
// (run_drivers.cuh:19-26): mode_name, parse_mode and run_mode, with the tensor-core configurations of
// run_mode executed by this library's run modes (attention, tcgen05 projection, grouped AllReduce) instead
// of run_drivers.cu.
//
// Use: link this file instead of run_drivers.cu, together with flash_attn_tc_dropin.cu and libefa_b200.so.
// run_mode keeps its contract: collective over the ranks of the context, writes the reduced fp32 [S][d]
// result to `output` (attention-only modes leave it untouched) and returns the wall time in ms, maxed over
// ranks (run_drivers.cuh:22-26). The library computes with fp16 O and fp16 W_O, fp32 accumulation, and —
// through proj_f32 — fp32 partial sums, reduction and output, the types the caller expects. W_O is rounded
// to fp16 before every call (outside the timed region, like the reference's per-call allocations).
//
// Configurations of the scalar v1 kernel are not this library's business. A build that still wants them
// compiles the reference's run_drivers.cu with its three public names prefixed (-Drun_mode=ref_run_mode
// -Dmode_name=ref_mode_name -Dparse_mode=ref_parse_mode) and defines EFA_DROPIN_HAVE_REF_DRIVERS here, and
// they are forwarded; without it they abort with a message.
#include "run_drivers.cuh"

#include "../../../include/efa_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

#ifdef EFA_DROPIN_HAVE_REF_DRIVERS
double ref_run_mode(int mode, const Weights& w, float* output, const AttnParams& p, const RunCtx& c);
#endif

namespace {

[[noreturn]] void die(const char* what)
{
    std::fprintf(stderr, "run_drivers drop-in: %s: %s\n", what, efa_last_error());
    MPI_Abort(MPI_COMM_WORLD, 1);
    std::abort();
}

int cb_barrier(void* comm) { return MPI_Barrier(*static_cast<MPI_Comm*>(comm)) != MPI_SUCCESS; }
int cb_max(void* comm, double* v)
{
    double g = *v;
    const int rc = MPI_Allreduce(v, &g, 1, MPI_DOUBLE, MPI_MAX, *static_cast<MPI_Comm*>(comm));
    *v = g;
    return rc != MPI_SUCCESS;
}
int cb_bcast(void* comm, void* buf, size_t n, int root)
{
    return MPI_Bcast(buf, (int)n, MPI_BYTE, root, *static_cast<MPI_Comm*>(comm)) != MPI_SUCCESS;
}
int cb_gather(void* comm, const void* in, void* out, size_t n)
{
    return MPI_Allgather(in, (int)n, MPI_BYTE, out, (int)n, MPI_BYTE, *static_cast<MPI_Comm*>(comm)) != MPI_SUCCESS;
}

// One library context per process, created on first use with the caller's communicator count
// (RunCtx::ncomm) and kept until exit: the reference's contexts live as long as the program too.
struct Bridge {
    MPI_Comm comm;
    efa_ctx* ctx = nullptr;
    int      ncomm = 0;
    void*    w_half = nullptr;      // fp16 copy of W_O
    size_t   w_half_bytes = 0;
};
Bridge g_bridge;

efa_ctx* context_for(const RunCtx& c)
{
    if (g_bridge.ctx && g_bridge.ncomm == c.ncomm) return g_bridge.ctx;
    if (g_bridge.ctx) { efa_destroy_ctx(g_bridge.ctx); g_bridge.ctx = nullptr; }
    g_bridge.comm = c.comm;
    efa_world w;
    std::memset(&w, 0, sizeof(w));
    w.user = &g_bridge.comm;
    MPI_Comm_rank(c.comm, &w.rank);
    MPI_Comm_size(c.comm, &w.size);
    if (cudaGetDevice(&w.local_device) != cudaSuccess) die("cudaGetDevice");
    w.barrier = cb_barrier; w.allreduce_max_f64 = cb_max; w.bcast_bytes = cb_bcast; w.allgather_bytes = cb_gather;
    if (efa_make_ctx(&g_bridge.ctx, &w, c.ncomm, /*prioritize=*/1)) die("efa_make_ctx");
    g_bridge.ncomm = c.ncomm;
    return g_bridge.ctx;
}

}  // namespace

const char* mode_name(int mode) { return efa_mode_name(mode); }
int parse_mode(const char* s) { return efa_parse_mode(s); }

double run_mode(int mode, const Weights& w, float* output, const AttnParams& p, const RunCtx& c)
{
    if (p.kernel != KERNEL_TC) {
#ifdef EFA_DROPIN_HAVE_REF_DRIVERS
        return ref_run_mode(mode, w, output, p, c);
#else
        std::fprintf(stderr, "run_drivers drop-in: only the tensor-core kernel (--kernel tc) is provided\n");
        MPI_Abort(MPI_COMM_WORLD, 1);
        std::abort();
#endif
    }
    efa_ctx* ctx = context_for(c);

    efa_params ep;
    if (efa_make_params(&ep, p.S, p.d, p.H, p.tile, p.nbuf, p.split, p.causal, p.R)) die("efa_make_params");
    ep.skip_proj = p.skip_proj;
    ep.skip_comm = p.skip_comm;
    ep.proj_f32 = 1;                              // fp32 partial sums, reduction and output
    if (const char* why = efa_attn_check_params(&ep)) {
        std::fprintf(stderr, "run_drivers drop-in: %s\n", why);
        MPI_Abort(MPI_COMM_WORLD, 1);
    }

    // fp16 copy of this rank's W_O slice [d_local][d]
    const size_t n_w = (size_t)ep.d_local * ep.d;
    if (g_bridge.w_half_bytes < n_w * 2) {
        if (g_bridge.w_half) cudaFree(g_bridge.w_half);
        if (cudaMalloc(&g_bridge.w_half, n_w * 2) != cudaSuccess) die("cudaMalloc(W_O fp16)");
        g_bridge.w_half_bytes = n_w * 2;
    }
    if (efa_convert_f32_to_f16(w.W_O, g_bridge.w_half, n_w, nullptr)) die("efa_convert_f32_to_f16");
    if (cudaStreamSynchronize(nullptr) != cudaSuccess) die("cudaStreamSynchronize");

    efa_weights ew;
    ew.Qh = w.Qh; ew.Kh = w.Kh; ew.Vh = w.Vh; ew.W_O = g_bridge.w_half;
    efa_run_stats st;
    std::memset(&st, 0, sizeof(st));
    if (efa_run_mode(ctx, mode, &ew, output, &ep, &st)) die("efa_run_mode");
    return st.wall_ms;
}
