// extern "C" surface of the library: argument checks, then the C++ implementation.
#include "fa_fwd_sm100.cuh"
#include "host_util.h"
#include "nvls_reduce.h"
#include "runtime.h"

#include <cuda_fp16.h>

#include <chrono>
#include <cstring>

#include <sys/mman.h>
#include <unistd.h>

using namespace efa;

extern "C" int efa_abi_version(void) { return EFA_ABI_VERSION; }
extern "C" const char* efa_last_error(void) { return last_error(); }

extern "C" int efa_flash_attn_tc_forward(const void* Q, const void* K, const void* V,
                                         void* O, int o_dtype, const efa_flash_partials* part,
                                         int q_start, int q_rows, const efa_flash_params* p, void* stream,
                                         int* tile_counters, int tile_rows)
{
    if (!Q || !K || !V || !p) { set_error("efa_flash_attn_tc_forward: null argument"); return 2; }
    return fa_forward(Q, K, V, O, o_dtype, part, q_start, q_rows, *p, (cudaStream_t)stream, tile_counters, tile_rows);
}

extern "C" int efa_flash_attn_tc_forward_noalloc(const void* Q, const void* K, const void* V,
                                                 void* O, int o_dtype, int q_start, int q_rows,
                                                 const efa_flash_params* p, void* stream)
{
    if (!Q || !K || !V || !p) { set_error("efa_flash_attn_tc_forward_noalloc: null argument"); return 2; }
    return fa_forward_noalloc(Q, K, V, O, o_dtype, q_start, q_rows, *p, (cudaStream_t)stream);
}

extern "C" int efa_flash_attn_tc_noalloc_status(int* out4, int reset)
{
    if (!out4) { set_error("efa_flash_attn_tc_noalloc_status: null argument"); return 2; }
    return noalloc_status(out4, reset);
}

extern "C" int efa_flash_attn_tc_combine(const efa_flash_partials* part, void* O, int o_dtype,
                                         int row0, int rows, const efa_flash_params* p, void* stream)
{
    if (!part || !O || !p) { set_error("efa_flash_attn_tc_combine: null argument"); return 2; }
    if (o_dtype != EFA_F32 && o_dtype != EFA_F16) { set_error("efa_flash_attn_tc_combine: unknown dtype"); return 2; }
    return fa_combine(*part, O, o_dtype, row0, rows, *p, (cudaStream_t)stream);
}

extern "C" const char* efa_flash_attn_tc_check_params(const efa_flash_params* p, int q_rows)
{
    if (!p) return "null params";
    return fa_check_params(*p, q_rows);
}

extern "C" int efa_convert_f32_to_f16(const float* in, void* out, size_t n, void* stream)
{
    if ((!in || !out) && n) { set_error("efa_convert_f32_to_f16: null argument"); return 2; }
    return convert_f32_to_f16_dev(in, out, n, (cudaStream_t)stream);
}

extern "C" int efa_project_f16(const void* O_tile, const void* W_O, void* out, int rows, int d_local, int d, void* stream)
{
    return project_f16(O_tile, W_O, out, rows, d_local, d, (cudaStream_t)stream);
}

extern "C" int efa_compute_qkv_f16(const void* X, const void* W_q, const void* W_k, const void* W_v,
                                   void* Qh, void* Kh, void* Vh, int S, int d, int H_local, int d_h, void* stream)
{
    if (!X || !W_q || !W_k || !W_v || !Qh || !Kh || !Vh) { set_error("efa_compute_qkv_f16: null argument"); return 2; }
    if (d_h != 64 && d_h != 128) { set_error("efa_compute_qkv_f16: d_h must be 64 or 128 (got %d)", d_h); return 2; }
    if (H_local < 1) { set_error("efa_compute_qkv_f16: H_local must be positive"); return 2; }
    const __half* W[3] = {static_cast<const __half*>(W_q), static_cast<const __half*>(W_k), static_cast<const __half*>(W_v)};
    __half* out[3] = {static_cast<__half*>(Qh), static_cast<__half*>(Kh), static_cast<__half*>(Vh)};
    for (int h = 0; h < H_local; h++)
        for (int t = 0; t < 3; t++)
            if (int rc = project_f16(X, W[t] + (size_t)h * d * d_h, out[t] + (size_t)h * S * d_h, S, d, d_h, (cudaStream_t)stream))
                return rc;
    return 0;
}

extern "C" int efa_kernel_status(int* out4)
{
    if (!out4) { set_error("efa_kernel_status: null argument"); return 2; }
    int* w = kernel_status_word();
    if (!w) { set_error("efa_kernel_status: no status word (no device?)"); return 1; }
    EFA_CUDA(cudaMemcpy(out4, w, 4 * sizeof(int), cudaMemcpyDeviceToHost));
    return 0;
}

extern "C" int efa_kernel_status_reset(void)
{
    int* w = kernel_status_word();
    if (!w) { set_error("efa_kernel_status_reset: no status word (no device?)"); return 1; }
    EFA_CUDA(cudaMemset(w, 0, 4 * sizeof(int)));
    return 0;
}

extern "C" int efa_run_mode(efa_ctx* ctx, int mode, const efa_weights* w, void* output,
                            const efa_params* p, efa_run_stats* stats)
{
    if (!ctx || !w || !p) { set_error("efa_run_mode: null argument"); return 2; }
    return run_mode_impl(ctx, mode, *w, output, *p, stats);
}

extern "C" int efa_run_mode_residual(efa_ctx* ctx, int mode, const efa_weights* w, const void* residual, void* output,
                                     const efa_params* p, efa_run_stats* stats)
{
    if (!ctx || !w || !p || !residual) { set_error("efa_run_mode_residual: null argument"); return 2; }
    return run_mode_impl(ctx, mode, *w, output, *p, stats, residual);
}

extern "C" int efa_run_mode_host_rows(efa_ctx* c, int mode,
                                      const uint16_t* Qh, const uint16_t* Kh, const uint16_t* Vh, const uint16_t* W_O,
                                      uint16_t* output, int out_row0, int out_rows, const efa_params* p, efa_run_stats* stats)
{
    if (!c || !Qh || !Kh || !Vh || !W_O || !p) { set_error("efa_run_mode_host: null argument"); return 2; }
    if (p->proj_f32) { set_error("efa_run_mode_host: the host-buffer path returns fp16 (proj_f32 must be 0)"); return 2; }
    if (!output) out_rows = 0;
    if (out_rows < 0 || out_row0 < 0 || (out_rows > 0 && out_row0 + out_rows > p->S)) {
        set_error("efa_run_mode_host: rows [%d, %d) are outside the result", out_row0, out_row0 + out_rows);
        return 2;
    }
    const size_t qkv = (size_t)p->H_local * p->S * p->d_h * 2;
    const size_t wb = (size_t)p->d_local * p->d * 2;
    const size_t rowb = (size_t)p->d * 2;
    const size_t ob = (size_t)p->S * rowb;
    {
        size_t a = c->h_qkv_bytes, b = c->h_qkv_bytes, d = c->h_qkv_bytes;
        const bool fresh = a < qkv || !c->h_Q || !c->h_K || !c->h_V;
        if (ensure_bytes(&c->h_Q, &a, qkv) || ensure_bytes(&c->h_K, &b, qkv) || ensure_bytes(&c->h_V, &d, qkv)) return 1;
        if (fresh) {
            // Rows that a chunked copy has not delivered yet may still be touched by a tile load (their scores are
            // masked, but 0 * NaN is NaN): new staging starts as zeros, never as whatever the allocator returned.
            EFA_CUDA(cudaMemset(c->h_Q, 0, a));
            EFA_CUDA(cudaMemset(c->h_K, 0, b));
            EFA_CUDA(cudaMemset(c->h_V, 0, d));
        }
        c->h_qkv_bytes = a < b ? (a < d ? a : d) : (b < d ? b : d);
        if (ensure_bytes(&c->h_W, &c->h_w_bytes, wb)) return 1;
    }
    // Device result: the multicast region's result buffer when the switch reduces (written in place), else staging.
    void* dev_out = nullptr;
    const bool nvls = (p->reduce == EFA_REDUCE_NVLS || p->reduce == EFA_REDUCE_PULL) && p->R > 1 && !p->skip_comm;
    if (nvls) { if (efa_nvls_output(c, p, &dev_out)) return 1; }
    else { if (ensure_bytes(&c->h_out, &c->h_out_bytes, ob)) return 1; dev_out = c->h_out; }
    if (mode == EFA_MODE_STREAM && p->causal && !p->skip_proj && p->reduce != EFA_REDUCE_P2P) {
        // copy-in, compute and copy-out overlap chunk by chunk
        efa_weights dev{c->h_Q, c->h_K, c->h_V, c->h_W};
        return run_stream_host_pipelined(c, Qh, Kh, Vh, W_O, output, out_row0, out_rows, dev, dev_out, *p, stats);
    }
    if (world_barrier(c->world)) return 1;
    const auto t0 = std::chrono::steady_clock::now();
    cudaStream_t s = c->compute_stream;
    EFA_CUDA(cudaMemcpyAsync(c->h_Q, Qh, qkv, cudaMemcpyHostToDevice, s));
    EFA_CUDA(cudaMemcpyAsync(c->h_K, Kh, qkv, cudaMemcpyHostToDevice, s));
    EFA_CUDA(cudaMemcpyAsync(c->h_V, Vh, qkv, cudaMemcpyHostToDevice, s));
    EFA_CUDA(cudaMemcpyAsync(c->h_W, W_O, wb, cudaMemcpyHostToDevice, s));
    EFA_CUDA(cudaStreamSynchronize(s));
    efa_weights w{c->h_Q, c->h_K, c->h_V, c->h_W};
    efa_run_stats inner;
    std::memset(&inner, 0, sizeof(inner));
    if (run_mode_impl(c, mode, w, dev_out, *p, &inner)) return 1;
    if (out_rows > 0 && mode != EFA_MODE_ATTN && mode != EFA_MODE_ATTN_TILED) {
        EFA_CUDA(cudaMemcpyAsync(output, static_cast<char*>(dev_out) + (size_t)out_row0 * rowb, (size_t)out_rows * rowb,
                                 cudaMemcpyDeviceToHost, s));
        EFA_CUDA(cudaStreamSynchronize(s));
    }
    double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (world_max(c->world, &ms)) return 1;
    if (stats) { *stats = inner; stats->wall_ms = ms; }
    return 0;
}

extern "C" int efa_run_mode_host(efa_ctx* c, int mode,
                                 const uint16_t* Qh, const uint16_t* Kh, const uint16_t* Vh, const uint16_t* W_O,
                                 uint16_t* output, const efa_params* p, efa_run_stats* stats)
{
    return efa_run_mode_host_rows(c, mode, Qh, Kh, Vh, W_O, output, 0, (output && p) ? p->S : 0, p, stats);
}

extern "C" int efa_world_selftest(const efa_world* w)
{
    if (!w) { set_error("efa_world_selftest: null world"); return 2; }
    if (w->size <= 1) return 0;
    if (!w->barrier || !w->allreduce_max_f64 || !w->bcast_bytes || !w->allgather_bytes) {
        set_error("efa_world_selftest: a callback is missing");
        return 2;
    }
    if (w->barrier(w->user)) { set_error("efa_world_selftest: barrier failed"); return 1; }
    double v = 10.0 + w->rank;
    if (w->allreduce_max_f64(w->user, &v) || v != 10.0 + (w->size - 1)) {
        set_error("efa_world_selftest: max gave %g, expected %g", v, 10.0 + (w->size - 1));
        return 1;
    }
    unsigned char buf[128];
    for (int i = 0; i < 128; i++) buf[i] = (unsigned char)(w->rank == 0 ? (i * 7 + 3) : 0);
    if (w->bcast_bytes(w->user, buf, sizeof(buf), 0)) { set_error("efa_world_selftest: broadcast failed"); return 1; }
    for (int i = 0; i < 128; i++)
        if (buf[i] != (unsigned char)(i * 7 + 3)) { set_error("efa_world_selftest: broadcast byte %d wrong", i); return 1; }
    unsigned char mine[64], all[64 * 64];
    if (w->size > 64) { set_error("efa_world_selftest: more than 64 ranks"); return 2; }
    for (int i = 0; i < 64; i++) mine[i] = (unsigned char)(w->rank * 3 + i);
    if (w->allgather_bytes(w->user, mine, all, sizeof(mine))) { set_error("efa_world_selftest: all-gather failed"); return 1; }
    for (int r = 0; r < w->size; r++)
        for (int i = 0; i < 64; i++)
            if (all[r * 64 + i] != (unsigned char)(r * 3 + i)) { set_error("efa_world_selftest: all-gather slot %d wrong", r); return 1; }
    // A file descriptor from rank 0 to the others (how the handle of a multicast object travels): an anonymous
    // file with a known word in it; every receiver reads the word through its own descriptor.
    int fd = -1, got = -1;
    const unsigned magic = 0x0efab200u;
    if (w->rank == 0) {
        fd = memfd_create("efa-selftest", 0);
        if (fd < 0 || write(fd, &magic, sizeof(magic)) != (ssize_t)sizeof(magic)) { set_error("efa_world_selftest: memfd"); if (fd >= 0) close(fd); fd = -1; }
    }
    int bad = share_fd(*w, fd, &got) != 0;
    if (!bad && w->rank != 0) {
        unsigned word = 0;
        bad = pread(got, &word, sizeof(word), 0) != (ssize_t)sizeof(word) || word != magic;
        close(got);
    }
    if (fd >= 0) close(fd);
    double vote = bad ? 1.0 : 0.0;
    if (w->allreduce_max_f64(w->user, &vote) || vote != 0.0) { set_error("efa_world_selftest: passing a file descriptor between the ranks failed"); return 1; }
    return 0;
}
