// Execution modes of the tensor-parallel attention block (attention -> projection -> sum AllReduce).
// Counterpart of run_drivers.cu of eager-flash-attention (run_drivers.cu:9-30, 48-292): same seven
// modes, same timing convention (barrier, host clock, enqueue, synchronise, max over ranks), same
// stream roles; fp16 O, and fp16 (or, with proj_f32, the reference's fp32) partial sums / reduction / output;
// scratch cached in the context.
#include "runtime.h"

#include "fa_fwd_sm100.cuh"
#include "host_util.h"
#include "nccl_dyn.h"
#include "nvls_reduce.h"
#include "p2p_reduce.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

namespace efa {

namespace {

const char* kModeNames[EFA_MODE_COUNT] = {"attn", "attn_tiled", "megatron", "sync", "overlap", "stream", "comm"};

double now_ms()
{
    using namespace std::chrono;
    return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

// Consumer of a reduced group of rows, the step after the block: out += residual (fp16, one rounding),
// eight elements per thread and iteration. HBM-bound: 6 bytes per element.
__global__ void __launch_bounds__(256)
add_residual_kernel(__half* __restrict__ out, const __half* __restrict__ residual, size_t n8)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        uint4 o = reinterpret_cast<uint4*>(out)[i];
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(residual) + i);
        __half2* oh = reinterpret_cast<__half2*>(&o);
        const __half2* rh = reinterpret_cast<const __half2*>(&r);
        #pragma unroll
        for (int q = 0; q < 4; q++) oh[q] = __hadd2(oh[q], rh[q]);
        reinterpret_cast<uint4*>(out)[i] = o;
    }
}

int add_residual(__half* out, const __half* residual, size_t n, cudaStream_t stream)
{
    const size_t n8 = n / 8;                       // n = rows * d and d is a multiple of 64
    if (n8 == 0) return 0;
    int dev = 0, sms = 148;
    EFA_CUDA(cudaGetDevice(&dev));
    EFA_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    size_t blocks = (n8 + 255) / 256;
    if (blocks > (size_t)sms * 8) blocks = (size_t)sms * 8;
    add_residual_kernel<<<(unsigned)blocks, 256, 0, stream>>>(out, residual, n8);
    EFA_CUDA(cudaGetLastError());
    return 0;
}

struct Run {
    efa_ctx* c;
    const efa_weights& w;
    const efa_params& p;
    const __half* residual = nullptr;   // optional [S][d]: added to each reduced group of rows as it lands
    const char*   out_base = nullptr;   // the output buffer `residual` runs parallel to
    int launches = 0;

    // `output` is fp16, or fp32 with proj_f32 (the reference's types).
    size_t esz() const { return p.proj_f32 ? sizeof(float) : sizeof(__half); }
    size_t row_bytes() const { return (size_t)p.d * esz(); }
    // The partial sums that cross the links (efa_params.wire): the fp32 accumulators by default, summed in fp32 and
    // rounded once into the fp16 output, as the reference's types are (run_drivers.cu:26-30); fp16 on request (half
    // the bytes; every partial sum then carries its own rounding, and NCCL rounds once more per hop). The fused
    // peer-memory kernel stages fp16 and accumulates in fp32.
    bool wire_f32() const
    {
        if (p.proj_f32) return true;
        if (p.skip_comm || p.R == 1 || p.reduce == EFA_REDUCE_P2P) return false;
        if (p.reduce == EFA_REDUCE_PULL) return true;            // the pulling reduction adds fp32 partial sums only
        return p.wire != EFA_WIRE_F16;
    }
    // both reductions that deliver through the NVLink multicast region
    bool nvls() const { return (p.reduce == EFA_REDUCE_NVLS || p.reduce == EFA_REDUCE_PULL) && !p.skip_comm && p.R > 1; }
    bool pull() const { return p.reduce == EFA_REDUCE_PULL && nvls(); }
    size_t send_row_bytes() const { return (size_t)p.d * (wire_f32() ? sizeof(float) : sizeof(__half)); }
    char* send_base() const { return static_cast<char*>(pull() ? nvls_pull_send_buf(c) : nvls() ? nvls_send_buf(c) : c->send_buf); }

    efa_flash_partials ws(int rows) const
    {
        efa_flash_partials q{c->ws_O, c->ws_m, c->ws_l, rows};
        if (p.split <= 1) q = efa_flash_partials{nullptr, nullptr, nullptr, rows};
        return q;
    }

    // Attention kernel only (launch_attention_raw, attn_main.cu:234-245).
    // ws_row0: workspace row that the launch's first row maps to (split partials of several launches side by side).
    // heavy_first: -1 = the kernel's default (last rows first when nobody waits for counters), 0 / 1 = first / last rows first.
    int attention_raw(__half* O, int ws_rows, int q_start, int q_rows, cudaStream_t s, int* counters, int tile_rows,
                      int reserve_sms = 0, int band_rows = 0, int ws_row0 = 0, int heavy_first = -1, const short* order_tab = nullptr)
    {
        efa_flash_partials q = ws(ws_rows);
        if (q.O_part && ws_row0 > 0) {
            q.O_part += (size_t)ws_row0 * p.d_local;
            q.m_part += (size_t)ws_row0 * p.H_local;
            q.l_part += (size_t)ws_row0 * p.H_local;
        }
        launches++;
        return fa_forward(w.Qh, w.Kh, w.Vh, O, EFA_F16, &q, q_start, q_rows, p.flash_tc, s, counters, tile_rows, reserve_sms,
                          band_rows, heavy_first, order_tab);
    }
    // launch_combine (attn_main.cu:247-252): no-op when split == 1.
    int combine(__half* O, int ws_rows, int row0, int rows, cudaStream_t s)
    {
        if (p.split <= 1) return 0;
        launches++;
        return fa_combine(ws(ws_rows), O, EFA_F16, row0, rows, p.flash_tc, s);
    }
    int attention(__half* O, int ws_rows, int q_start, int q_rows, cudaStream_t s)
    {
        if (attention_raw(O, ws_rows, q_start, q_rows, s, nullptr, 0)) return 1;
        return combine(O, ws_rows, 0, q_rows, s);
    }
    // project (attn_main.cu:262-273) on the projection stream; `out` is a place in the send buffer.
    int project(const __half* O_tile, void* out, int rows)
    {
        if (p.skip_proj) return 0;
        launches++;
        return project_f16(O_tile, w.W_O, out, rows, p.d_local, p.d, c->proj_stream, wire_f32() ? EFA_F32 : EFA_F16);
    }
    // allreduce (run_drivers.cu:26-30): sum of n partial sums at `send` (a place in the send buffer) over the ranks
    // into `recv` (a place in `output`), on communicator / stream `slot`.
    int allreduce(int slot, void* send, void* recv, size_t n)
    {
        if (p.skip_comm) return 0;
        cudaStream_t cs = c->comm_streams[slot];
        if (nvls()) {
            // the switch sums the ranks' send buffers into every rank's result buffer; one local copy to `output`
            const bool f32 = wire_f32();
            const size_t first = (size_t)(static_cast<char*>(send) - send_base()) / (f32 ? sizeof(float) : sizeof(__half));
            launches++;
            if (nvls_allreduce(c, slot, first, n, f32, pull(), cs)) return 1;
            char* landed = static_cast<char*>(nvls_result_buf(c)) + first * sizeof(__half);
            if (landed != static_cast<char*>(recv))      // an output inside the region (efa_nvls_output) is written in place
                EFA_CUDA(cudaMemcpyAsync(recv, landed, n * sizeof(__half), cudaMemcpyDeviceToDevice, cs));
        } else {
            const NcclApi* nccl = nccl_api();
            if (!nccl) return 1;
            const bool f32 = wire_f32();
            void* dst = (f32 && !p.proj_f32) ? send : recv;          // fp32 sum in place, rounded into `output` below
            ncclResult_t r = nccl->AllReduce(send, dst, n, f32 ? ncclFloat : ncclHalf, ncclSum, c->nccls[slot], cs);
            if (r != ncclSuccess) { set_error("ncclAllReduce: %s", nccl->GetErrorString(r)); return 1; }
            if (f32 && !p.proj_f32) {
                launches++;
                if (convert_f32_to_f16_dev(static_cast<const float*>(send), recv, n, cs)) return 1;
            }
        }
        if (residual) {
            // consume the rows where they landed, on the stream that reduced them
            launches++;
            const size_t first = (size_t)(static_cast<const char*>(recv) - out_base) / sizeof(__half);   // fp16 output only
            return add_residual(static_cast<__half*>(recv), residual + first, n, cs);
        }
        return 0;
    }
};

// Release every front-end wait on the tile counters by storing a value above any target into them, from a stream
// that holds nothing else.
void release_counter_waits(efa_ctx* c, int* counters, size_t ncounters)
{
    if (!counters || !ncounters) return;
    if (!c->rescue_stream && cudaStreamCreateWithFlags(&c->rescue_stream, cudaStreamNonBlocking) != cudaSuccess) {
        (void)cudaGetLastError();
        return;
    }
    cudaMemsetAsync(counters, 0x7f, ncounters * sizeof(int), c->rescue_stream);
}

// Wait for a stream with a deadline. When the deadline passes (a tile counter that never reaches its target would
// block cuStreamWaitValue32 forever), the counters are overwritten so that every pending wait is released, the
// stream is given the same time again to drain, and an error is returned either way.
int sync_stream(efa_ctx* c, cudaStream_t s, int* counters, size_t ncounters)
{
    const double deadline_ms = c->host_wait_limit_ms;
    auto poll = [&](double limit_ms) -> int {        // 0 done, 1 not ready in time, 2 error
        const double t0 = now_ms();
        long spins = 0;
        while (true) {
            cudaError_t e = cudaStreamQuery(s);
            if (e == cudaSuccess) return 0;
            if (e != cudaErrorNotReady) { check_cuda(e, "cudaStreamQuery", __FILE__, __LINE__); return 2; }
            if ((++spins & 1023) == 0) {
                const double el = now_ms() - t0;
                if (el > limit_ms) return 1;
                if (el > 2000.0) std::this_thread::sleep_for(std::chrono::microseconds(200));
            }
        }
    };
    const int first = poll(deadline_ms);
    if (first == 0) return 0;
    if (first == 2) return 1;
    bool drained = false;
    if (counters && ncounters) {
        release_counter_waits(c, counters, ncounters);
        drained = poll(deadline_ms) == 0;
    }
    set_error("stream did not finish within %.1f s; pending tile waits were released%s", deadline_ms / 1e3,
              drained ? "" : " but the stream has not drained");
    return 4;
}

int sync_comm_streams(efa_ctx* c)
{
    for (int i = 0; i < c->ncomm; i++)
        if (sync_stream(c, c->comm_streams[i], nullptr, 0)) return 1;
    return 0;
}

int finish_timing(efa_ctx* c, double t0, efa_run_stats* st, bool attn_events, bool proj_events, int launches)
{
    double ms = now_ms() - t0;
    if (world_max(c->world, &ms)) return 1;
    if (st) {
        st->wall_ms = ms;
        st->attn_kernel_ms = 0.f;
        st->proj_ms = 0.f;
        st->kernel_launches = launches;
        if (attn_events) EFA_CUDA(cudaEventElapsedTime(&st->attn_kernel_ms, c->ev_t0, c->ev_t1));
        if (proj_events) EFA_CUDA(cudaEventElapsedTime(&st->proj_ms, c->ev_t2, c->ev_t3));
    }
    return 0;
}

int scratch(efa_ctx* c, const Run& r, size_t o_rows, size_t send_rows, size_t ncounters, size_t ws_rows, size_t nevents)
{
    const efa_params& p = r.p;
    if (o_rows && ensure_bytes(&c->O_all, &c->O_all_bytes, o_rows * p.d_local * sizeof(__half))) return 1;
    if (r.nvls()) { if (nvls_prepare(c, p)) return 1; }
    else if (send_rows && ensure_bytes(&c->send_buf, &c->send_bytes, send_rows * r.send_row_bytes())) return 1;
    if (ncounters) {
        size_t have = c->counters_n * sizeof(int);
        if (ensure_bytes((void**)&c->counters, &have, ncounters * sizeof(int))) return 1;
        c->counters_n = have / sizeof(int);
    }
    if (p.split > 1 && ws_rows) {
        size_t haveO = c->ws_O_n * sizeof(float);
        if (ensure_bytes((void**)&c->ws_O, &haveO, (size_t)p.split * ws_rows * p.d_local * sizeof(float))) return 1;
        c->ws_O_n = haveO / sizeof(float);
        size_t want = (size_t)p.split * ws_rows * p.H_local * sizeof(float);
        size_t haveM = c->ws_ml_n * sizeof(float), haveL = c->ws_ml_n * sizeof(float);
        if (ensure_bytes((void**)&c->ws_m, &haveM, want)) return 1;
        if (ensure_bytes((void**)&c->ws_l, &haveL, want)) return 1;
        c->ws_ml_n = std::min(haveM, haveL) / sizeof(float);
    }
    if (nevents && ensure_events(c, nevents)) return 1;
    return 0;
}

// ---------------------------------------------------------------------------------------------

// run_attn_only (run_drivers.cu:48-70)
int run_attn_only(Run& r, efa_run_stats* st, bool tiled)
{
    efa_ctx* c = r.c; const efa_params& p = r.p;
    if (scratch(c, r, p.S, 0, 0, tiled ? p.tile : p.S, 0)) return 1;
    __half* O_all = static_cast<__half*>(c->O_all);
    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();
    EFA_CUDA(cudaEventRecord(c->ev_t0, c->compute_stream));
    if (tiled) {
        for (int t = 0; t < p.num_tiles; t++)
            if (r.attention(O_all + (size_t)t * p.tile * p.d_local, p.tile, t * p.tile, p.tile, c->compute_stream)) return 1;
    } else {
        if (r.attention(O_all, p.S, 0, p.S, c->compute_stream)) return 1;
    }
    EFA_CUDA(cudaEventRecord(c->ev_t1, c->compute_stream));
    if (sync_stream(c, c->compute_stream, nullptr, 0)) return 1;
    return finish_timing(c, t0, st, true, false, r.launches);
}

// run_megatron (run_drivers.cu:72-106)
int run_megatron(Run& r, char* output, efa_run_stats* st)
{
    efa_ctx* c = r.c; const efa_params& p = r.p;
    if (scratch(c, r, p.S, p.S, 0, p.S, 2)) return 1;
    __half* O_all = static_cast<__half*>(c->O_all);
    char* send_buf = r.send_base();
    cudaEvent_t attn_done = c->events[0], proj_done = c->events[1];

    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();
    EFA_CUDA(cudaEventRecord(c->ev_t0, c->compute_stream));
    if (r.attention(O_all, p.S, 0, p.S, c->compute_stream)) return 1;
    EFA_CUDA(cudaEventRecord(c->ev_t1, c->compute_stream));
    EFA_CUDA(cudaEventRecord(attn_done, c->compute_stream));

    EFA_CUDA(cudaStreamWaitEvent(c->proj_stream, attn_done, 0));
    EFA_CUDA(cudaEventRecord(c->ev_t2, c->proj_stream));
    if (r.project(O_all, send_buf, p.S)) return 1;
    EFA_CUDA(cudaEventRecord(c->ev_t3, c->proj_stream));
    EFA_CUDA(cudaEventRecord(proj_done, c->proj_stream));

    EFA_CUDA(cudaStreamWaitEvent(c->comm_streams[0], proj_done, 0));
    if (r.allreduce(0, send_buf, output, (size_t)p.S * p.d)) return 1;
    if (sync_stream(c, c->comm_streams[0], nullptr, 0)) return 1;
    return finish_timing(c, t0, st, true, true, r.launches);
}

// run_sync (run_drivers.cu:108-136)
int run_sync(Run& r, char* output, efa_run_stats* st)
{
    efa_ctx* c = r.c; const efa_params& p = r.p;
    if (scratch(c, r, p.tile, p.tile, 0, p.tile, 0)) return 1;
    __half* O_tile = static_cast<__half*>(c->O_all);
    char* send_buf = r.send_base();
    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();
    for (int t = 0; t < p.num_tiles; t++) {
        if (r.attention(O_tile, p.tile, t * p.tile, p.tile, c->compute_stream)) return 1;
        if (sync_stream(c, c->compute_stream, nullptr, 0)) return 1;
        if (r.project(O_tile, send_buf, p.tile)) return 1;
        if (sync_stream(c, c->proj_stream, nullptr, 0)) return 1;
        if (r.allreduce(0, send_buf, output + (size_t)t * p.tile * r.row_bytes(), (size_t)p.tile * p.d)) return 1;
        if (sync_stream(c, c->comm_streams[0], nullptr, 0)) return 1;
    }
    return finish_timing(c, t0, st, false, false, r.launches);
}

// run_overlap (run_drivers.cu:143-194): every tile enqueued up front, three streams ordered by events:
//   compute: attn(t)  waits proj_done(t - nbuf)            (O buffer b free)
//   proj:    gemm(t)  waits attn_done(t), comm_done(t - nbuf)   (send buffer b free)
//   comm[t % ncomm]: allreduce(t) waits proj_done(t)
int run_overlap(Run& r, char* output, efa_run_stats* st)
{
    efa_ctx* c = r.c; const efa_params& p = r.p;
    const int nbuf = p.nbuf;
    if (scratch(c, r, (size_t)nbuf * p.tile, (size_t)nbuf * p.tile, 0, p.tile, (size_t)3 * nbuf)) return 1;
    __half* O_buf = static_cast<__half*>(c->O_all);
    char* S_buf = r.send_base();
    auto attn_done = [&](int b) { return c->events[3 * b]; };
    auto proj_done = [&](int b) { return c->events[3 * b + 1]; };
    auto comm_done = [&](int b) { return c->events[3 * b + 2]; };

    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();
    for (int t = 0; t < p.num_tiles; t++) {
        const int b = t % nbuf;
        __half* O_t = O_buf + (size_t)b * p.tile * p.d_local;
        char* S_t = S_buf + (size_t)b * p.tile * r.send_row_bytes();
        if (t >= nbuf) EFA_CUDA(cudaStreamWaitEvent(c->compute_stream, proj_done(b), 0));
        if (r.attention(O_t, p.tile, t * p.tile, p.tile, c->compute_stream)) return 1;
        EFA_CUDA(cudaEventRecord(attn_done(b), c->compute_stream));

        EFA_CUDA(cudaStreamWaitEvent(c->proj_stream, attn_done(b), 0));
        if (t >= nbuf) EFA_CUDA(cudaStreamWaitEvent(c->proj_stream, comm_done(b), 0));
        if (r.project(O_t, S_t, p.tile)) return 1;
        EFA_CUDA(cudaEventRecord(proj_done(b), c->proj_stream));

        const int slot = t % c->ncomm;
        EFA_CUDA(cudaStreamWaitEvent(c->comm_streams[slot], proj_done(b), 0));
        if (r.allreduce(slot, S_t, output + (size_t)t * p.tile * r.row_bytes(), (size_t)p.tile * p.d)) return 1;
        EFA_CUDA(cudaEventRecord(comm_done(b), c->comm_streams[slot]));
    }
    if (sync_stream(c, c->compute_stream, nullptr, 0)) return 1;
    if (sync_stream(c, c->proj_stream, nullptr, 0)) return 1;
    if (sync_comm_streams(c)) return 1;
    return finish_timing(c, t0, st, false, false, r.launches);
}

// run_stream (run_drivers.cu:201-255): one attention launch over all rows; the kernel counts finished
// 64-row blocks per tile; the projection stream holds, for every tile, a front-end wait on that
// tile's counter (cuStreamWaitValue32, no SM involved), the split combine, the projection and an
// event; the tile's AllReduce follows on communicator t % ncomm.
int run_stream(Run& r, char* output, efa_run_stats* st)
{
    efa_ctx* c = r.c; const efa_params& p = r.p;
    const DriverApi* api = driver_api();
    if (!api) return 1;
    if (scratch(c, r, p.S, p.S, p.num_tiles, p.S, (size_t)p.num_tiles + 1)) return 1;
    __half* O_all = static_cast<__half*>(c->O_all);
    char* send_buf = r.send_base();
    int* counters = c->counters;
    const int target = efa_blocks_per_tile(&p) + p.debug_target_bias;
    const bool fused = (p.reduce == EFA_REDUCE_P2P) && !p.skip_comm && !p.skip_proj;
    // Launch plan (efa_stream_plan): groups of consecutive tiles per projection + reduction launch in the order in
    // which they complete, and the band of rows within which the attention kernel may reorder its work (better
    // K/V reuse in L2 than strict row order when the local heads' K and V exceed the L2).
    std::vector<efa_stream_group> groups(p.num_tiles);
    int band_rows = 0, descending = 0;
    const int ngroups = efa_stream_plan(&p, groups.data(), p.num_tiles, &band_rows, &descending);
    if (ngroups < 0) return 1;
    // p.trace: timing events around every group (counters reached, projection done, reduction done) and a
    // timeline on stderr after the run, relative to the start of the attention kernel. Diagnostic; the events
    // cost a few microseconds each, so traced runs are not benchmark numbers.
    const bool trace = p.trace != 0 && !fused;
    if (trace && ensure_trace_events(c, (size_t)3 * ngroups)) return 1;
    if (fused) {
        // One persistent kernel does projection and reduction of every tile beside the attention kernel:
        // it polls the tile counters itself, so nothing is enqueued per tile. The attention kernel is
        // launched first: the first launch of a kernel may have to load its code, which can wait for
        // running kernels to drain, and a kernel that spins on the attention kernel's counters must
        // never be what that load waits for. The persistent CTAs (high-priority stream) take SMs as
        // the first attention CTAs retire. It takes the row blocks first to last, so the attention kernel does too.
        if (p2p_prepare(c, p, output)) return 1;
        if (world_barrier(c->world)) return 1;
        const double t0f = now_ms();
        EFA_CUDA(cudaEventRecord(c->ev_t0, c->compute_stream));
        if (r.attention_raw(O_all, p.S, 0, p.S, c->compute_stream, p2p_counters(c), p.tile, 0, 0, 0, 0)) return 1;
        EFA_CUDA(cudaEventRecord(c->ev_t1, c->compute_stream));
        if (p2p_launch(c, p, r.w, O_all, &r.launches)) return 1;
        if (r.residual) {
            // the persistent kernel ends when every row block of this rank's output has been written
            r.launches++;
            if (add_residual(reinterpret_cast<__half*>(output), r.residual, (size_t)p.S * p.d, c->proj_stream)) return 1;
        }
        if (sync_stream(c, c->compute_stream, nullptr, 0)) return 1;
        if (sync_stream(c, c->proj_stream, nullptr, 0)) return 1;
        return finish_timing(c, t0f, st, true, false, r.launches);
    }

    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();

    cudaEvent_t reset_done = c->events[p.num_tiles];
    EFA_CUDA(cudaMemsetAsync(counters, 0, (size_t)p.num_tiles * sizeof(int), c->compute_stream));
    EFA_CUDA(cudaEventRecord(reset_done, c->compute_stream));
    // p.reserve_sms = k runs the attention kernel in its persistent form on (SMs - k) CTAs, so that the
    // projection and the reduction of finished tiles always find an SM. Measured on 8 GPUs (benchmark
    // shape) this loses: the projection of a group is then confined to the k reserved SMs, while with the
    // plain grid its CTAs (higher stream priority) spread over every SM an attention CTA retires from.
    // EFA_ROWS_MIXED: the order of the 256-row blocks as a table in device memory (uploaded when it changes)
    const short* order_tab = nullptr;
    {
        std::vector<short> order(((size_t)p.S + 255) / 256);
        const int nb = efa_stream_row_blocks(&p, order.data(), (int)order.size());
        if (nb < 0) return 1;
        if (nb > 0) {
            order.resize(nb);
            if (order != c->order_tab_host) {
                size_t have = c->order_tab_n * sizeof(short);
                if (ensure_bytes((void**)&c->order_tab, &have, order.size() * sizeof(short))) return 1;
                c->order_tab_n = have / sizeof(short);
                c->order_tab_host = order;
                EFA_CUDA(cudaMemcpyAsync(c->order_tab, c->order_tab_host.data(), order.size() * sizeof(short),
                                         cudaMemcpyHostToDevice, c->compute_stream));
            }
            order_tab = c->order_tab;
        }
    }
    EFA_CUDA(cudaEventRecord(c->ev_t0, c->compute_stream));
    if (r.attention_raw(O_all, p.S, 0, p.S, c->compute_stream, counters, p.tile, p.reserve_sms, band_rows, 0, descending, order_tab)) return 1;
    EFA_CUDA(cudaEventRecord(c->ev_t1, c->compute_stream));

    EFA_CUDA(cudaStreamWaitEvent(c->proj_stream, reset_done, 0));   // never observe a stale counter
    // Tiles are signalled one by one; the projection and the reduction are launched once per group of
    // consecutive tiles, after a front-end wait on every counter of the group. group_tiles = 1 is the
    // reference's schedule. Small tiles make one launch and one collective per tile cost more than the
    // attention of the tile (a 128-row tile of the benchmark shape is a few microseconds of attention on
    // eight GPUs), so the default groups about S/8 rows.
    // From here on an error must not leave front-end waits behind on the projection stream: `fail` releases them.
    auto fail = [&]() {
        cudaStreamSynchronize(c->compute_stream);                 // the attention kernel no longer touches the counters
        release_counter_waits(c, counters, (size_t)p.num_tiles);
        return 1;
    };
    for (int gidx = 0; gidx < ngroups; gidx++) {
        const int t0g = groups[gidx].first_tile, nt = groups[gidx].ntiles;
        for (int t = t0g; t < t0g + nt; t++)
            if (check_cu(api->cuStreamWaitValue32((CUstream)c->proj_stream, (CUdeviceptr)(counters + t), (cuuint32_t)target,
                                                  CU_STREAM_WAIT_VALUE_GEQ), "cuStreamWaitValue32", __FILE__, __LINE__)) return fail();
        const int rows = nt * p.tile;
        __half* O_t = O_all + (size_t)t0g * p.tile * p.d_local;
        char* S_t = send_buf + (size_t)t0g * p.tile * r.send_row_bytes();
        if (trace) cudaEventRecord(c->trace_events[3 * gidx], c->proj_stream);
        if (r.combine(O_t, p.S, t0g * p.tile, rows, c->proj_stream)) return fail();
        if (r.project(O_t, S_t, rows)) return fail();
        if (cudaEventRecord(c->events[gidx], c->proj_stream) != cudaSuccess) return fail();
        if (trace) cudaEventRecord(c->trace_events[3 * gidx + 1], c->proj_stream);
        const int slot = gidx % c->ncomm;
        if (cudaStreamWaitEvent(c->comm_streams[slot], c->events[gidx], 0) != cudaSuccess) return fail();
        if (r.allreduce(slot, S_t, output + (size_t)t0g * p.tile * r.row_bytes(), (size_t)rows * p.d)) return fail();
        if (trace) cudaEventRecord(c->trace_events[3 * gidx + 2], c->comm_streams[slot]);
    }
    const double t_enqueued = now_ms() - t0;
    if (sync_stream(c, c->compute_stream, counters, p.num_tiles) || sync_stream(c, c->proj_stream, counters, p.num_tiles) ||
        sync_comm_streams(c)) {
        // a wait ran out and the counters were overwritten: what was enqueued behind the waits now drains (sync_stream
        // has given it time to); report
        return 1;
    }
    const int rc = finish_timing(c, t0, st, true, false, r.launches);
    if (trace && rc == 0) {
        float attn_end = 0.f;
        EFA_CUDA(cudaEventElapsedTime(&attn_end, c->ev_t0, c->ev_t1));
        fprintf(stderr, "efa trace rank %d: host enqueue done at %.3f ms after the barrier; attention kernel 0 .. %.3f ms\n",
                c->world.rank, t_enqueued, attn_end);
        for (int g = 0; g < ngroups; g++) {
            float t[3] = {0.f, 0.f, 0.f};
            for (int k = 0; k < 3; k++) EFA_CUDA(cudaEventElapsedTime(&t[k], c->ev_t0, c->trace_events[3 * g + k]));
            fprintf(stderr, "efa trace rank %d: rows %6d..%6d  counters reached %.3f  projected %.3f  reduced %.3f ms\n",
                    c->world.rank, groups[g].first_tile * p.tile, (groups[g].first_tile + groups[g].ntiles) * p.tile, t[0], t[1], t[2]);
        }
    }
    return rc;
}

// run_comm_only (run_drivers.cu:259-275): the per-tile AllReduces of a full pass, back to back on
// communicator 0; sweeping the tile size gives t_allreduce(bytes).
int run_comm_only(Run& r, char* output, efa_run_stats* st)
{
    efa_ctx* c = r.c; const efa_params& p = r.p;
    if (scratch(c, r, 0, p.S, 0, 0, 0)) return 1;
    char* send_buf = r.send_base();
    EFA_CUDA(cudaMemset(send_buf, 0, (size_t)p.S * r.send_row_bytes()));
    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();
    for (int t = 0; t < p.num_tiles; t++)
        if (r.allreduce(0, send_buf + (size_t)t * p.tile * r.send_row_bytes(), output + (size_t)t * p.tile * r.row_bytes(), (size_t)p.tile * p.d)) return 1;
    if (sync_stream(c, c->comm_streams[0], nullptr, 0)) return 1;
    return finish_timing(c, t0, st, false, false, r.launches);
}

}  // namespace

int run_stream_host_pipelined(efa_ctx* c, const uint16_t* Qh, const uint16_t* Kh, const uint16_t* Vh, const uint16_t* W_O,
                              uint16_t* host_out, int out_row0, int out_rows, const efa_weights& dev, void* dev_out,
                              const efa_params& p, efa_run_stats* stats)
{
    const DriverApi* api = driver_api();
    if (!api) return 1;
    if (!p.causal || p.skip_proj) { set_error("pipelined host path: causal mask and projection required"); return 2; }
    if (!c->h2d_stream) EFA_CUDA(cudaStreamCreateWithFlags(&c->h2d_stream, cudaStreamNonBlocking));
    if (!c->d2h_stream) EFA_CUDA(cudaStreamCreateWithFlags(&c->d2h_stream, cudaStreamNonBlocking));
    // Chunks of about S/8 rows, whole tiles, and every chunk boundary a multiple of 128 rows: the attention
    // kernels load keys in stages of up to 128 rows, and a stage must never reach into rows of the next chunk,
    // which are still on their way to the device.
    // The copy-in is the long pole (three tensors over PCIe), so what follows the last copy-in should be short: the
    // last eighth of the rows is cut into S/16, S/32 and S/32 where the alignment allows.
    int ct = (p.S / 8) / p.tile; if (ct < 1) ct = 1;
    while (((long)ct * p.tile) % 128 != 0) ct++;
    std::vector<int> chunk_first, chunk_tiles;          // in tiles
    for (int t = 0; t < p.num_tiles; ) {
        int nt = std::min(ct, p.num_tiles - t);
        if (t + ct >= p.num_tiles && nt == ct && ct % 4 == 0 && ((long)(ct / 4) * p.tile) % 128 == 0) {
            const int parts[3] = {ct / 2, ct / 4, ct / 4};
            for (int k = 0; k < 3; k++) { chunk_first.push_back(t); chunk_tiles.push_back(parts[k]); t += parts[k]; }
            break;
        }
        chunk_first.push_back(t); chunk_tiles.push_back(nt);
        t += nt;
    }
    const int nchunk = (int)chunk_first.size();
    Run r{c, dev, p};
    if (scratch(c, r, p.S, p.S, p.num_tiles, p.S, (size_t)3 * nchunk + 2)) return 1;
    __half* O_all = static_cast<__half*>(c->O_all);
    char* send_buf = r.send_base();
    char* output = static_cast<char*>(dev_out);
    char* host_bytes = reinterpret_cast<char*>(host_out);
    const size_t rb = r.row_bytes(), sb = r.send_row_bytes();
    int* counters = c->counters;
    const int target = efa_blocks_per_tile(&p);
    auto ev_in = [&](int i) { return c->events[3 * i]; };
    auto ev_proj = [&](int i) { return c->events[3 * i + 1]; };
    auto ev_ar = [&](int i) { return c->events[3 * i + 2]; };
    cudaEvent_t ev_w = c->events[3 * nchunk], reset_done = c->events[3 * nchunk + 1];
    const size_t head_pitch = (size_t)p.S * p.d_h * 2;            // bytes between heads, host and device alike

    if (world_barrier(c->world)) return 1;
    const double t0 = now_ms();
    EFA_CUDA(cudaMemcpyAsync(dev.W_O, W_O, (size_t)p.d_local * p.d * 2, cudaMemcpyHostToDevice, c->h2d_stream));
    EFA_CUDA(cudaEventRecord(ev_w, c->h2d_stream));
    EFA_CUDA(cudaMemsetAsync(counters, 0, (size_t)p.num_tiles * sizeof(int), c->compute_stream));
    EFA_CUDA(cudaEventRecord(reset_done, c->compute_stream));
    EFA_CUDA(cudaStreamWaitEvent(c->proj_stream, reset_done, 0));
    EFA_CUDA(cudaStreamWaitEvent(c->proj_stream, ev_w, 0));
    for (int i = 0; i < nchunk; i++) {
        const int t0c = chunk_first[i], nt = chunk_tiles[i];
        const int row0 = t0c * p.tile, rows = nt * p.tile;
        const size_t off = (size_t)row0 * p.d_h * 2, width = (size_t)rows * p.d_h * 2;
        // rows [row0, row0 + rows) of every head: one strided copy per tensor
        const void* src[3] = {Qh, Kh, Vh};
        void* dst[3] = {dev.Qh, dev.Kh, dev.Vh};
        for (int k = 0; k < 3; k++)
            EFA_CUDA(cudaMemcpy2DAsync(static_cast<char*>(dst[k]) + off, head_pitch, static_cast<const char*>(src[k]) + off, head_pitch,
                                       width, (size_t)p.H_local, cudaMemcpyHostToDevice, c->h2d_stream));
        EFA_CUDA(cudaEventRecord(ev_in(i), c->h2d_stream));
        // causal: rows of chunk i need keys of chunks 0..i only, and those are on the device now
        EFA_CUDA(cudaStreamWaitEvent(c->compute_stream, ev_in(i), 0));
        // split partials of all chunks share one [split][S] workspace, each chunk at its own rows
        if (r.attention_raw(O_all + (size_t)row0 * p.d_local, p.S, row0, rows, c->compute_stream, counters + t0c, p.tile, 0,
                            /* the chunk is consumed as a whole: */ rows >= 512 ? (rows > 2048 ? 2048 : (rows / 256) * 256) : 0,
                            row0)) return 1;
        for (int t = t0c; t < t0c + nt; t++)
            EFA_CU(api->cuStreamWaitValue32((CUstream)c->proj_stream, (CUdeviceptr)(counters + t), (cuuint32_t)target, CU_STREAM_WAIT_VALUE_GEQ));
        if (r.combine(O_all + (size_t)row0 * p.d_local, p.S, row0, rows, c->proj_stream)) return 1;
        if (r.project(O_all + (size_t)row0 * p.d_local, send_buf + (size_t)row0 * sb, rows)) return 1;
        EFA_CUDA(cudaEventRecord(ev_proj(i), c->proj_stream));
        const int slot = i % c->ncomm;
        EFA_CUDA(cudaStreamWaitEvent(c->comm_streams[slot], ev_proj(i), 0));
        if (p.skip_comm) {
            EFA_CUDA(cudaMemcpyAsync(output + (size_t)row0 * rb, send_buf + (size_t)row0 * sb, (size_t)rows * rb,
                                     cudaMemcpyDeviceToDevice, c->comm_streams[slot]));
        } else if (r.allreduce(slot, send_buf + (size_t)row0 * sb, output + (size_t)row0 * rb, (size_t)rows * p.d)) return 1;
        EFA_CUDA(cudaEventRecord(ev_ar(i), c->comm_streams[slot]));
        // the part of this chunk that the caller wants on the host
        const int lo = std::max(row0, out_row0), hi = std::min(row0 + rows, out_row0 + out_rows);
        if (host_out && hi > lo) {
            EFA_CUDA(cudaStreamWaitEvent(c->d2h_stream, ev_ar(i), 0));
            EFA_CUDA(cudaMemcpyAsync(host_bytes + (size_t)(lo - out_row0) * rb, output + (size_t)lo * rb, (size_t)(hi - lo) * rb,
                                     cudaMemcpyDeviceToHost, c->d2h_stream));
        }
    }
    if (sync_stream(c, c->h2d_stream, nullptr, 0)) return 1;
    if (sync_stream(c, c->compute_stream, counters, p.num_tiles)) return 1;
    if (sync_stream(c, c->proj_stream, counters, p.num_tiles)) return 1;
    if (sync_comm_streams(c)) return 1;
    if (sync_stream(c, c->d2h_stream, nullptr, 0)) return 1;
    return finish_timing(c, t0, stats, false, false, r.launches);
}

int modes_preload()
{
    cudaFuncAttributes attr;
    EFA_CUDA(cudaFuncGetAttributes(&attr, add_residual_kernel));
    return 0;
}

int run_mode_impl(efa_ctx* c, int mode, const efa_weights& w, void* output, const efa_params& p, efa_run_stats* stats,
                  const void* residual)
{
    if (!c) { set_error("run_mode: null context"); return 2; }
    if (const char* why = efa_attn_check_params(&p)) { set_error("invalid params: %s", why); return 2; }
    if (p.R != c->world.size) { set_error("params are for %d ranks, the context has %d", p.R, c->world.size); return 2; }
    if (!w.Qh || !w.Kh || !w.Vh || !w.W_O) { set_error("run_mode: null weights"); return 2; }
    if (mode != EFA_MODE_ATTN && mode != EFA_MODE_ATTN_TILED && !output) { set_error("run_mode: null output"); return 2; }
    if (residual && (p.skip_comm || p.skip_proj)) { set_error("run_mode: a residual needs the projection and the reduction"); return 2; }
    if (residual && (mode == EFA_MODE_ATTN || mode == EFA_MODE_ATTN_TILED || mode == EFA_MODE_COMM)) {
        set_error("run_mode: mode %s writes no block output to add a residual to", kModeNames[mode]);
        return 2;
    }
    if (p.proj_f32 && (residual || p.reduce != EFA_REDUCE_NCCL)) {
        set_error("run_mode: fp32 partial sums (proj_f32) go with the NCCL reduction and without a residual");
        return 2;
    }
    if (p.reduce != EFA_REDUCE_NCCL && p.reduce != EFA_REDUCE_P2P && p.reduce != EFA_REDUCE_NVLS && p.reduce != EFA_REDUCE_PULL) {
        set_error("run_mode: unknown reduction %d", p.reduce);
        return 2;
    }
    if ((p.reduce == EFA_REDUCE_NVLS || p.reduce == EFA_REDUCE_PULL) && p.R > 1 && !p.skip_comm) {
        const char* why = nullptr;
        if (!nvls_supported(c, p, &why)) { set_error("%s", why); return 5; }
    }
    Run r{c, w, p};
    char* out = static_cast<char*>(output);
    r.residual = static_cast<const __half*>(residual);
    r.out_base = out;
    switch (mode) {
        case EFA_MODE_ATTN:       return run_attn_only(r, stats, false);
        case EFA_MODE_ATTN_TILED: return run_attn_only(r, stats, true);
        case EFA_MODE_MEGATRON:   return run_megatron(r, out, stats);
        case EFA_MODE_SYNC:       return run_sync(r, out, stats);
        case EFA_MODE_OVERLAP:    return run_overlap(r, out, stats);
        case EFA_MODE_STREAM:     return run_stream(r, out, stats);
        case EFA_MODE_COMM:       return run_comm_only(r, out, stats);
    }
    set_error("unknown mode %d", mode);
    return 2;
}

}  // namespace efa

extern "C" const char* efa_mode_name(int mode)
{
    return (mode >= 0 && mode < EFA_MODE_COUNT) ? efa::kModeNames[mode] : "?";
}

extern "C" int efa_parse_mode(const char* s)
{
    if (!s) return -1;
    for (int i = 0; i < EFA_MODE_COUNT; i++)
        if (std::strcmp(s, efa::kModeNames[i]) == 0) return i;
    return -1;
}
