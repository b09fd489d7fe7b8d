// attn_bench: benchmark CLI of the tensor-parallel attention block, one process per GPU.
// Same flags, defaults and CSV columns as attn_bench of eager-flash-attention (attn_bench.cu:48-58,
// 72-86, 139, 149-152); five columns are appended (tokens_per_s, attn_kernel_ms, reduce, data, wire).
// Ranks come from the MPI subset in mpi_shim/ (start with: efa_launch -n R attn_bench ...).
//
//   S,H,d_h,causal,R,kernel,tile,nbuf,split,ncomm,proj,mode,min_ms,max_ms,mean_ms,median_ms,std_ms,...
#include <mpi.h>

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <utility>
#include <string>
#include <vector>

#include "../../include/efa_b200.h"

static int g_rank = 0;

// Command line as a table: "--name value" pairs and bare "--switch" words. A name given twice keeps its last
// value, so a wrapper's defaults can be overridden by appending.
class CommandLine {
public:
    CommandLine(int argc, char** argv, std::initializer_list<const char*> switches)
    {
        for (int i = 1; i < argc; i++) {
            const std::string word = argv[i];
            const bool is_switch = std::find_if(switches.begin(), switches.end(), [&](const char* s) { return word == s; }) != switches.end();
            if (is_switch) { flags_.push_back(word); continue; }
            if (word.rfind("--", 0) == 0 && i + 1 < argc) { values_.emplace_back(word, argv[i + 1]); i++; }
        }
    }
    bool on(const char* name) const { return std::find(flags_.begin(), flags_.end(), name) != flags_.end(); }
    std::string text(const char* name, const char* fallback) const
    {
        std::string v = fallback;
        for (const auto& kv : values_) if (kv.first == name) v = kv.second;
        return v;
    }
    int number(const char* name, int fallback) const
    {
        const std::string v = text(name, "");
        return v.empty() ? fallback : std::atoi(v.c_str());
    }
private:
    std::vector<std::pair<std::string, std::string>> values_;
    std::vector<std::string> flags_;
};

[[noreturn]] static void fail(const char* what)
{
    if (g_rank == 0) fprintf(stderr, "ERROR: %s\n", what);
    MPI_Abort(MPI_COMM_WORLD, 1);
    std::exit(1);
}
#define EFA_OK(call) do { if ((call) != 0) { fprintf(stderr, "rank %d: %s: %s\n", g_rank, #call, efa_last_error()); MPI_Abort(MPI_COMM_WORLD, 1); } } while (0)
#define CUDA_OK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { fprintf(stderr, "rank %d: %s: %s\n", g_rank, #call, cudaGetErrorString(e_)); MPI_Abort(MPI_COMM_WORLD, 1); } } while (0)

static int cb_barrier(void*) { return MPI_Barrier(MPI_COMM_WORLD) != MPI_SUCCESS; }
static int cb_max(void*, double* v)
{
    double g = *v;
    int rc = MPI_Allreduce(v, &g, 1, MPI_DOUBLE, MPI_MAX, MPI_COMM_WORLD);
    *v = g;
    return rc != MPI_SUCCESS;
}
static int cb_bcast(void*, void* buf, size_t n, int root) { return MPI_Bcast(buf, (int)n, MPI_BYTE, root, MPI_COMM_WORLD) != MPI_SUCCESS; }
static int cb_gather(void*, const void* in, void* out, size_t n)
{
    return MPI_Allgather(in, (int)n, MPI_BYTE, out, (int)n, MPI_BYTE, MPI_COMM_WORLD) != MPI_SUCCESS;
}

// The five figures of a CSV row (attn_bench.cu:149-152 of the reference prints the same five).
struct Summary { double lo, hi, mean, median, stddev; };
static Summary summarize(const std::vector<double>& samples)
{
    Summary r{samples[0], samples[0], 0.0, 0.0, 0.0};
    for (double x : samples) { r.lo = std::min(r.lo, x); r.hi = std::max(r.hi, x); r.mean += x / samples.size(); }
    for (double x : samples) r.stddev += (x - r.mean) * (x - r.mean) / samples.size();
    r.stddev = std::sqrt(r.stddev);
    std::vector<double> mid(samples);
    std::nth_element(mid.begin(), mid.begin() + mid.size() / 2, mid.end());
    r.median = mid[mid.size() / 2];                       // upper median for an even count, as the reference takes it
    return r;
}

static void usage(const char* prog)
{
    fprintf(stderr,
        "usage: %s [--S 4096] [--H 16] [--d_h 64] [--tile 256] [--kernel tc]\n"
        "          [--nbuf 2] [--split 1] [--ncomm 1] [--warmup 3] [--trials 10]\n"
        "          [--modes attn,attn_tiled,megatron,sync,overlap,stream,comm] [--no-header]\n"
        "          [--causal] [--proj fp16|fp32] [--no_prio] [--no_proj] [--no_comm]\n"
        "          [--reduce nccl|p2p|nvls|pull] [--group_tiles 0] [--order auto|asc|desc|mixed] [--data normal|ref] [--seed 42] [--residual]\n"
        "          [--wire auto|f16|f32] [--band_rows 0] [--reserve_sms 0] [--reduce_ctas 0] [--trace] [--own_output]\n", prog);
}

int main(int argc, char** argv)
{
    int provided = 0, world = 1;
    if (MPI_Init_thread(&argc, &argv, MPI_THREAD_MULTIPLE, &provided) != MPI_SUCCESS) return 1;
    MPI_Comm_rank(MPI_COMM_WORLD, &g_rank);
    MPI_Comm_size(MPI_COMM_WORLD, &world);
    int ndev = 0;
    CUDA_OK(cudaGetDeviceCount(&ndev));
    if (ndev == 0) fail("no CUDA devices found");
    const int device = g_rank % ndev;
    CUDA_OK(cudaSetDevice(device));

    const CommandLine cl(argc, argv, {"--help", "--causal", "--no-header", "--no_prio", "--no_proj", "--no_comm", "--residual", "--trace", "--own_output"});
    if (cl.on("--help")) {
        if (g_rank == 0) usage(argv[0]);
        MPI_Finalize();
        return 0;
    }
    const int S = cl.number("--S", 4096), H = cl.number("--H", 16), d_h = cl.number("--d_h", 64);
    const int tile = cl.number("--tile", 256), nbuf = cl.number("--nbuf", 2);
    const int split = cl.number("--split", 1), ncomm = cl.number("--ncomm", 1);
    const int causal = cl.on("--causal") ? 1 : 0;
    const int warmup = cl.number("--warmup", 3), trials = cl.number("--trials", 10);
    const int seed = cl.number("--seed", 42);
    const std::string kernel_s = cl.text("--kernel", "tc"), proj_s = cl.text("--proj", "fp16");
    const std::string reduce_s = cl.text("--reduce", "nccl"), data_s = cl.text("--data", "normal"), order_s = cl.text("--order", "auto");
    const char* kernel = kernel_s.c_str();
    const char* proj = proj_s.c_str();
    const char* reduce = reduce_s.c_str();
    const char* data = data_s.c_str();
    const bool header = !cl.on("--no-header");
    const int d = H * d_h;

    if (std::strcmp(kernel, "tc") != 0) fail("--kernel must be tc (the scalar v1 prototype is not part of this build)");
    // --proj (attn_bench.cu:55,113-117 of the reference: fp32 | tf32 cuBLAS math). Here the operands are fp16 and the
    // accumulator fp32 in every case; the switch picks the type of the partial sums, the reduction and the output:
    // fp16 (default), or fp32 as in the reference. tf32 is accepted as a synonym of fp32.
    int proj_f32 = 0;
    if (std::strcmp(proj, "fp32") == 0 || std::strcmp(proj, "tf32") == 0) {
        if (std::strcmp(proj, "tf32") == 0 && g_rank == 0) fprintf(stderr, "note: --proj tf32 runs as fp32 (fp16 operands, fp32 partial sums)\n");
        proj = "fp32";
        proj_f32 = 1;
    } else if (std::strcmp(proj, "fp16") != 0) fail("--proj must be fp16 or fp32");
    if (trials < 1) fail("--trials must be >= 1");

    std::vector<int> modes;
    {
        // comma-separated mode names; empty items are ignored
        std::string item;
        const std::string list = cl.text("--modes", "attn,megatron,sync,overlap,stream") + ",";
        for (char ch : list) {
            if (ch != ',') { item.push_back(ch); continue; }
            if (item.empty()) continue;
            const int m = efa_parse_mode(item.c_str());
            if (m < 0) { if (g_rank == 0) fprintf(stderr, "ERROR: unknown mode '%s'\n", item.c_str()); MPI_Abort(MPI_COMM_WORLD, 1); }
            modes.push_back(m);
            item.clear();
        }
    }

    efa_params p;
    EFA_OK(efa_make_params(&p, S, d, H, tile, nbuf, split, causal, world));
    p.skip_proj = cl.on("--no_proj");
    p.skip_comm = cl.on("--no_comm");
    p.group_tiles = cl.number("--group_tiles", 0);
    p.band_rows = cl.number("--band_rows", 0);
    p.reserve_sms = cl.number("--reserve_sms", 0);
    p.reduce_ctas = cl.number("--reduce_ctas", 0);
    p.trace = cl.on("--trace") ? 1 : 0;
    p.proj_f32 = proj_f32;
    if (std::strcmp(reduce, "p2p") == 0) p.reduce = EFA_REDUCE_P2P;
    else if (std::strcmp(reduce, "nvls") == 0) p.reduce = EFA_REDUCE_NVLS;
    else if (std::strcmp(reduce, "pull") == 0) p.reduce = EFA_REDUCE_PULL;
    else if (std::strcmp(reduce, "nccl") != 0) fail("--reduce must be nccl, p2p, nvls or pull");
    if (order_s == "asc") p.row_order = EFA_ROWS_ASCENDING;
    else if (order_s == "desc") p.row_order = EFA_ROWS_DESCENDING;
    else if (order_s == "mixed") p.row_order = EFA_ROWS_MIXED;
    else if (order_s != "auto") fail("--order must be auto, asc, desc or mixed");
    const std::string wire_s = cl.text("--wire", "auto");
    if (wire_s == "f16") p.wire = EFA_WIRE_F16;
    else if (wire_s == "f32") p.wire = EFA_WIRE_F32;
    else if (wire_s != "auto") fail("--wire must be auto, f16 or f32");
    if (const char* why = efa_attn_check_params(&p)) {
        if (g_rank == 0) fprintf(stderr, "ERROR: invalid params: %s\n", why);
        MPI_Abort(MPI_COMM_WORLD, 1);
    }
    int recipe = 1;
    if (std::strcmp(data, "ref") == 0) recipe = 0;
    else if (std::strcmp(data, "normal") != 0) fail("--data must be normal or ref");

    efa_world w;
    std::memset(&w, 0, sizeof(w));
    w.rank = g_rank; w.size = world; w.local_device = device;
    w.barrier = cb_barrier; w.allreduce_max_f64 = cb_max; w.bcast_bytes = cb_bcast; w.allgather_bytes = cb_gather;
    efa_ctx* ctx = nullptr;
    EFA_OK(efa_make_ctx(&ctx, &w, ncomm, !cl.on("--no_prio")));

    const size_t qkv_n = (size_t)p.H_local * p.S * p.d_h, wo_n = (size_t)p.d_local * p.d, out_n = (size_t)p.S * p.d;
    std::vector<uint16_t> hq(qkv_n), hk(qkv_n), hv(qkv_n), hw(wo_n);
    EFA_OK(efa_fill_host_inputs(&p, g_rank, seed, recipe, hq.data(), hk.data(), hv.data(), hw.data()));
    efa_weights dw;
    void* output = nullptr;
    CUDA_OK(cudaMalloc(&dw.Qh, qkv_n * 2)); CUDA_OK(cudaMalloc(&dw.Kh, qkv_n * 2)); CUDA_OK(cudaMalloc(&dw.Vh, qkv_n * 2));
    CUDA_OK(cudaMalloc(&dw.W_O, wo_n * 2));
    // With the multicast reduction the output lives in the context's symmetric region, where the switch writes it in
    // place; --own_output keeps the reference's arrangement (the caller's cudaMalloc, one extra device copy per reduction).
    const bool symmetric_out = (p.reduce == EFA_REDUCE_NVLS || p.reduce == EFA_REDUCE_PULL) && world > 1 && !p.skip_comm && !cl.on("--own_output");
    if (symmetric_out) EFA_OK(efa_nvls_output(ctx, &p, &output));
    else CUDA_OK(cudaMalloc(&output, out_n * (proj_f32 ? 4 : 2)));
    CUDA_OK(cudaMemcpy(dw.Qh, hq.data(), qkv_n * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw.Kh, hk.data(), qkv_n * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw.Vh, hv.data(), qkv_n * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw.W_O, hw.data(), wo_n * 2, cudaMemcpyHostToDevice));

    // --residual: time the block together with the step after it (output = residual + block, the residual
    // added to each reduced group of rows as it lands); modes without a block output run as usual.
    void* residual = nullptr;
    if (cl.on("--residual")) {
        if (proj_f32) fail("--residual goes with --proj fp16");
        CUDA_OK(cudaMalloc(&residual, out_n * 2));
        CUDA_OK(cudaMemset(residual, 0x2c, out_n * 2));          // every element 0x2c2c = 0.0652
    }

    if (g_rank == 0 && header)
        printf("S,H,d_h,causal,R,kernel,tile,nbuf,split,ncomm,proj,mode,min_ms,max_ms,mean_ms,median_ms,std_ms,"
               "tokens_per_s,attn_kernel_ms,reduce,data,wire\n");
    for (int mode : modes) {
        std::vector<double> times, attn;
        for (int t = 0; t < warmup + trials; t++) {
            efa_run_stats st;
            const bool block_output = mode != EFA_MODE_ATTN && mode != EFA_MODE_ATTN_TILED && mode != EFA_MODE_COMM;
            if (residual && block_output) EFA_OK(efa_run_mode_residual(ctx, mode, &dw, residual, output, &p, &st));
            else EFA_OK(efa_run_mode(ctx, mode, &dw, output, &p, &st));
            if (t >= warmup) { times.push_back(st.wall_ms); attn.push_back(st.attn_kernel_ms); }
        }
        int status[4] = {0, 0, 0, 0};
        EFA_OK(efa_kernel_status(status));
        if (status[0] != 0) {
            fprintf(stderr, "rank %d: a kernel reported status %d (block %d, site %d)\n", g_rank, status[0], status[1], status[2]);
            MPI_Abort(MPI_COMM_WORLD, 1);
        }
        if (g_rank == 0) {
            const Summary s = summarize(times);
            const Summary a = summarize(attn);
            printf("%d,%d,%d,%d,%d,%s,%d,%d,%d,%d,%s,%s,%.4f,%.4f,%.4f,%.4f,%.4f,%.1f,%.4f,%s,%s,%s\n",
                   S, H, d_h, causal, world, kernel, tile, nbuf, split, ncomm, proj, efa_mode_name(mode),
                   s.lo, s.hi, s.mean, s.median, s.stddev, (double)S / (s.median * 1e-3), a.median, reduce, data,
                   p.wire == EFA_WIRE_F16 ? "f16" : "f32");
            fflush(stdout);
        }
    }
    cudaFree(dw.Qh); cudaFree(dw.Kh); cudaFree(dw.Vh); cudaFree(dw.W_O); cudaFree(residual);
    if (!symmetric_out) cudaFree(output);
    EFA_OK(efa_destroy_ctx(ctx));
    MPI_Finalize();
    return 0;
}
