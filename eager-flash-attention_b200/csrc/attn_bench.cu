// attn_bench: benchmark CLI of the tensor-parallel attention block, one process per GPU.
// Same flags, defaults and CSV columns as attn_bench of eager-flash-attention (attn_bench.cu:48-58,
// 72-86, 139, 149-152); four columns are appended (tokens_per_s, attn_kernel_ms, reduce, data).
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
#include <numeric>
#include <string>
#include <vector>

#include "../../include/efa_b200.h"

static int g_rank = 0;

static const char* arg_str(int argc, char** argv, const char* flag, const char* def)
{
    const char* val = def;                       // the last occurrence wins, so a wrapper's defaults can be overridden
    for (int i = 1; i + 1 < argc; i++)
        if (std::strcmp(argv[i], flag) == 0) val = argv[i + 1];
    return val;
}
static int arg_int(int argc, char** argv, const char* flag, int def)
{
    const char* s = arg_str(argc, argv, flag, nullptr);
    return s ? std::atoi(s) : def;
}
static bool has_flag(int argc, char** argv, const char* flag)
{
    for (int i = 1; i < argc; i++)
        if (std::strcmp(argv[i], flag) == 0) return true;
    return false;
}

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

struct Stats { double min, max, mean, median, std; };
static Stats compute_stats(std::vector<double> v)
{
    std::sort(v.begin(), v.end());
    const double mean = std::accumulate(v.begin(), v.end(), 0.0) / v.size();
    double sq = 0.0;
    for (double x : v) sq += (x - mean) * (x - mean);
    return {v.front(), v.back(), mean, v[v.size() / 2], std::sqrt(sq / v.size())};
}

static void usage(const char* prog)
{
    fprintf(stderr,
        "usage: %s [--S 4096] [--H 16] [--d_h 64] [--tile 256] [--kernel tc]\n"
        "          [--nbuf 2] [--split 1] [--ncomm 1] [--warmup 3] [--trials 10]\n"
        "          [--modes attn,attn_tiled,megatron,sync,overlap,stream,comm] [--no-header]\n"
        "          [--causal] [--proj fp16|fp32] [--no_prio] [--no_proj] [--no_comm]\n"
        "          [--reduce nccl|p2p] [--group_tiles 0] [--data normal|ref] [--seed 42] [--residual]\n", prog);
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

    if (has_flag(argc, argv, "--help")) {
        if (g_rank == 0) usage(argv[0]);
        MPI_Finalize();
        return 0;
    }
    const int S = arg_int(argc, argv, "--S", 4096), H = arg_int(argc, argv, "--H", 16), d_h = arg_int(argc, argv, "--d_h", 64);
    const int tile = arg_int(argc, argv, "--tile", 256), nbuf = arg_int(argc, argv, "--nbuf", 2);
    const int split = arg_int(argc, argv, "--split", 1), ncomm = arg_int(argc, argv, "--ncomm", 1);
    const int causal = has_flag(argc, argv, "--causal") ? 1 : 0;
    const int warmup = arg_int(argc, argv, "--warmup", 3), trials = arg_int(argc, argv, "--trials", 10);
    const int seed = arg_int(argc, argv, "--seed", 42);
    const char* kernel = arg_str(argc, argv, "--kernel", "tc");
    const char* proj = arg_str(argc, argv, "--proj", "fp16");
    const char* reduce = arg_str(argc, argv, "--reduce", "nccl");
    const char* data = arg_str(argc, argv, "--data", "normal");
    const bool header = !has_flag(argc, argv, "--no-header");
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
        std::string list = arg_str(argc, argv, "--modes", "attn,megatron,sync,overlap,stream");
        size_t start = 0;
        while (start <= list.size()) {
            size_t end = list.find(',', start);
            if (end == std::string::npos) end = list.size();
            const std::string tok = list.substr(start, end - start);
            if (!tok.empty()) {
                const int m = efa_parse_mode(tok.c_str());
                if (m < 0) { if (g_rank == 0) fprintf(stderr, "ERROR: unknown mode '%s'\n", tok.c_str()); MPI_Abort(MPI_COMM_WORLD, 1); }
                modes.push_back(m);
            }
            start = end + 1;
        }
    }

    efa_params p;
    EFA_OK(efa_make_params(&p, S, d, H, tile, nbuf, split, causal, world));
    p.skip_proj = has_flag(argc, argv, "--no_proj");
    p.skip_comm = has_flag(argc, argv, "--no_comm");
    p.group_tiles = arg_int(argc, argv, "--group_tiles", 0);
    p.proj_f32 = proj_f32;
    if (std::strcmp(reduce, "p2p") == 0) p.reduce = EFA_REDUCE_P2P;
    else if (std::strcmp(reduce, "nccl") != 0) fail("--reduce must be nccl or p2p");
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
    EFA_OK(efa_make_ctx(&ctx, &w, ncomm, !has_flag(argc, argv, "--no_prio")));

    const size_t qkv_n = (size_t)p.H_local * p.S * p.d_h, wo_n = (size_t)p.d_local * p.d, out_n = (size_t)p.S * p.d;
    std::vector<uint16_t> hq(qkv_n), hk(qkv_n), hv(qkv_n), hw(wo_n);
    EFA_OK(efa_fill_host_inputs(&p, g_rank, seed, recipe, hq.data(), hk.data(), hv.data(), hw.data()));
    efa_weights dw;
    void* output = nullptr;
    CUDA_OK(cudaMalloc(&dw.Qh, qkv_n * 2)); CUDA_OK(cudaMalloc(&dw.Kh, qkv_n * 2)); CUDA_OK(cudaMalloc(&dw.Vh, qkv_n * 2));
    CUDA_OK(cudaMalloc(&dw.W_O, wo_n * 2)); CUDA_OK(cudaMalloc(&output, out_n * (proj_f32 ? 4 : 2)));
    CUDA_OK(cudaMemcpy(dw.Qh, hq.data(), qkv_n * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw.Kh, hk.data(), qkv_n * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw.Vh, hv.data(), qkv_n * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw.W_O, hw.data(), wo_n * 2, cudaMemcpyHostToDevice));

    // --residual: time the block together with the step after it (output = residual + block, the residual
    // added to each reduced group of rows as it lands); modes without a block output run as usual.
    void* residual = nullptr;
    if (has_flag(argc, argv, "--residual")) {
        if (proj_f32) fail("--residual goes with --proj fp16");
        CUDA_OK(cudaMalloc(&residual, out_n * 2));
        CUDA_OK(cudaMemset(residual, 0x2c, out_n * 2));          // every element 0x2c2c = 0.0652
    }

    if (g_rank == 0 && header)
        printf("S,H,d_h,causal,R,kernel,tile,nbuf,split,ncomm,proj,mode,min_ms,max_ms,mean_ms,median_ms,std_ms,"
               "tokens_per_s,attn_kernel_ms,reduce,data\n");
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
            const Stats s = compute_stats(times);
            const Stats a = compute_stats(attn);
            printf("%d,%d,%d,%d,%d,%s,%d,%d,%d,%d,%s,%s,%.4f,%.4f,%.4f,%.4f,%.4f,%.1f,%.4f,%s,%s\n",
                   S, H, d_h, causal, world, kernel, tile, nbuf, split, ncomm, proj, efa_mode_name(mode),
                   s.min, s.max, s.mean, s.median, s.std, (double)S / (s.median * 1e-3), a.median, reduce, data);
            fflush(stdout);
        }
    }
    cudaFree(dw.Qh); cudaFree(dw.Kh); cudaFree(dw.Vh); cudaFree(dw.W_O); cudaFree(output); cudaFree(residual);
    EFA_OK(efa_destroy_ctx(ctx));
    MPI_Finalize();
    return 0;
}
