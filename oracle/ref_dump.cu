// TEST INFRASTRUCTURE - generates the golden vectors under tests/golden/.
//
// Links against the UNMODIFIED sources of eager-flash-attention (compiled where they lie, see the
// Makefile) and runs that project's own GPU checker - baseline_attention (cuBLAS SGEMM +
// materialised softmax, baseline_attention.cu:82-143) followed by the cuBLAS projection of
// attn_tests.cu:41-48 - on inputs from its own recipe (allocate_and_fill + compute_qkv,
// attn_main.cu:98-153). A case with `ranks` > 1 is the block of that many ranks worked out one rank after the other
// on this one GPU: rank r's inputs (allocate_and_fill seeds by rank) and head share give its [S][d] partial sums, and
// the partial sums are added on the host in double precision, which is what the checker's sum over ranks
// (attn_tests.cu:50-60) yields up to fp32 rounding. Each case is written as raw little-endian fp32 [S][d] to
// <outdir>/<name>.f32 plus a line in <outdir>/manifest.txt. Needs a GPU; run as a single process.
#include "attn_main.cuh"
#include "baseline_attention.cuh"

#include <cmath>
#include <cstdio>
#include <string>
#include <vector>

struct Case { const char* name; int S, d, H, causal, seed, ranks; };

int main(int argc, char** argv)
{
    int rank, world;
    init_mpi(&argc, &argv, rank, world);
    init_cuda(rank);
    if (argc < 2 || world != 1) { fprintf(stderr, "usage: ref_dump <outdir>   (single rank)\n"); return 2; }
    const std::string outdir = argv[1];
    RunCtx ctx = make_ctx(MPI_COMM_WORLD, rank, world, 1);

    const Case cases[] = {
        {"ref_S128_d64_H4_nc_seed42",     128,  64, 4, 0,  42, 1},
        {"ref_S256_d128_H4_c_seed123",    256, 128, 4, 1, 123, 1},
        {"ref_S256_d256_H4_nc_seed777",   256, 256, 4, 0, 777, 1},
        {"ref_S128_d512_H4_c_seed42",     128, 512, 4, 1,  42, 1},
        {"ref_S256_d512_H4_c_seed42_R2",  256, 512, 4, 1,  42, 2},
        {"ref_S128_d1024_H8_nc_seed7_R4", 128, 1024, 8, 0,  7, 4},
        {"ref_S192_d512_H8_c_seed99_R8",  192, 512, 8, 1,  99, 8},
    };
    FILE* man = fopen((outdir + "/manifest.txt").c_str(), "w");
    if (!man) { perror("manifest"); return 1; }
    fprintf(man, "# name S d H causal seed max_abs_value ranks\n");

    for (const Case& cs : cases) {
        std::vector<double> sum((size_t)cs.S * cs.d, 0.0);
        for (int r = 0; r < cs.ranks; r++) {
            AttnParams p = make_params(cs.S, cs.d, cs.H, 64, 32, 64, KERNEL_TC, 2, 1, cs.causal, cs.ranks);
            Weights w = allocate_and_fill(p, r, cs.seed, ctx.compute_stream);
            CUDA_CHECK(cudaStreamSynchronize(ctx.compute_stream));
            CUBLAS_CHECK(cublasSetStream(ctx.cublas, ctx.proj_stream));
            compute_qkv(w, p, ctx.cublas);
            CUDA_CHECK(cudaStreamSynchronize(ctx.proj_stream));

            float *O_attn, *out, *workspace;
            CUDA_CHECK(cudaMalloc(&O_attn, (size_t)p.S * p.d_local * sizeof(float)));
            CUDA_CHECK(cudaMalloc(&out, (size_t)p.S * p.d * sizeof(float)));
            CUDA_CHECK(cudaMalloc(&workspace, baseline_attention_workspace_bytes(p.S)));
            baseline_attention(w.Q, w.K, w.V, O_attn, workspace, p.H_local, p.S, p.d_h, p.causal,
                               ctx.compute_stream, ctx.cublas);
            CUDA_CHECK(cudaStreamSynchronize(ctx.compute_stream));
            const float alpha = 1.f, beta = 0.f;
            CUBLAS_CHECK(cublasSetStream(ctx.cublas, ctx.proj_stream));
            CUBLAS_CHECK(cublasSgemm(ctx.cublas, CUBLAS_OP_N, CUBLAS_OP_N, p.d, p.S, p.d_local,
                                     &alpha, w.W_O, p.d, O_attn, p.d_local, &beta, out, p.d));
            CUDA_CHECK(cudaStreamSynchronize(ctx.proj_stream));

            std::vector<float> part((size_t)p.S * p.d);
            CUDA_CHECK(cudaMemcpy(part.data(), out, part.size() * sizeof(float), cudaMemcpyDeviceToHost));
            for (size_t i = 0; i < part.size(); i++) sum[i] += (double)part[i];
            CUDA_CHECK(cudaFree(O_attn));
            CUDA_CHECK(cudaFree(out));
            CUDA_CHECK(cudaFree(workspace));
            free_weights(w);
        }
        std::vector<float> h(sum.size());
        float mx = 0.f;
        for (size_t i = 0; i < sum.size(); i++) { h[i] = (float)sum[i]; mx = std::fabs(h[i]) > mx ? std::fabs(h[i]) : mx; }
        FILE* f = fopen((outdir + "/" + cs.name + ".f32").c_str(), "wb");
        if (!f) { perror("open"); return 1; }
        fwrite(h.data(), sizeof(float), h.size(), f);
        fclose(f);
        fprintf(man, "%s %d %d %d %d %d %.9g %d\n", cs.name, cs.S, cs.d, cs.H, cs.causal, cs.seed, mx, cs.ranks);
        printf("dumped %s max|v|=%g\n", cs.name, mx);
    }
    fclose(man);
    destroy_ctx(ctx);
    MPI_CHECK(MPI_Finalize());
    return 0;
}
