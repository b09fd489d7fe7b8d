// Output projection for sm_100a: out[rows][d] = A[rows][d_local] * W[d_local][d], fp16 operands,
// fp32 accumulation in tensor memory, fp16 result (or the fp32 accumulator itself, the reference's output type).
//
// Stands in for project() of eager-flash-attention (attn_main.cu:262-273), which calls cublasSgemm on
// fp32 data. Warp-specialised: warp 0 streams A (K-major, [128 rows][64 k]) and W (MN-major,
// [64 k][BN columns] as 64-column boxes) through a ring of shared-memory stages with TMA; warp 1
// issues tcgen05.mma (128 x BN x 16) into a BN-column fp32 accumulator in tensor memory and frees each
// stage with tcgen05.commit; warps 2-5 read the accumulator (tcgen05.ld), round to fp16 and store.
#include "fa_fwd_sm100.cuh"
#include "host_util.h"
#include "sm100_ptx.cuh"

namespace efa {

namespace {

constexpr int PJ_BM = 128;
constexpr int PJ_BK = 64;

template <int BN>
struct PjCfg {
    static constexpr int A_BYTES    = PJ_BM * PJ_BK * 2;          // 16 KB
    static constexpr int B_BOX      = PJ_BK * 64 * 2;             // one [64 k][64 n] box, 8 KB
    static constexpr int B_BYTES    = B_BOX * (BN / 64);
    static constexpr int STAGE      = A_BYTES + B_BYTES;
    static constexpr int NSTAGE     = BN == 256 ? 4 : 6;
    static constexpr int SMEM_BYTES = STAGE * NSTAGE + 1024;
};

struct PjArgs {
    void* out;          // fp16 or fp32 [M][N]
    int M, N, K;
    int* status;
};

template <int BN, bool OUT_F32>
__global__ void __launch_bounds__(192)
proj_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const PjArgs a)
{
    using C = PjCfg<BN>;
    constexpr uint32_t IDESC = idesc_f16_f32(PJ_BM, BN, 0, 1);
    constexpr uint32_t SWZ = swizzle_code(128);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    __shared__ __align__(8) uint64_t bar_full[C::NSTAGE];
    __shared__ __align__(8) uint64_t bar_empty[C::NSTAGE];
    __shared__ __align__(8) uint64_t bar_acc;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_word;

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * BN;
    const int m0 = blockIdx.y * PJ_BM;
    const int num_k = (a.K + PJ_BK - 1) / PJ_BK;

    if (tid == 0) {
        abort_word = 0;
        for (int s = 0; s < C::NSTAGE; s++) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
        mbar_init(&bar_acc, 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
    }
    __syncwarp();
    if (warp == 1) tmem_alloc(&tmem_base_smem, BN);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_acc = tmem_base_smem;

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            for (int kb = 0; kb < num_k; kb++) {
                const int s = kb % C::NSTAGE;
                const int use = kb / C::NSTAGE;
                if (use > 0 && !mbar_wait(&bar_empty[s], (uint32_t)((use - 1) & 1), &abort_word, 11)) break;
                uint8_t* sa = smem + s * C::STAGE;
                uint8_t* sb = sa + C::A_BYTES;
                mbar_expect_tx(&bar_full[s], C::STAGE);
                tma_load_2d(sa, &tmA, &bar_full[s], kb * PJ_BK, m0);
                #pragma unroll
                for (int nb = 0; nb < BN / 64; nb++)
                    tma_load_2d(sb + nb * C::B_BOX, &tmW, &bar_full[s], n0 + nb * 64, kb * PJ_BK);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < num_k && ok; kb++) {
                const int s = kb % C::NSTAGE;
                ok = mbar_wait(&bar_full[s], (uint32_t)((kb / C::NSTAGE) & 1), &abort_word, 12);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(smem + s * C::STAGE);
                const uint32_t sb = sa + C::A_BYTES;
                #pragma unroll
                for (int ks = 0; ks < PJ_BK / 16; ks++) {
                    tc_mma_ss(tmem_acc,
                              smem_desc(sa + ks * 32, 16, 1024, SWZ),                    // K-major: 32 B per 16 k
                              smem_desc(sb + ks * 16 * 128, C::B_BOX, 1024, SWZ),        // MN-major: 16 k rows of 128 B
                              IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(&bar_empty[s]);
            }
            if (ok) tc_commit(&bar_acc);
        }
    } else {
        // ---- epilogue: warps 2..5 own TMEM lanes 32*(warp % 4) .. +31
        const int lane_grp = warp & 3;
        const int row = m0 + lane_grp * 32 + lane;
        if (mbar_wait(&bar_acc, 0, &abort_word, 13)) {
            tc_fence_after_sync();
            const uint32_t taddr = tmem_acc + ((uint32_t)(lane_grp * 32) << 16);
            #pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                tmem_wait_ld();
                const int col = n0 + c * 32;
                if (OUT_F32) {
                    if (row < a.M && col < a.N) {
                        uint4* dst = reinterpret_cast<uint4*>(static_cast<float*>(a.out) + (size_t)row * a.N + col);
                        #pragma unroll
                        for (int q = 0; q < 8; q++) dst[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    }
                } else if (row < a.M && col < a.N) {   // N is a multiple of 64, so a 32-column chunk is all in or all out
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(a.out) + (size_t)row * a.N + col);
                    #pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint4 v;
                        v.x = pack_f16x2(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                        v.y = pack_f16x2(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                        v.z = pack_f16x2(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                        v.w = pack_f16x2(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                        dst[q] = v;
                    }
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (abort_word != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(100000);
        if (tid == 0 && a.status != nullptr) {
            if (atomicCAS(a.status, 0, (int)KS_WAIT_TIMEOUT) == 0) {
                a.status[1] = (int)(blockIdx.y * gridDim.x + blockIdx.x);
                a.status[2] = abort_word;
            }
        }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_acc, BN);
}

template <int BN, bool OUT_F32>
int launch_proj(const CUtensorMap& ta, const CUtensorMap& tw, const PjArgs& args, cudaStream_t stream)
{
    using C = PjCfg<BN>;
    static bool configured[64] = {};
    int dev = 0;
    EFA_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        EFA_CUDA(cudaFuncSetAttribute(proj_gemm_kernel<BN, OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        configured[dev] = true;
    }
    dim3 grid((args.N + BN - 1) / BN, (args.M + PJ_BM - 1) / PJ_BM);
    proj_gemm_kernel<BN, OUT_F32><<<grid, 192, C::SMEM_BYTES, stream>>>(ta, tw, args);
    EFA_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace

int project_f16(const void* A, const void* W, void* out, int rows, int d_local, int d, cudaStream_t stream, int out_dtype)
{
    if (out_dtype != EFA_F16 && out_dtype != EFA_F32) { set_error("project: unknown output type %d", out_dtype); return 2; }
    if (rows <= 0 || rows % 64 != 0) { set_error("project: rows (%d) must be a positive multiple of 64", rows); return 2; }
    if (d_local <= 0 || d_local % 16 != 0) { set_error("project: d_local (%d) must be a positive multiple of 16", d_local); return 2; }
    if (d <= 0 || d % 64 != 0) { set_error("project: d (%d) must be a positive multiple of 64", d); return 2; }
    if (!A || !W || !out) { set_error("project: null pointer"); return 2; }

    CUtensorMap ta, tw;
    {
        unsigned long long dims[2] = {(unsigned long long)d_local, (unsigned long long)rows};
        unsigned long long strides[1] = {(unsigned long long)d_local * 2ull};
        unsigned box[2] = {64u, 128u};
        if (make_tmap_f16(&ta, A, 2, dims, strides, box)) return 1;
    }
    {
        unsigned long long dims[2] = {(unsigned long long)d, (unsigned long long)d_local};
        unsigned long long strides[1] = {(unsigned long long)d * 2ull};
        unsigned box[2] = {64u, 64u};
        if (make_tmap_f16(&tw, W, 2, dims, strides, box)) return 1;
    }
    PjArgs a{out, rows, d, d_local, kernel_status_word()};
    const long tiles256 = (long)((rows + 127) / 128) * (d / 256);
    const bool wide = d % 256 == 0 && tiles256 >= 148;
    if (out_dtype == EFA_F32) return wide ? launch_proj<256, true>(ta, tw, a, stream) : launch_proj<128, true>(ta, tw, a, stream);
    return wide ? launch_proj<256, false>(ta, tw, a, stream) : launch_proj<128, false>(ta, tw, a, stream);
}


namespace {
template <class K> int touch_kernel(K kernel)
{
    cudaFuncAttributes attr;
    EFA_CUDA(cudaFuncGetAttributes(&attr, kernel));
    return 0;
}
}  // namespace

int proj_preload()
{
    return touch_kernel(proj_gemm_kernel<128, false>) || touch_kernel(proj_gemm_kernel<128, true>) ||
           touch_kernel(proj_gemm_kernel<256, false>) || touch_kernel(proj_gemm_kernel<256, true>);
}

}  // namespace efa
