// Projection fused with the cross-rank reduction, as ONE persistent kernel per rank that runs beside
// the attention kernel: the alternative to "projection kernel + ncclAllReduce per tile"
// (project + allreduce of eager-flash-attention, attn_main.cu:262-273, run_drivers.cu:26-30, as
// scheduled by run_stream, run_drivers.cu:201-255).
//
// G CTAs (one per SM, a small share of the GPU) loop over work items in row order:
//   GEMM item (rb, n):   wait until the attention kernel's tile counters say the 128 rows of row block
//                        rb are complete; out[128][128] = O[rb][:, :d_local] * W_O[:, n*128 : n*128+128]
//                        with tcgen05.mma (TMA-fed ring, double-buffered accumulator in tensor memory);
//                        the fp16 partial is written straight into the staging buffer of the rank that owns
//                        column block n (peer memory over NVLink, plain coalesced 16-byte stores), followed by
//                        a system-scope fence and an atomic increment of that rank's arrival flag.
//   REDUCE item (rb, m): the owner waits for R arrivals, sums the R staged partials in fp32, rounds once
//                        to fp16 and stores the result into every rank's output (peer stores), then
//                        increments every rank's done flag for row block rb.
// GEMM items come in groups (all column blocks one rank owns, for one row block) with one signal per
// group: a system-scope fence costs a round trip, so it is paid per group, not per tile. REDUCE work
// runs on four warps of its own, so a rank never holds back its projections while it waits for a
// peer's partial, and the projection side never waits on a peer at all.
// Flags and tile counters are never reset: targets grow with an epoch number that is the same on all
// ranks (runs are collective and separated by a host barrier), which removes the reset race between
// a rank that starts early and a peer that still clears its flags.
//
// With one rank there is nothing to reduce: the GEMM epilogue writes the output directly.
//
// Co-residency: a CTA of this kernel requests enough shared memory that no CTA of the two-tile
// attention kernel (which needs all 512 tensor-memory columns) can share its SM, so a tensor-memory
// allocation can never block on a CTA that only ends when the whole run ends.
//
// Every wait (mbarrier, tile counter, arrival flag, done flag) is bounded; on expiry the CTA records
// a status, stops taking work and frees its tensor memory. No TMA multicast is used.
#include "p2p_reduce.h"

#include "fa_fwd_sm100.cuh"
#include "host_util.h"
#include "sm100_ptx.cuh"

#include <cstring>
#include <map>
#include <string>
#include <vector>

struct P2PState {
    // shape the buffers were built for
    int S = 0, d = 0, d_local = 0, R = 0, tile = 0, target = 0;
    void* out_local = nullptr;
    long epoch = 0;
    // local allocations
    __half* stage = nullptr;     // [nrb][NBR][R][128][128]
    int* flags = nullptr;        // arrive[nrb*NBR] then done[nrb]
    int* counters = nullptr;     // tile counters, monotonic across runs
    // peer views (index = rank; own rank = local pointer)
    __half* stage_peer[8] = {};
    int* flags_peer[8] = {};
    __half* out_peer[8] = {};
    std::vector<void*> opened;   // pointers returned by cudaIpcOpenMemHandle
    CUtensorMap tmA, tmW;
    const void* tm_O = nullptr; const void* tm_W = nullptr;
    bool launched_this_run = false;
};

namespace efa {

namespace {

constexpr int PR_BM = 128, PR_BK = 64;
constexpr int PR_A_BYTES = PR_BM * PR_BK * 2;            // 16 KB
constexpr int PR_B_BOX = PR_BK * 64 * 2;                 // one [64 k][64 n] box of W_O, 8 KB
constexpr int PR_OUT_BYTES = PR_BM * 128 * 2;            // 32 KB staging of one 128x128 fp16 output tile
constexpr int PR_THREADS = 320;   // producer warp, MMA warp, 4 epilogue warps, 4 reduction warps
constexpr unsigned long long kChainSlackNs = 2000000000ull;  // waits inside the CTA that depend on a flag wait get this much longer

// BN = accumulator width. 256 keeps the tensor pipe fed: with 128 the two shared-memory operand reads
// of every MMA plus the TMA writes of the next stage exceed the shared-memory bandwidth and the MMAs run
// at about half rate. 128 remains for shapes whose per-rank column share is a single 128-column block.
template <int BN>
struct PrCfg {
    static constexpr int CB      = BN / 128;                          // 128-column blocks per item
    static constexpr int B_BYTES = (BN / 64) * PR_B_BOX;
    static constexpr int STAGE   = PR_A_BYTES + B_BYTES;              // 48 KB (BN = 256) or 32 KB
    static constexpr int NSTAGE  = BN == 256 ? 4 : 6;                 // 192 KB of operands in flight
    static constexpr int SMEM    = NSTAGE * STAGE + PR_OUT_BYTES + 1024;   // 225 KB: no attention CTA can share the SM
    static constexpr int TMEM    = 2 * BN;                            // two accumulators
};

struct PrArgs {
    int S, d, d_local, R, rank;
    int nrb, NB, NBR;              // row blocks of 128 rows; column blocks of 128; column blocks per rank
    int GS;                        // column blocks per work group (divides NBR): one signal per group
    int tile;                      // rows per tile counter
    int tile_target, arrive_target, done_target;
    const int* counters;
    __half* stage_peer[8];
    int* arrive_peer[8];
    int* done_peer[8];
    __half* out_peer[8];
    int* status;
    unsigned long long flag_wait_ns;   // limit of a wait on the attention kernel or on a peer
    unsigned long long chain_wait_ns;  // limit of the waits inside the CTA that depend on such a wait
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_add_sys(int* p, int v)
{
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// Poll until `*p` has reached `target` (counters only grow; the comparison survives their wrap-around), with a
// deadline. scope_sys: the writer is another GPU.
__device__ __forceinline__ bool wait_flag(const int* p, int target, bool scope_sys, volatile int* abort_word, int site,
                                          unsigned long long limit_ns)
{
    const unsigned long long t0 = globaltimer_ns();
    int spins = 0;
    while (true) {
        const int v = scope_sys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
        if ((int)((unsigned)v - (unsigned)target) >= 0) return true;
        if (*abort_word != 0) return false;
        if ((++spins & 15) == 0 && globaltimer_ns() - t0 > limit_ns) { *abort_word = site; return false; }
        __nanosleep(spins < 64 ? 100 : 500);
    }
}

__device__ __forceinline__ void bar_sync_epilogue() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void bar_sync_reduce() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
__device__ __forceinline__ bool bar_or_reduce(bool flag)
{
    int out;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.s32 p, %1, 0;\n"
        "bar.red.or.pred q, 2, 128, p;\n"
        "selp.s32 %0, 1, 0, q;\n"
        "}\n" : "=r"(out) : "r"((int)flag) : "memory");
    return out != 0;
}

// Barrier of the 128 epilogue threads that also ORs a flag over them: every thread gets the same
// answer, so all of them leave the work loop together (a thread that read the abort word a moment
// later than its neighbours must not take a different branch and strand them at the next barrier).
__device__ __forceinline__ bool bar_or_epilogue(bool flag)
{
    int out;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.s32 p, %1, 0;\n"
        "bar.red.or.pred q, 1, 128, p;\n"
        "selp.s32 %0, 1, 0, q;\n"
        "}\n" : "=r"(out) : "r"((int)flag) : "memory");
    return out != 0;
}

template <int BN>
__global__ void __launch_bounds__(PR_THREADS, 1)
tile_proj_reduce_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const PrArgs a)
{
    using C = PrCfg<BN>;
    constexpr uint32_t IDESC = idesc_f16_f32(PR_BM, BN, 0, 1);
    constexpr uint32_t SWZ = swizzle_code(128);
    constexpr int NST = C::NSTAGE;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_out = smem + NST * C::STAGE;

    __shared__ __align__(8) uint64_t bar_full[NST], bar_empty[NST];
    __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_word;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, g = blockIdx.x;
    const int num_k = (a.d_local + PR_BK - 1) / PR_BK;
    const int ngr = a.NB / a.GS;                   // GEMM groups per row block
    const int nrg = a.NBR / a.GS;                  // REDUCE groups per row block (this rank's shard)
    const int ipg = a.GS / C::CB;                  // GEMM items per group
    const long n_gemm = (long)a.nrb * ngr;         // GEMM groups
    const long n_red = (a.R > 1) ? (long)a.nrb * nrg : 0;

    if (tid == 0) {
        abort_word = 0;
        for (int s = 0; s < NST; s++) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
    }
    __syncwarp();
    if (warp == 1) tmem_alloc(&tmem_base_smem, C::TMEM);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ---- producer: waits for the row block's tiles, then streams A and W k-blocks
        if (lane == 0) {
            long kcount = 0;
            int ready_rb = -1;
            bool ok = true;
            for (long it = g; it < n_gemm && ok; it += G) {
                const int rb = (int)(it / ngr), gi = (int)(it % ngr);
                if (rb > ready_rb) {
                    const int t0 = (rb * PR_BM) / a.tile;
                    const int t1 = min(rb * PR_BM + PR_BM - 1, a.S - 1) / a.tile;
                    for (int t = t0; t <= t1 && ok; t++) ok = wait_flag(a.counters + t, a.tile_target, false, &abort_word, 41, a.flag_wait_ns);
                    if (!ok) break;
                    asm volatile("fence.proxy.async.global;" ::: "memory");   // O rows were written by generic-proxy stores
                    ready_rb = rb;
                }
                for (int j = 0; j < ipg && ok; j++) {
                    const int n0 = gi * a.GS + j * C::CB;          // first 128-column block of the item
                    for (int kb = 0; kb < num_k; kb++, kcount++) {
                        const int s = (int)(kcount % NST);
                        const long use = kcount / NST;
                        if (use > 0 && !mbar_wait(&bar_empty[s], (uint32_t)((use - 1) & 1), &abort_word, 42, a.chain_wait_ns)) { ok = false; break; }
                        uint8_t* sa = smem + s * C::STAGE;
                        uint8_t* sb = sa + PR_A_BYTES;
                        mbar_expect_tx(&bar_full[s], C::STAGE);
                        tma_load_2d(sa, &tmA, &bar_full[s], kb * PR_BK, rb * PR_BM);
                        #pragma unroll
                        for (int nb = 0; nb < BN / 64; nb++)
                            tma_load_2d(sb + nb * PR_B_BOX, &tmW, &bar_full[s], n0 * 128 + nb * 64, kb * PR_BK);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: accumulator buffer alternates per item
        if (lane == 0) {
            long kcount = 0, item = 0;
            bool ok = true;
            const long my_groups = (n_gemm > g) ? (n_gemm - g + G - 1) / G : 0;
            const long my_items = my_groups * ipg;            // the issuer only needs to count items
            for (; item < my_items && ok; item++) {
                const int b = (int)(item & 1);
                const long use = item >> 1;
                if (use > 0) ok = mbar_wait(&acc_empty[b], (uint32_t)((use - 1) & 1), &abort_word, 43, a.chain_wait_ns);
                if (!ok) break;
                tc_fence_after_sync();
                for (int kb = 0; kb < num_k; kb++, kcount++) {
                    const int s = (int)(kcount % NST);
                    ok = mbar_wait(&bar_full[s], (uint32_t)((kcount / NST) & 1), &abort_word, 44, a.chain_wait_ns);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * C::STAGE);
                    const uint32_t sb = sa + PR_A_BYTES;
                    #pragma unroll
                    for (int ks = 0; ks < PR_BK / 16; ks++)
                        tc_mma_ss(tmem_base + b * BN, smem_desc(sa + ks * 32, 16, 1024, SWZ),
                                  smem_desc(sb + ks * 16 * 128, PR_B_BOX, 1024, SWZ), IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
                    tc_commit(&bar_empty[s]);
                }
                if (ok) tc_commit(&acc_full[b]);
            }
        }
    } else if (warp >= 6) {
        // ---- reduction warps (128 threads): REDUCE groups in row order, independent of the GEMM flow
        const int et = tid - 192;                      // 0..127
        bool alive = true;
        for (long ri = g; ri < n_red && alive; ri += G) {
            const int rb = (int)(ri / nrg), cg = (int)(ri % nrg);
            if (et == 0) wait_flag(a.arrive_peer[a.rank] + rb, a.arrive_target, true, &abort_word, 45, a.flag_wait_ns);
            if (bar_or_reduce(abort_word != 0)) { alive = false; break; }
            for (int m = cg * a.GS; m < (cg + 1) * a.GS; m++) {
                const __half* src = a.stage_peer[a.rank] + ((size_t)rb * a.NBR + m) * a.R * (PR_BM * 128);
                const int col0 = (a.rank * a.NBR + m) * 128;
                // four 16-byte chunks per thread at a time, all R partials of each in flight together
                #pragma unroll 1
                for (int k4 = 0; k4 < 16; k4 += 4) {
                    float acc[4][8];
                    #pragma unroll
                    for (int u = 0; u < 4; u++)
                        #pragma unroll
                        for (int i = 0; i < 8; i++) acc[u][i] = 0.f;
                    for (int r = 0; r < a.R; r++) {
                        uint4 v[4];
                        #pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int ci = (k4 + u) * 128 + et;
                            v[u] = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)r * (PR_BM * 128) + (ci >> 4) * 128 + (ci & 15) * 8));
                        }
                        #pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const __half2* h = reinterpret_cast<const __half2*>(&v[u]);
                            #pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const float2 f = __half22float2(h[i]);
                                acc[u][2 * i] += f.x;
                                acc[u][2 * i + 1] += f.y;
                            }
                        }
                    }
                    #pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int ci = (k4 + u) * 128 + et;
                        const int row = ci >> 4, c = ci & 15;
                        uint4 o;
                        o.x = pack_f16x2(acc[u][0], acc[u][1]); o.y = pack_f16x2(acc[u][2], acc[u][3]);
                        o.z = pack_f16x2(acc[u][4], acc[u][5]); o.w = pack_f16x2(acc[u][6], acc[u][7]);
                        const int grow = rb * PR_BM + row;
                        if (grow < a.S) {
                            const size_t off = (size_t)grow * a.d + col0 + c * 8;
                            for (int q = 0; q < a.R; q++)
                                *reinterpret_cast<uint4*>(a.out_peer[q] + off) = o;
                        }
                    }
                }
            }
            __threadfence_system();
            bar_sync_reduce();
            if (et < a.R) red_add_sys(a.done_peer[et] + rb, 1);
        }
        // the output of this rank is complete when every owner has delivered every row block
        if (alive && a.R > 1 && et == 0)
            for (int rb = g; rb < a.nrb; rb += G)
                if (!wait_flag(a.done_peer[a.rank] + rb, a.done_target, true, &abort_word, 47, a.flag_wait_ns)) break;
    } else {
        // ---- epilogue warps (128 threads); TMEM lane quarter = warp % 4
        const int et = tid - 64;                       // 0..127
        const int lane_grp = warp & 3;
        const int erow = lane_grp * 32 + lane;         // accumulator row owned by this thread
        const uint32_t taddr0 = tmem_base + ((uint32_t)(lane_grp * 32) << 16);
        long item = 0;
        bool alive = true;

        for (long it = g; it < n_gemm && alive; it += G) {
            const int rb = (int)(it / ngr), gi = (int)(it % ngr);
            const int owner = (gi * a.GS) / a.NBR;
            for (int j = 0; j < ipg && alive; j++, item++) {
                const int n0 = gi * a.GS + j * C::CB;
                const int b = (int)(item & 1);
                // warp-uniform decision: the tensor-memory loads below need whole warps
                const bool got = __all_sync(0xffffffffu, mbar_wait(&acc_full[b], (uint32_t)((item >> 1) & 1), &abort_word, 46, a.chain_wait_ns));
                if (got) tc_fence_after_sync();
                #pragma unroll 1
                for (int h = 0; h < C::CB && alive; h++) {
                    if (got) {
                        // accumulator row -> fp16 -> shared memory (16-byte chunks XOR-swizzled by row against bank conflicts)
                        #pragma unroll
                        for (int c = 0; c < 4; c++) {
                            uint32_t r[32];
                            tmem_ld32(taddr0 + b * BN + h * 128 + c * 32, r);
                            tmem_wait_ld();
                            #pragma unroll
                            for (int q4 = 0; q4 < 4; q4++) {
                                uint4 v;
                                v.x = pack_f16x2(__uint_as_float(r[8 * q4 + 0]), __uint_as_float(r[8 * q4 + 1]));
                                v.y = pack_f16x2(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3]));
                                v.z = pack_f16x2(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5]));
                                v.w = pack_f16x2(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7]));
                                const int chunk = c * 4 + q4;
                                *reinterpret_cast<uint4*>(s_out + erow * 256 + ((chunk ^ (erow & 15)) << 4)) = v;
                            }
                        }
                        if (h == C::CB - 1) {
                            tc_fence_before_sync();
                            mbar_arrive(&acc_empty[b]);
                        }
                    }
                    if (bar_or_epilogue(abort_word != 0)) { alive = false; break; }

                    // coalesced copy-out of the staged 128x128 tile
                    const int n = n0 + h;
                    __half* dst;
                    size_t row_stride;
                    if (a.R > 1) {
                        dst = a.stage_peer[owner] + (((size_t)rb * a.NBR + (n % a.NBR)) * a.R + a.rank) * (PR_BM * 128);
                        row_stride = 128;
                    } else {
                        dst = a.out_peer[0] + (size_t)rb * PR_BM * a.d + (size_t)n * 128;
                        row_stride = (size_t)a.d;
                    }
                    #pragma unroll 4
                    for (int k = 0; k < 16; k++) {
                        const int ci = k * 128 + et;
                        const int row = ci >> 4, c = ci & 15;
                        const uint4 v = *reinterpret_cast<const uint4*>(s_out + row * 256 + ((c ^ (row & 15)) << 4));
                        if (a.R > 1 || rb * PR_BM + row < a.S)
                            *reinterpret_cast<uint4*>(dst + (size_t)row * row_stride + c * 8) = v;
                    }
                    if (a.R > 1 && j == ipg - 1 && h == C::CB - 1) {
                        // one signal per group: the fence covers the stores of all its tiles
                        __threadfence_system();
                        bar_sync_epilogue();
                        if (et == 0) red_add_sys(a.arrive_peer[owner] + rb, 1);
                    } else {
                        bar_sync_epilogue();               // s_out is reused by the next tile
                    }
                }
            }
        }
    }

    // ---- teardown
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (abort_word != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(100000);
        if (tid == 0 && a.status != nullptr) {
            if (atomicCAS(a.status, 0, (int)KS_WAIT_TIMEOUT) == 0) {
                a.status[1] = (int)blockIdx.x;
                a.status[2] = abort_word;
            }
        }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM);
}

template <int BN>
int launch_tile_kernel(const CUtensorMap& ta, const CUtensorMap& tw, const PrArgs& a, int G, cudaStream_t stream)
{
    using C = PrCfg<BN>;
    static bool configured[64] = {};
    int dev = 0;
    EFA_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        EFA_CUDA(cudaFuncSetAttribute(tile_proj_reduce_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[dev] = true;
    }
    tile_proj_reduce_kernel<BN><<<G, PR_THREADS, C::SMEM, stream>>>(ta, tw, a);
    EFA_CUDA(cudaGetLastError());
    return 0;
}

struct IpcPacket {
    cudaIpcMemHandle_t stage, flags, out;
    unsigned long long out_offset;
    int ok;
};

void release(P2PState* st)
{
    for (void* p : st->opened) cudaIpcCloseMemHandle(p);
    st->opened.clear();
    if (st->stage) cudaFree(st->stage);
    if (st->flags) cudaFree(st->flags);
    if (st->counters) cudaFree(st->counters);
    st->stage = nullptr; st->flags = nullptr; st->counters = nullptr;
    st->S = 0;
}

}  // namespace

int p2p_supported(const efa_params& p, const char** why)
{
    *why = nullptr;
    if (p.R > 8) *why = "reduce=p2p handles at most 8 ranks (one NVSwitch box)";
    else if (p.d % (128 * p.R) != 0) *why = "reduce=p2p needs d to be a multiple of 128 * ranks";
    else if (p.tile % 64 != 0) *why = "reduce=p2p needs a tile that is a multiple of 64";
    else if (p.split != 1) *why = "reduce=p2p needs split == 1 (the projection consumes O as the attention kernel writes it)";
    return *why == nullptr;
}

int p2p_prepare(efa_ctx* c, const efa_params& p, void* output)
{
    const char* why = nullptr;
    if (!p2p_supported(p, &why)) { set_error("%s", why); return 5; }
    if (!c->p2p) c->p2p = new P2PState();
    P2PState* st = c->p2p;
    const int R = p.R, rank = c->world.rank;
    const int nrb = (p.S + 127) / 128, NB = p.d / 128, NBR = NB / R;
    const int target = efa_blocks_per_tile(&p);
    st->launched_this_run = false;
    const bool same = st->S == p.S && st->d == p.d && st->d_local == p.d_local && st->R == R && st->tile == p.tile &&
                      st->target == target && st->out_local == output;
    // The rebuild is collective (handle exchange), so the ranks vote: one rank whose output pointer
    // changed makes all of them rebuild.
    double vote = same ? 0.0 : 1.0;
    if (world_max(c->world, &vote)) return 1;
    if (vote == 0.0) { st->epoch++; return 0; }
    if (world_barrier(c->world)) return 1;
    EFA_CUDA(cudaDeviceSynchronize());
    release(st);
    const size_t stage_bytes = (size_t)nrb * NB * 128 * 128 * sizeof(__half);
    const size_t nflags = (size_t)2 * nrb;          // arrive[nrb] then done[nrb]
    (void)NBR;
    // The rebuild is collective. A failure on one rank (no memory, an export or an import that fails) must not leave
    // the others inside the next exchange, so every local result is folded into a word that all ranks agree on
    // before anyone returns.
    auto agreed = [&](bool mine_ok) {
        double v = mine_ok ? 0.0 : 1.0;
        if (world_max(c->world, &v)) return false;
        return v == 0.0;
    };
    bool ok = true;
    if (R > 1) ok = cudaMalloc(&st->stage, stage_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&st->flags, nflags * sizeof(int)) == cudaSuccess &&
         cudaMemset(st->flags, 0, nflags * sizeof(int)) == cudaSuccess &&
         cudaMalloc(&st->counters, (size_t)p.num_tiles * sizeof(int)) == cudaSuccess &&
         cudaMemset(st->counters, 0, (size_t)p.num_tiles * sizeof(int)) == cudaSuccess &&
         cudaDeviceSynchronize() == cudaSuccess;
    if (!ok) (void)cudaGetLastError();
    if (!agreed(ok)) { release(st); set_error("reduce=p2p: a rank could not allocate its staging buffers"); return 1; }
    for (int r = 0; r < 8; r++) { st->stage_peer[r] = nullptr; st->flags_peer[r] = nullptr; st->out_peer[r] = nullptr; }
    st->stage_peer[rank] = st->stage; st->flags_peer[rank] = st->flags; st->out_peer[rank] = static_cast<__half*>(output);

    if (R > 1) {
        if (!c->world.allgather_bytes) { release(st); set_error("reduce=p2p needs the world's allgather_bytes callback"); return 2; }
        const DriverApi* api = driver_api();
        IpcPacket mine;
        std::memset(&mine, 0, sizeof(mine));
        mine.ok = api ? 1 : 0;
        CUdeviceptr base = 0; size_t range = 0;
        if (mine.ok && api->cuMemGetAddressRange(&base, &range, (CUdeviceptr)output) != CUDA_SUCCESS) mine.ok = 0;
        if (mine.ok && cudaIpcGetMemHandle(&mine.out, (void*)base) != cudaSuccess) mine.ok = 0;
        mine.out_offset = (unsigned long long)((CUdeviceptr)output - base);
        if (mine.ok && cudaIpcGetMemHandle(&mine.stage, st->stage) != cudaSuccess) mine.ok = 0;
        if (mine.ok && cudaIpcGetMemHandle(&mine.flags, st->flags) != cudaSuccess) mine.ok = 0;
        if (!mine.ok) (void)cudaGetLastError();
        std::vector<IpcPacket> all(R);
        if (c->world.allgather_bytes(c->world.user, &mine, all.data(), sizeof(IpcPacket))) { release(st); set_error("reduce=p2p: handle exchange failed"); return 1; }
        for (int r = 0; r < R; r++)
            if (!all[r].ok) {
                release(st);
                set_error("reduce=p2p: rank %d could not export its buffers over CUDA IPC (is the output a cudaMalloc allocation?)", r);
                return 5;
            }
        bool opened = true;
        for (int r = 0; r < R && opened; r++) {
            if (r == rank) continue;
            void* ps = nullptr; void* pf = nullptr; void* po = nullptr;
            opened = cudaIpcOpenMemHandle(&ps, all[r].stage, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
            if (opened) { st->opened.push_back(ps); opened = cudaIpcOpenMemHandle(&pf, all[r].flags, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess; }
            if (opened) { st->opened.push_back(pf); opened = cudaIpcOpenMemHandle(&po, all[r].out, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess; }
            if (opened) {
                st->opened.push_back(po);
                st->stage_peer[r] = static_cast<__half*>(ps);
                st->flags_peer[r] = static_cast<int*>(pf);
                st->out_peer[r] = reinterpret_cast<__half*>(static_cast<char*>(po) + all[r].out_offset);
            }
        }
        if (!opened) (void)cudaGetLastError();
        if (!agreed(opened)) { release(st); set_error("reduce=p2p: a rank could not map a peer's buffers (cudaIpcOpenMemHandle)"); return 5; }
        if (world_barrier(c->world)) return 1;
    }
    st->S = p.S; st->d = p.d; st->d_local = p.d_local; st->R = R; st->tile = p.tile; st->target = target;
    st->out_local = output;
    st->epoch = 1;
    st->tm_O = nullptr; st->tm_W = nullptr;
    return 0;
}

int* p2p_counters(efa_ctx* c) { return c->p2p ? c->p2p->counters : nullptr; }

// Launch the persistent kernel for this run.
int p2p_launch(efa_ctx* c, const efa_params& p, const efa_weights& w, const void* O_all, int* launches)
{
    P2PState* st = c->p2p;
    if (!st || st->S != p.S) { set_error("p2p_launch without p2p_prepare"); return 2; }
    if (st->launched_this_run) return 0;
    if (st->tm_O != O_all || st->tm_W != w.W_O) {
        unsigned long long dimsA[2] = {(unsigned long long)p.d_local, (unsigned long long)p.S};
        unsigned long long strA[1] = {(unsigned long long)p.d_local * 2ull};
        unsigned boxA[2] = {64u, 128u};
        if (make_tmap_f16(&st->tmA, O_all, 2, dimsA, strA, boxA)) return 1;
        unsigned long long dimsW[2] = {(unsigned long long)p.d, (unsigned long long)p.d_local};
        unsigned long long strW[1] = {(unsigned long long)p.d * 2ull};
        unsigned boxW[2] = {64u, 64u};
        if (make_tmap_f16(&st->tmW, w.W_O, 2, dimsW, strW, boxW)) return 1;
        st->tm_O = O_all; st->tm_W = w.W_O;
    }
    PrArgs a;
    std::memset(&a, 0, sizeof(a));
    a.S = p.S; a.d = p.d; a.d_local = p.d_local; a.R = p.R; a.rank = c->world.rank;
    a.nrb = (p.S + 127) / 128; a.NB = p.d / 128; a.NBR = a.NB / p.R;
    a.tile = p.tile;
    a.GS = (p.R > 1) ? a.NBR : 1;
    // Counters and flags only grow; the targets wrap with them (see wait_flag).
    a.tile_target = (int)(unsigned)((unsigned long long)st->epoch * (unsigned long long)st->target) + p.debug_target_bias;
    a.arrive_target = (int)(unsigned)((unsigned long long)st->epoch * (unsigned long long)(p.R * (a.NBR / a.GS)));
    a.done_target = a.arrive_target;
    a.flag_wait_ns = c->wait_limit_ns;
    a.chain_wait_ns = c->wait_limit_ns + kChainSlackNs;
    a.counters = st->counters;
    for (int r = 0; r < p.R; r++) {
        a.stage_peer[r] = st->stage_peer[r];
        a.arrive_peer[r] = st->flags_peer[r];
        a.done_peer[r] = st->flags_peer[r] + (size_t)a.nrb;
        a.out_peer[r] = st->out_peer[r];
    }
    a.status = kernel_status_word();

    // Accumulator width: two 128-column blocks per item whenever a group holds an even number of them.
    const bool wide = (a.GS % 2 == 0) || (p.R == 1 && a.NB % 2 == 0);
    if (p.R == 1 && wide) a.GS = 2;
    // Share of the GPU: projection FLOPs relative to attention + projection FLOPs, with head room.
    int G = 16;
    {
        const double attn = (p.causal ? 2.0 : 4.0) * (double)p.S * p.S * p.d_h * p.H_local;
        const double proj = 2.0 * (double)p.S * p.d_local * p.d;
        G = (int)(148.0 * proj / (attn + proj) * 0.9 + 0.5);   // measured: the projection runs at a higher fraction of peak than attention
        if (G < 6) G = 6;
        if (G > 48) G = 48;
        if (p.reduce_ctas >= 1 && p.reduce_ctas <= 148) G = p.reduce_ctas;
        const long groups = (long)a.nrb * (a.NB / a.GS);
        if (G > groups) G = (int)groups;
    }
    if (wide) { if (launch_tile_kernel<256>(st->tmA, st->tmW, a, G, c->proj_stream)) return 1; }
    else      { if (launch_tile_kernel<128>(st->tmA, st->tmW, a, G, c->proj_stream)) return 1; }
    if (launches) (*launches)++;
    st->launched_this_run = true;
    return 0;
}

void p2p_destroy(efa_ctx* c)
{
    if (!c->p2p) return;
    release(c->p2p);
    delete c->p2p;
    c->p2p = nullptr;
}


namespace {
template <class K> int touch_kernel(K kernel)
{
    cudaFuncAttributes attr;
    EFA_CUDA(cudaFuncGetAttributes(&attr, kernel));
    return 0;
}
}  // namespace

int p2p_preload() { return touch_kernel(tile_proj_reduce_kernel<128>) || touch_kernel(tile_proj_reduce_kernel<256>); }

}  // namespace efa
