// Warp-specialised FlashAttention forward for sm_100a, d_h = 64 or 128: the fast path behind
// flash_attn_tc_forward (flash_attn_tc.cu:73-312 of eager-flash-attention), same interface and
// semantics as the one-tile kernel in fa_fwd_sm100.cu.
//
// One CTA = 256 query rows (two 128-row Q tiles) of one (head, split), 384 threads:
//   warps 0-3   softmax of Q tile 0        (one thread per row; registers raised with setmaxnreg)
//   warps 4-7   softmax of Q tile 1
//   warp  8     TMA producer: Q tiles once, then K and V 128-key stages through two rings
//   warp  9     tcgen05.mma issuer; owns the tensor-memory allocation
//   warps 10-11 idle (they give their registers to the softmax warps)
// Both Q tiles share each K/V stage, which halves the L2 -> shared-memory traffic per FLOP. Each tile is a
// chain  S(j) -> softmax -> P(j) -> P(j)*V(j) -> Q*K^T(j+1) -> S(j+1)  (P overwrites S in tensor memory, and the
// tensor pipe executes in issue order), and the two chains run half a period apart: the one issuing thread
// serves them in turn,
//     ... PV0(j) QK0(j+1) | PV1(j) QK1(j+1) | PV0(j+1) QK0(j+2) | ...
// so that while one tile's softmax runs on the SIMT pipes (and has the special-function unit to itself) the
// tensor pipe executes the other tile's MMAs. A period is one softmax plus one tile's MMAs; timestamps taken
// inside the kernel (d_h = 128) put it at about 1770 + 1890 cycles against 2048 cycles of pure MMA time for
// both tiles. Two things were tried against that and measured slower: an issuing thread per tile (the tiles fall
// into step, both softmaxes then share the special-function unit and both MMA groups the tensor pipe), and
// 64-key stages with two S buffers per tile so that Q*K^T runs a stage ahead (a 128x64x16 MMA takes 48 cycles,
// not 32, and the issuing thread needs about as long per MMA as the tensor pipe). What did pay: descriptors kept
// in registers as (low, high) words, so that an MMA costs the issuing thread two additions and the instruction
// (it shares its scheduler with two softmax warps); a V ring one slot deeper than the K ring (V(j) is wanted
// right at the start of stage j, K(j+1) a whole stage after its slot is freed); packed fp32 pairs in the softmax.
// Computing a share of the exponentials with a polynomial on the FMA pipes lengthens the softmax and with it the
// chain; it was measured slower at every share.
// Tensor memory (512 columns): S0/P0 [0,128) S1/P1 [128,256) O0 [256,256+D) O1 [384,384+D).
// O is rescaled in tensor memory by the softmax warps themselves, and only when a row maximum grew
// by more than 2^8 since the value last used as the exponent offset (P then stays below 256, well
// inside fp16); the final division by the row sum makes the result independent of the offset.
// P reaches the MMA warp in two 64-key halves, each on its own mbarrier, so the first four k-steps of
// P*V start while the exponentials of the second half are still being computed.
//
// Work items (256 rows of one head/split) are taken either one per CTA from the grid, or, in the
// persistent form, by fewer CTAs than SMs from a global counter; the barriers are rebuilt per item.
// The order of the items is strict row order, or bands of rows taken head by head when the caller
// allows rows to complete band by band (see fetch_item).
//
// All waits are bounded; a warp leaves its loop as a whole when a wait fails, every other role then
// runs into its own bounded wait or sees the CTA's abort word, and the CTA frees its tensor memory.
#include "fa_fwd_sm100.cuh"
#include "fa_args.cuh"
#include "host_util.h"
#include "sm100_ptx.cuh"

#include <cmath>

namespace efa {

namespace {

constexpr int WS_BM = 128;          // rows per Q tile
constexpr int WS_BN = 128;          // keys per stage
constexpr int WS_THREADS = 384;
constexpr float kNegInfW = -INFINITY;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

template <int D>
struct WsCfg {
    static constexpr int SWB        = 128;
    static constexpr int BOXC       = 64;
    static constexpr int NBOX       = D / 64;
    static constexpr int BOX_BYTES  = 128 * SWB;                 // 16 KB
    static constexpr int TILE_BYTES = 128 * D * 2;
    static constexpr int NSTAGE_K   = D == 128 ? 2 : 4;           // K(j+1) is wanted a whole stage after its slot is freed,
    static constexpr int NSTAGE_V   = D == 128 ? 3 : 4;           // V(j) right at the start of the stage: the deeper ring
    static constexpr int SMEM_BYTES = TILE_BYTES * (2 + NSTAGE_K + NSTAGE_V) + 1024;
    static constexpr int TMEM_COLS  = 512;
};

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Two fp32 lanes per instruction (fma.rn.f32x2 / add.rn.f32x2: same rounding as the scalar forms): scale-and-offset
// and the row sum of the softmax take half the instructions. Measured: 3 % of the attention launch.
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}





__device__ __forceinline__ void setmaxnreg_dec_56() { asm volatile("setmaxnreg.dec.sync.aligned.u32 56;"); }
__device__ __forceinline__ void setmaxnreg_inc_224() { asm volatile("setmaxnreg.inc.sync.aligned.u32 224;"); }

// PERSIST = false: one work item (256 rows of one head/split) per CTA, grid (H_local*split, row blocks).
// PERSIST = true: a 1-D grid of fewer CTAs than SMs; each CTA takes work items from a global counter in
// the same row-major order. The SMs left without a CTA stay free for the projection and the AllReduce
// of finished tiles, which otherwise can only start when an attention CTA retires.
template <int D, bool OUT_F16, bool PERSIST>
__global__ void __launch_bounds__(WS_THREADS, 1)
fa_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmQ,
                 const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV,
                 const FaArgs a, int* work_counter, int items_x, int items_total)
{
    using C = WsCfg<D>;
    constexpr uint32_t SWZ = swizzle_code(128);
    constexpr uint32_t IDESC_QK = idesc_f16_f32(WS_BM, WS_BN, 0, 0);
    constexpr uint32_t IDESC_PV = idesc_f16_f32(WS_BM, D, 0, 1);
    constexpr int NSK = C::NSTAGE_K, NSV = C::NSTAGE_V;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                                   // 2 tiles
    uint8_t* sK = sQ + 2 * C::TILE_BYTES;                 // NSK stages
    uint8_t* sV = sK + NSK * C::TILE_BYTES;               // NSV stages

    __shared__ __align__(8) uint64_t q_full[2];
    __shared__ __align__(8) uint64_t k_full[NSK], k_empty[NSK], v_full[NSV], v_empty[NSV];
    __shared__ __align__(8) uint64_t s_full[2], p_full[2][2], o_done[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_word;
    __shared__ int half_done[2][2];                       // [tile][64-row half]: warps that finished their stores
    __shared__ int s_item;

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // ---- once per CTA
    if (tid == 0) {
        abort_word = 0;
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 9) tmem_alloc(&tmem_base_smem, C::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_smem;
    const int kv_len = a.kv_len;

    struct ItemInfo { int head, split, block_row0, kv_lo, kv_hi, nblk_max; int q_abs0[2], rows_q[2], nblk[2]; };
    // Next work item. Thread 0 rebuilds the barriers for every item: all threads are past the previous one.
    // Both role branches below call this the same number of times, so its __syncthreads pair up.
    auto fetch_item = [&](int round, ItemInfo& it) -> bool {
        // ---- next work item; barriers are rebuilt for every item (all threads are past the previous one)
        if (tid == 0) {
            s_item = PERSIST ? atomicAdd(work_counter, 1) : (int)(blockIdx.y * gridDim.x + blockIdx.x);
            half_done[0][0] = half_done[0][1] = half_done[1][0] = half_done[1][1] = 0;
            if (round > 0) {
                for (int q = 0; q < 2; q++) { mbar_inval(&q_full[q]); mbar_inval(&s_full[q]); mbar_inval(&p_full[q][0]); mbar_inval(&p_full[q][1]); mbar_inval(&o_done[q]); }
                for (int s = 0; s < NSK; s++) { mbar_inval(&k_full[s]); mbar_inval(&k_empty[s]); }
                for (int s = 0; s < NSV; s++) { mbar_inval(&v_full[s]); mbar_inval(&v_empty[s]); }
            }
            for (int q = 0; q < 2; q++) {
                mbar_init(&q_full[q], 1);
                mbar_init(&s_full[q], 1);
                mbar_init(&p_full[q][0], WS_BM);
                mbar_init(&p_full[q][1], WS_BM);
                mbar_init(&o_done[q], 1);
            }
            for (int s = 0; s < NSK; s++) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
            for (int s = 0; s < NSV; s++) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
            mbar_fence_init();
        }
        __syncthreads();
        const int item = s_item;
        if (item >= items_total || abort_word != 0) return false;

        // Work order. Strict row order (heads fastest) makes every head's K/V stream live at once, far more than
        // the L2 holds. With bands, the blocks of one band of rows are taken head by head: the CTAs in flight then
        // share a few heads' K/V, and rows still complete band by band, which is all a consumer that handles
        // groups of tiles needs.
        int item_x, item_y;
        {
            const int items_y = items_total / items_x;
            const int band = a.band_blocks > 1 ? min(a.band_blocks, items_y) : 1;
            const int per_band = items_x * band;
            const int full = items_y / band;
            int b = item / per_band, rem = item - b * per_band, nb = band;
            if (b >= full) { b = full; rem = item - full * per_band; nb = items_y - full * band; }
            item_x = rem / nb;
            item_y = b * band + rem % nb;
            // Longest items first: list scheduling then ends on the shortest items instead of the longest, which
            // is worth up to one item's duration (a fifth of the launch with four heads per GPU at 32k rows).
            if (a.order_tab != nullptr && band == 1) item_y = a.order_tab[item_y];
            else if (a.heavy_first) item_y = items_y - 1 - item_y;
        }
        it.head  = item_x % a.H_local;
        it.split = item_x / a.H_local;
        it.block_row0 = item_y * (2 * WS_BM);
        const int rows_valid = min(2 * WS_BM, a.q_rows - it.block_row0);      // 64, 128, 192 or 256
        it.kv_lo = it.split * kv_len;
        it.kv_hi = it.kv_lo + kv_len;

        // Per Q tile: first absolute row, valid rows, number of key stages.
        #pragma unroll
        for (int q = 0; q < 2; q++) {
            it.q_abs0[q] = a.q_start + it.block_row0 + q * WS_BM;
            it.rows_q[q] = max(0, min(WS_BM, rows_valid - q * WS_BM));
            const int kv_end = a.causal ? min(it.kv_hi, it.q_abs0[q] + it.rows_q[q]) : it.kv_hi;
            it.nblk[q] = (it.rows_q[q] > 0 && kv_end > it.kv_lo) ? (kv_end - it.kv_lo + WS_BN - 1) / WS_BN : 0;
        }
        it.nblk_max = max(it.nblk[0], it.nblk[1]);
        return true;
    };
    auto end_item = [&]() {
        __syncwarp();
        tc_fence_before_sync();
        __syncthreads();
        tc_fence_after_sync();
    };
#define EFA_ITEM_LOCALS \
    const int head = it.head, split = it.split, block_row0 = it.block_row0, kv_lo = it.kv_lo, kv_hi = it.kv_hi, nblk_max = it.nblk_max; \
    const int* q_abs0 = it.q_abs0; const int* rows_q = it.rows_q; const int* nblk = it.nblk; \
    (void)head; (void)split; (void)block_row0; (void)kv_lo; (void)kv_hi; (void)nblk_max; (void)q_abs0; (void)rows_q; (void)nblk;

    if (warp >= 8) {
        setmaxnreg_dec_56();
        for (int round = 0; ; round++) {
            ItemInfo it;
            if (!fetch_item(round, it)) break;
            EFA_ITEM_LOCALS
            // =====================================================================================
            // Producer / MMA warpgroup
            // =====================================================================================
            if (warp == 8 && lane == 0) {
                // ---- TMA producer
                auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row) {
                    mbar_expect_tx(bar, C::TILE_BYTES);
                    #pragma unroll
                    for (int b = 0; b < C::NBOX; b++)
                        tma_load_3d(dst + b * C::BOX_BYTES, tm, bar, b * C::BOXC, row, head);
                };
                for (int q = 0; q < 2; q++)
                    if (nblk[q] > 0) load_tile(sQ + q * C::TILE_BYTES, &tmQ, &q_full[q], q_abs0[q]);
                for (int j = 0; j < nblk_max; j++) {
                    const int sk = j % NSK, uk = j / NSK, sv = j % NSV, uv = j / NSV;
                    if (uk > 0 && !mbar_wait(&k_empty[sk], (uint32_t)((uk - 1) & 1), &abort_word, 21)) break;
                    load_tile(sK + sk * C::TILE_BYTES, &tmK, &k_full[sk], kv_lo + j * WS_BN);
                    if (uv > 0 && !mbar_wait(&v_empty[sv], (uint32_t)((uv - 1) & 1), &abort_word, 22)) break;
                    load_tile(sV + sv * C::TILE_BYTES, &tmV, &v_full[sv], kv_lo + j * WS_BN);
                }
            } else if (warp == 9 && lane == 0) {
                // ---- MMA issuer. Descriptors as (low, high) words; a k-step or a ring slot only moves the address
                // field of the low word.
                const uint64_t dq0 = smem_desc(smem_u32(sQ), 16, 1024, SWZ);
                const uint64_t dk0 = smem_desc(smem_u32(sK), 16, 1024, SWZ);
                const uint64_t dv0 = smem_desc(smem_u32(sV), C::BOX_BYTES, 1024, SWZ);
                const uint32_t dq_lo = (uint32_t)dq0, dq_hi = (uint32_t)(dq0 >> 32);
                const uint32_t dk_lo = (uint32_t)dk0, dk_hi = (uint32_t)(dk0 >> 32);
                const uint32_t dv_lo = (uint32_t)dv0, dv_hi = (uint32_t)(dv0 >> 32);
                auto issue_qk = [&](int q, int slot) {
                    const uint32_t qa = dq_lo + (uint32_t)q * (C::TILE_BYTES >> 4);
                    const uint32_t ka = dk_lo + (uint32_t)slot * (C::TILE_BYTES >> 4);
                    const uint32_t tS = tmem_base + q * 128;
                    #pragma unroll
                    for (int ks = 0; ks < D / 16; ks++) {
                        const uint32_t off = ((uint32_t)((ks * 16) / C::BOXC) * C::BOX_BYTES + (uint32_t)((ks * 16) % C::BOXC) * 2u) >> 4;
                        tc_mma_ss_lh(tS, qa + off, dq_hi, ka + off, dk_hi, IDESC_QK, ks > 0 ? 1u : 0u);
                    }
                };
                auto issue_pv = [&](int q, int slot, uint32_t acc0, int half) {
                    const uint32_t va = dv_lo + (uint32_t)slot * (C::TILE_BYTES >> 4);
                    const uint32_t tS = tmem_base + q * 128, tO = tmem_base + 256 + q * 128;
                    #pragma unroll
                    for (int ks = half * 4; ks < half * 4 + 4; ks++)
                        tc_mma_ts_lh(tO, tS + ks * 8, va + ((ks * 16 * 128) >> 4), dv_hi, IDESC_PV, ks > 0 ? 1u : acc0);
                };
                bool ok = true;
                if (nblk_max > 0) {
                    ok = mbar_wait(&k_full[0], 0, &abort_word, 23);
                    for (int q = 0; q < 2 && ok; q++) {
                        if (nblk[q] > 0) {
                            ok = mbar_wait(&q_full[q], 0, &abort_word, 24);
                            if (!ok) break;
                            tc_fence_after_sync();
                            issue_qk(q, 0);
                            tc_commit(&s_full[q]);
                        }
                    }
                    if (ok) tc_commit(&k_empty[0]);
                }
                for (int j = 0; j < nblk_max && ok; j++) {
                    const int sv = j % NSV;
                    ok = mbar_wait(&v_full[sv], (uint32_t)((j / NSV) & 1), &abort_word, 25);
                    if (!ok) break;
                    bool k_next_ready = false;
                    for (int q = 0; q < 2 && ok; q++) {
                        if (j >= nblk[q]) continue;
                        ok = mbar_wait(&p_full[q][0], (uint32_t)(j & 1), &abort_word, 26);
                        if (!ok) break;
                        tc_fence_after_sync();
                        issue_pv(q, sv, j > 0 ? 1u : 0u, 0);
                        ok = mbar_wait(&p_full[q][1], (uint32_t)(j & 1), &abort_word, 29);
                        if (!ok) break;
                        tc_fence_after_sync();
                        issue_pv(q, sv, 1u, 1);
                        if (j + 1 < nblk[q]) {
                            const int sk = (j + 1) % NSK;
                            if (!k_next_ready) {
                                ok = mbar_wait(&k_full[sk], (uint32_t)(((j + 1) / NSK) & 1), &abort_word, 27);
                                if (!ok) break;
                                tc_fence_after_sync();
                                k_next_ready = true;
                            }
                            issue_qk(q, sk);
                            tc_commit(&s_full[q]);
                        } else {
                            tc_commit(&o_done[q]);
                        }
                    }
                    if (!ok) break;
                    tc_commit(&v_empty[sv]);
                    if (j + 1 < nblk_max) tc_commit(&k_empty[(j + 1) % NSK]);
                }
                // The last commit has to land before the barriers are rebuilt for the next work item.
                if (ok && nblk_max > 0)
                    mbar_wait(&v_empty[(nblk_max - 1) % NSV], (uint32_t)(((nblk_max - 1) / NSV) & 1), &abort_word, 28);
            }
            end_item();
            if (!PERSIST) break;
        }
    } else {
        setmaxnreg_inc_224();
        for (int round = 0; ; round++) {
            ItemInfo it;
            if (!fetch_item(round, it)) break;
            EFA_ITEM_LOCALS
            // =====================================================================================
            // Softmax warpgroups: tile q = warp / 4, row = thread index within the warpgroup
            // =====================================================================================
            const int q = warp >> 2;
            const int row = tid - q * WS_BM;
            const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
            const uint32_t tmem_S = tmem_base + q * 128 + lane_base;
            const uint32_t tmem_O = tmem_base + 256 + q * 128 + lane_base;
            const int my_rows = rows_q[q];
            const int my_nblk = nblk[q];
            const int my_abs0 = q_abs0[q];

            float m_ref = kNegInfW;     // exponent offset in use (a past row maximum), scaled by scale*log2(e)
            float m_true = kNegInfW;    // true running row maximum, same scaling
            float l_run = 0.f;          // running denominator relative to m_ref
            bool ok = true;

            for (int j = 0; j < my_nblk; j++) {
                const int kb = kv_lo + j * WS_BN;
                ok = __all_sync(0xffffffffu, mbar_wait(&s_full[q], (uint32_t)(j & 1), &abort_word, 31));
                if (!ok) break;
                tc_fence_after_sync();

                uint32_t su[4][32];
                #pragma unroll
                for (int c = 0; c < 4; c++) tmem_ld32(tmem_S + c * 32, su[c]);
                tmem_wait_ld();

                const bool need_mask = (kb + WS_BN > kv_hi) || (a.causal && kb + WS_BN - 1 > my_abs0);
                if (need_mask) {
                    int lim = kv_hi - 1 - kb;
                    if (a.causal) lim = min(lim, my_abs0 + row - kb);
                    #pragma unroll
                    for (int c = 0; c < 4; c++)
                        #pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (c * 32 + i > lim) su[c][i] = 0xff800000u;
                }

                // row maximum: four independent chains of three-input max (half the instructions of fmaxf)
                float mx0 = kNegInfW, mx1 = kNegInfW, mx2 = kNegInfW, mx3 = kNegInfW;
                #pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    mx0 = max3(mx0, __uint_as_float(su[0][i]), __uint_as_float(su[0][i + 1]));
                    mx1 = max3(mx1, __uint_as_float(su[1][i]), __uint_as_float(su[1][i + 1]));
                    mx2 = max3(mx2, __uint_as_float(su[2][i]), __uint_as_float(su[2][i + 1]));
                    mx3 = max3(mx3, __uint_as_float(su[3][i]), __uint_as_float(su[3][i + 1]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                m_true = fmaxf(m_true, mx * a.scale_log2e);

                // Move the exponent offset only when the maximum grew by more than the threshold.
                float alpha = 1.f;
                if (m_true - m_ref > kRescaleThreshold || m_ref == kNegInfW) {     // (-inf) - (-inf) is NaN: second test
                    const float m_new = m_true;
                    const float m_use = (m_new == kNegInfW) ? 0.f : m_new;
                    alpha = (m_ref == kNegInfW) ? 0.f : ex2(m_ref - m_use);
                    m_ref = m_new;
                }
                const float m_off = (m_ref == kNegInfW) ? 0.f : m_ref;

                // S(j) complete implies PV(j-1) of this tile complete (the tensor pipe runs in order), and no
                // part of PV(j) is issued before this thread's first arrival below: O may be rescaled here.
                if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                    #pragma unroll
                    for (int c = 0; c < D / 32; c++) {
                        uint32_t o[32];
                        tmem_ld32(tmem_O + c * 32, o);
                        tmem_wait_ld();
                        #pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tmem_O + c * 32, o);
                    }
                }

                // P is handed to the MMA warp in two halves of 64 keys: the first four k-steps of P*V run on
                // the tensor pipe while the exponentials of the second half are still being computed.
                const uint64_t scale2 = pack2(a.scale_log2e, a.scale_log2e), off2 = pack2(-m_off, -m_off);
                uint64_t psum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
                #pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t pk[16];
                    #pragma unroll
                    for (int i = 0; i < 16; i++) {
                        float x0, x1;
                        unpack2(fma2(pack2(__uint_as_float(su[c][2 * i]), __uint_as_float(su[c][2 * i + 1])), scale2, off2), x0, x1);
                        const float q0 = ex2(x0), q1 = ex2(x1);
                        psum2[i & 1] = add2(psum2[i & 1], pack2(q0, q1));
                        pk[i] = pack_f16x2(q0, q1);
                    }
                    tmem_st16(tmem_S + c * 16, pk);
                    if (c == 1 || c == 3) {
                        tmem_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive(&p_full[q][c >> 1]);
                    }
                }
                float ps0, ps1;
                {
                    float s0, s1, s2, s3;
                    unpack2(psum2[0], s0, s1);
                    unpack2(psum2[1], s2, s3);
                    ps0 = s0 + s2;
                    ps1 = s1 + s3;
                }
                l_run = l_run * alpha + (ps0 + ps1);
            }

            if (ok && my_nblk > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(&o_done[q], 0, &abort_word, 32));
                tc_fence_after_sync();
            }

            // ---- epilogue: this thread's row (warps take this branch as a whole: my_rows is 0, 64 or 128)
            if (ok && (warp & 3) * 32 < my_rows) {
                const size_t ld_o = (size_t)a.H_local * D;
                const size_t orow = (size_t)block_row0 + q * WS_BM + row;
                float mult;
                float*  dst32 = nullptr;
                __half* dst16 = nullptr;
                if (a.nsplit == 1) {
                    mult = 1.f / l_run;
                    if constexpr (OUT_F16) dst16 = a.O16 + orow * ld_o + (size_t)head * D;
                    else                   dst32 = a.O32 + orow * ld_o + (size_t)head * D;
                } else {
                    // partials are stored relative to the true row maximum
                    mult = (m_true == kNegInfW) ? 0.f : ex2(m_ref - m_true);
                    dst32 = a.O_part + ((size_t)split * a.part_rows + orow) * ld_o + (size_t)head * D;
                    const size_t s0 = ((size_t)split * a.part_rows + orow) * a.H_local + head;
                    a.m_part[s0] = m_true;
                    a.l_part[s0] = l_run * mult;
                }
                #pragma unroll
                for (int c = 0; c < D / 16; c++) {
                    uint32_t o[16];
                    if (my_nblk > 0) {
                        tmem_ld16(tmem_O + c * 16, o);
                        tmem_wait_ld();
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 16; i++) o[i] = 0u;
                    }
                    if (dst16) {
                        uint4 v0, v1;
                        v0.x = pack_f16x2(__uint_as_float(o[0]) * mult,  __uint_as_float(o[1]) * mult);
                        v0.y = pack_f16x2(__uint_as_float(o[2]) * mult,  __uint_as_float(o[3]) * mult);
                        v0.z = pack_f16x2(__uint_as_float(o[4]) * mult,  __uint_as_float(o[5]) * mult);
                        v0.w = pack_f16x2(__uint_as_float(o[6]) * mult,  __uint_as_float(o[7]) * mult);
                        v1.x = pack_f16x2(__uint_as_float(o[8]) * mult,  __uint_as_float(o[9]) * mult);
                        v1.y = pack_f16x2(__uint_as_float(o[10]) * mult, __uint_as_float(o[11]) * mult);
                        v1.z = pack_f16x2(__uint_as_float(o[12]) * mult, __uint_as_float(o[13]) * mult);
                        v1.w = pack_f16x2(__uint_as_float(o[14]) * mult, __uint_as_float(o[15]) * mult);
                        uint4* d = reinterpret_cast<uint4*>(dst16 + c * 16);
                        d[0] = v0;
                        d[1] = v1;
                    } else {
                        float4* d = reinterpret_cast<float4*>(dst32 + c * 16);
                        #pragma unroll
                        for (int qd = 0; qd < 4; qd++)
                            d[qd] = make_float4(__uint_as_float(o[4 * qd]) * mult, __uint_as_float(o[4 * qd + 1]) * mult,
                                                __uint_as_float(o[4 * qd + 2]) * mult, __uint_as_float(o[4 * qd + 3]) * mult);
                    }
                }

                // ---- completion signal: one count per finished 64-row block, after its rows are visible.
                // A 64-row block is two warps; the second of them to get here publishes the count.
                if (a.tile_counters != nullptr) {
                    if (a.counters_sys) __threadfence_system(); else __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        const int half = (warp & 3) >> 1;
                        if (atomicAdd(&half_done[q][half], 1) == 1) {
                            if (a.counters_sys) __threadfence_system(); else __threadfence();
                            atomicAdd(a.tile_counters + (block_row0 + q * WS_BM + half * 64) / a.tile_rows, 1);
                        }
                    }
                }
            }
            end_item();
            if (!PERSIST) break;
        }
    }
#undef EFA_ITEM_LOCALS
    __syncthreads();

    // ---- teardown
    if (abort_word != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(100000);
        if (tid == 0 && a.status != nullptr) {
            if (atomicCAS(a.status, 0, (int)KS_WAIT_TIMEOUT) == 0) {
                a.status[1] = s_item;
                a.status[2] = abort_word;
            }
        }
        __syncthreads();
    }
    if (warp == 9) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D, bool OUT_F16, bool PERSIST>
int launch_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaArgs& args,
              int reserve_sms, cudaStream_t stream)
{
    using C = WsCfg<D>;
    static bool configured[64] = {};
    int dev = 0;
    EFA_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        EFA_CUDA(cudaFuncSetAttribute(fa_fwd_ws_kernel<D, OUT_F16, PERSIST>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        configured[dev] = true;
    }
    const int items_x = args.H_local * args.nsplit;
    const int items_y = (args.q_rows + 2 * WS_BM - 1) / (2 * WS_BM);
    const int total = items_x * items_y;
    if (PERSIST) {
        int sms = 148;
        EFA_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        int ctas = sms - reserve_sms;
        if (ctas < 1) ctas = 1;
        if (ctas > total) ctas = total;
        int* counter = work_counter_slot();
        if (!counter) { set_error("no device memory for the work counter"); return 1; }
        EFA_CUDA(cudaMemsetAsync(counter, 0, sizeof(int), stream));
        fa_fwd_ws_kernel<D, OUT_F16, true><<<ctas, WS_THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, args, counter, items_x, total);
    } else {
        dim3 grid(items_x, items_y);
        fa_fwd_ws_kernel<D, OUT_F16, false><<<grid, WS_THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, args, nullptr, items_x, total);
    }
    EFA_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace

// Launch of the warp-specialised kernel; the caller has validated the arguments and built the maps.
// reserve_sms > 0 selects the persistent form with that many SMs left free.
int fa_forward_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaArgs& a,
                  int d_h, bool out_f16, int reserve_sms, cudaStream_t stream)
{
    const bool persist = reserve_sms > 0;
    if (d_h == 64) {
        if (persist) return out_f16 ? launch_ws<64, true, true>(tq, tk, tv, a, reserve_sms, stream) : launch_ws<64, false, true>(tq, tk, tv, a, reserve_sms, stream);
        return out_f16 ? launch_ws<64, true, false>(tq, tk, tv, a, 0, stream) : launch_ws<64, false, false>(tq, tk, tv, a, 0, stream);
    }
    if (d_h == 128) {
        if (persist) return out_f16 ? launch_ws<128, true, true>(tq, tk, tv, a, reserve_sms, stream) : launch_ws<128, false, true>(tq, tk, tv, a, reserve_sms, stream);
        return out_f16 ? launch_ws<128, true, false>(tq, tk, tv, a, 0, stream) : launch_ws<128, false, false>(tq, tk, tv, a, 0, stream);
    }
    set_error("fa_forward_ws: d_h=%d is not handled by the warp-specialised kernel", d_h);
    return 2;
}

int fa_ws_kv_box_rows() { return WS_BN; }


namespace {
template <class K> int touch_kernel(K kernel)
{
    cudaFuncAttributes attr;
    EFA_CUDA(cudaFuncGetAttributes(&attr, kernel));
    return 0;
}
}  // namespace

// Loads the code of every instantiation now. A kernel's first launch may otherwise have to wait for the device to go
// idle, which it never does while a stream sits in a front-end wait on a counter that is not coming.
int fa_ws_preload()
{
    return touch_kernel(fa_fwd_ws_kernel<64, true, false>) || touch_kernel(fa_fwd_ws_kernel<64, false, false>) ||
           touch_kernel(fa_fwd_ws_kernel<64, true, true>) || touch_kernel(fa_fwd_ws_kernel<64, false, true>) ||
           touch_kernel(fa_fwd_ws_kernel<128, true, false>) || touch_kernel(fa_fwd_ws_kernel<128, false, false>) ||
           touch_kernel(fa_fwd_ws_kernel<128, true, true>) || touch_kernel(fa_fwd_ws_kernel<128, false, true>);
}

}  // namespace efa
