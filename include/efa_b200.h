/* C ABI of the B200 (sm_100a) tensor-parallel attention block.
 *
 * The block is: head-sharded FlashAttention -> per-rank output projection -> sum AllReduce, with the
 * projection and reduction of each finished row tile started while attention is still running.
 * Every entry point takes plain pointers and sizes. Device pointers are CUDA device pointers of
 * the current device; `stream` arguments are cudaStream_t handles passed as void*.
 *
 * Unless stated otherwise a function returns 0 on success and a non-zero code on failure, in
 * which case efa_last_error() describes the failure (per thread). Nothing in this library falls
 * back to host arithmetic: without a usable sm_100 device the compute entry points fail.
 *
 * Each declaration cites the interface of eager-flash-attention (file:line within that project)
 * that it stands in for.
 */
#ifndef EFA_B200_H
#define EFA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EFA_ABI_VERSION 3

/* Element types of O / output buffers. */
#define EFA_F32 0
#define EFA_F16 1

int         efa_abi_version(void);
const char* efa_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Kernel launch interface
 * ------------------------------------------------------------------------------------------ */

/* Same fields, order and meaning as FlashAttnTCParams (flash_attn_tc.cuh:16-23). */
typedef struct efa_flash_params {
    int   S;
    int   d_h;      /* 16, 32, 64 or 128 */
    int   H_local;
    int   split;    /* split-KV factor (1 = off) */
    int   causal;
    float scale;    /* softmax scale, 1/sqrt(d_h) */
} efa_flash_params;

/* Same fields, order and meaning as FlashAttnTCPartials (flash_attn_tc.cuh:25-34):
 *   O_part [split][rows][H_local*d_h] unnormalised, m_part / l_part [split][rows][H_local],
 *   row max in the log2 domain and row denominator. */
typedef struct efa_flash_partials {
    float* O_part;
    float* m_part;
    float* l_part;
    int    rows;
} efa_flash_partials;

/* flash_attn_tc_forward (flash_attn_tc.cuh:45-50; kernel flash_attn_tc.cu:73-312).
 * Q, K, V: fp16 [H_local][S][d_h]. O: [q_rows][H_local*d_h], fp32 (EFA_F32, the reference's type)
 * or fp16 (EFA_F16, what the projection kernel consumes). Rows q_start .. q_start+q_rows.
 * With split > 1 the partials go to `part` and O is untouched until efa_flash_attn_tc_combine.
 * If tile_counters != NULL, tile_counters[(row within launch)/tile_rows] is incremented once per
 * finished 64-row block per (head, split) after that block's rows are visible device-wide
 * (__threadfence + atomicAdd, flash_attn_tc.cu:305-311). Asynchronous on `stream`. */
int efa_flash_attn_tc_forward(const void* Q, const void* K, const void* V,
                              void* O, int o_dtype, const efa_flash_partials* part,
                              int q_start, int q_rows, const efa_flash_params* p, void* stream,
                              int* tile_counters, int tile_rows);

/* flash_attn_tc_combine (flash_attn_tc.cuh:54-57; kernel flash_attn_tc.cu:319-361): merge the
 * split partials of workspace rows [row0, row0+rows) into O[0..rows). */
int efa_flash_attn_tc_combine(const efa_flash_partials* part, void* O, int o_dtype,
                              int row0, int rows, const efa_flash_params* p, void* stream);

/* Size of the fixed device array that efa_flash_attn_tc_forward_noalloc keeps its split-KV partials in. */
#define EFA_STATIC_SCRATCH_BYTES (8u << 20)

/* Attention for rows q_start .. q_start+q_rows with split-KV, partials and merge in one call, and
 * without any device allocation: not by the caller, not by this library. It has no counterpart in
 * the reference, whose callers always allocate the partials workspace themselves
 * (alloc_workspace). It is for callers that cannot get device memory when they call: a process
 * whose memory pool already owns the whole GPU, where a plain cudaMalloc fails, or a loop that
 * cannot afford the device-wide synchronisation an allocation implies.
 * The partials live in a fixed array of EFA_STATIC_SCRATCH_BYTES inside the library (every GPU that
 * loads the library holds that much until the process exits). The call is rejected, with a message
 * that names the sizes, when p->split * q_rows * (H_local*d_h + 2*H_local) * 4 exceeds it.
 * O: [q_rows][H_local*d_h] in o_dtype, written for every p->split >= 1. No tile counters.
 * The first call on a device looks up the array's device address and configures the kernel; make
 * that first call before any stream capture starts. All calls share the one array and it keeps
 * the previous call's contents (nothing in it needs clearing: each call writes every element it
 * later reads). Two calls that overlap on the GPU (different streams, or different host threads) race on it:
 * order them on one stream or with events. Kernels launched here do not report to
 * efa_kernel_status (its word is allocated memory) but to a word of their own inside the library, read with
 * efa_flash_attn_tc_noalloc_status. */
int efa_flash_attn_tc_forward_noalloc(const void* Q, const void* K, const void* V,
                                      void* O, int o_dtype, int q_start, int q_rows,
                                      const efa_flash_params* p, void* stream);

/* out4 = {code, block, site, 0} of the current device: code 0 = no kernel launched by
 * efa_flash_attn_tc_forward_noalloc gave up a bounded wait since the word was last cleared; reset != 0 clears
 * it after reading. A call whose kernel gave up leaves its output incomplete, so check after synchronising.
 * Synchronous copies from and to a symbol of the library; allocates nothing. Like the entry point it belongs
 * to, it has no counterpart in the reference. */
int efa_flash_attn_tc_noalloc_status(int* out4, int reset);

/* flash_attn_tc_check_params (flash_attn_tc.cuh:59-60, flash_attn_tc.cu:401-409):
 * NULL when the launch is legal, else a static description. */
const char* efa_flash_attn_tc_check_params(const efa_flash_params* p, int q_rows);

/* convert_f32_to_f16 (flash_attn_tc.cuh:62, flash_attn_tc.cu:411-424), round to nearest even. */
int efa_convert_f32_to_f16(const float* in, void* out, size_t n, void* stream);

/* project (attn_main.cuh:62-65, attn_main.cu:262-273) for the fp16 data path:
 * out[rows][d] = O_tile[rows][d_local] * W_O[d_local][d], fp16 operands, fp32 accumulate, fp16 out.
 * rows must be a multiple of 64, d_local a multiple of 16, d a multiple of 64. */
int efa_project_f16(const void* O_tile, const void* W_O, void* out,
                    int rows, int d_local, int d, void* stream);

/* compute_qkv (attn_main.cuh:30-31, attn_main.cu:127-153) on fp16 data, the step before the block:
 * per local head h, Q_h[S][d_h] = X[S][d] * W_q_h[d][d_h] (and K, V alike) with the projection kernel,
 * fp32 accumulate, written as fp16 head-major [H_local][S][d_h] directly (the reference computes in
 * fp32 with cuBLAS and converts in a second pass). X fp16 [S][d]; W_q/W_k/W_v fp16 [H_local][d][d_h].
 * d_h must be 64 or 128, S a multiple of 64, d a multiple of 16. Untimed in the reference. */
int efa_compute_qkv_f16(const void* X, const void* W_q, const void* W_k, const void* W_v,
                        void* Qh, void* Kh, void* Vh, int S, int d, int H_local, int d_h, void* stream);

/* Status word written by kernels whose bounded waits ran out: out4 = {code, block, site, 0};
 * code 0 = no kernel reported a problem since the last efa_kernel_status_reset(). */
int efa_kernel_status(int* out4);
int efa_kernel_status_reset(void);

/* ------------------------------------------------------------------------------------------
 * Runtime interface
 * ------------------------------------------------------------------------------------------ */

/* Execution modes, same numbering and names as RunMode (run_drivers.cuh:6-17, run_drivers.cu:9-11). */
enum {
    EFA_MODE_ATTN = 0, EFA_MODE_ATTN_TILED = 1, EFA_MODE_MEGATRON = 2, EFA_MODE_SYNC = 3,
    EFA_MODE_OVERLAP = 4, EFA_MODE_STREAM = 5, EFA_MODE_COMM = 6, EFA_MODE_COUNT = 7
};
const char* efa_mode_name(int mode);     /* mode_name  (run_drivers.cuh:19) */
int         efa_parse_mode(const char* s); /* parse_mode (run_drivers.cuh:20), -1 if unknown */

/* How the per-tile partial sums are reduced across ranks (allreduce, run_drivers.cu:26-30).
 *   NCCL: ncclAllReduce on communicator t % ncomm as the reference does, on the fp32 accumulators (ncclFloat) with one
 *         conversion into the fp16 output afterwards; ncclHalf with wire = EFA_WIRE_F16 (NCCL then adds fp16 in fp16,
 *         one rounding per hop).
 *   P2P:  stream mode only: one persistent kernel does projection and reduction over peer-mapped memory.
 *   NVLS: the NVSwitch sums the ranks' partial sums (fp32; or fp16 with fp32 accumulation, one rounding) through an NVLink
 *         multicast object; one small kernel per reduction on the communication stream. Needs a device and fabric
 *         with multicast support; otherwise the call fails with a message (nothing falls back silently).
 *   PULL: every rank fetches its share of all ranks' fp32 partial sums over peer mappings with bulk asynchronous
 *         copies, adds them in rank order, rounds once and multicasts the fp16 result through the switch. More
 *         bytes per link than NVLS ((R-1)/R of the partial sums inbound instead of 1/R) for far fewer thread
 *         blocks taken from the attention kernel. Same requirements as NVLS, plus CUDA IPC between the ranks. */
enum { EFA_REDUCE_NCCL = 0, EFA_REDUCE_P2P = 1, EFA_REDUCE_NVLS = 2, EFA_REDUCE_PULL = 3 };

enum { EFA_WIRE_AUTO = 0, EFA_WIRE_F16 = 1, EFA_WIRE_F32 = 2 };

/* Order in which stream mode takes the rows of a causal problem (row_order). */
enum { EFA_ROWS_AUTO = 0, EFA_ROWS_ASCENDING = 1, EFA_ROWS_DESCENDING = 2, EFA_ROWS_MIXED = 3 };

/* Derived problem description: AttnParams (attn_defs.cuh:70-84) without the fields of the
 * removed legacy kernel (B_M, B_N, kernel, flash). */
typedef struct efa_params {
    int S, d, H, R;
    int H_local, d_h, d_local;
    int tile, num_tiles;
    int nbuf, split, causal;
    int skip_proj, skip_comm;
    int reduce;                 /* EFA_REDUCE_* */
    int group_tiles;            /* stream mode, NCCL reduction: consecutive tiles handled by one projection +
                                   AllReduce launch (each tile's counter is still waited on). 1 = the reference's
                                   per-tile schedule; 0 = automatic (about S/8 rows per launch). */
    int proj_f32;               /* 0 (default): the projection rounds its fp32 accumulator to fp16, the reduction sums
                                   fp16 and `output` is fp16. 1: partial sums, reduction and `output` are fp32 — the
                                   reference's types (attn_main.cu:262-273, run_drivers.cu:26-30), whose own --proj switch
                                   chose fp32 or tf32 math (attn_bench.cu:55,113-117). Operands stay fp16 either way.
                                   NCCL reduction only; not with a residual or the host-buffer entry point. */
    int row_order;              /* stream mode: EFA_ROWS_ASCENDING = tiles complete first to last, the reference's order
                                   (flash_attn_tc.cu:100-103). EFA_ROWS_DESCENDING = last rows first: under a causal mask the
                                   last rows sweep the most keys, so the launch then ends on its shortest work items and
                                   the consumer waits for the tiles in that same order; but the rows then complete slowly at first and in
                                   a rush at the end. EFA_ROWS_MIXED (causal, strict row order) = two blocks from the end, one
                                   from the start, and so on: rows complete at a steady rate from both ends and the launch
                                   still ends on middle-weight items. AUTO = descending for a causal problem on one rank,
                                   else ascending. */
    int reduce_ctas;            /* thread blocks of the persistent kernel (P2P), 0 = chosen from the FLOP shares */
    int band_rows;              /* stream mode: rows within which the attention kernel may take its work head by head
                                   instead of in strict row order (K/V reuse in L2); 0 = chosen by efa_stream_plan,
                                   -1 = strict row order */
    int reserve_sms;            /* stream mode, diagnostics: > 0 runs the attention kernel in its persistent form and
                                   leaves that many SMs without an attention CTA */
    int trace;                  /* stream mode, diagnostics: 1 prints the timeline of the groups on stderr */
    int wire;                   /* element type of the partial sums that cross the links (NCCL and NVLS reductions):
                                   EFA_WIRE_F16 = the projection rounds its accumulator to fp16 and the reduction sums those
                                   (fp32 accumulation in the NVSwitch; one fp16 rounding per hop in NCCL) - half the bytes,
                                   and an error of up to half an fp16 ulp of every partial sum on top of the final rounding;
                                   EFA_WIRE_F32 = the fp32 accumulators are summed (the reference's types, run_drivers.cu:26-30)
                                   and the sum is rounded once into the fp16 output. EFA_WIRE_AUTO = fp32. */
    int debug_target_bias;      /* test hook, 0 in normal use: added on the HOST to the counter target that stream mode's
                                   consumers wait for (the cuStreamWaitValue32 of the projection stream, the polling of
                                   the persistent kernel), so that a guarded wait runs out and its recovery can be
                                   tested without any fault on the GPU */
    efa_flash_params flash_tc;
} efa_params;

/* make_params (attn_main.cuh:18-19, attn_main.cu:35-60). */
int efa_make_params(efa_params* out, int S, int d, int H, int tile, int nbuf, int split, int causal, int world_size);
/* attn_check_params (attn_main.cuh:22, attn_main.cu:62-74): NULL if runnable. */
const char* efa_attn_check_params(const efa_params* p);
/* blocks_per_tile (attn_main.cuh:68, attn_main.cu:275-280): the counter target of a tile. */
int efa_blocks_per_tile(const efa_params* p);

/* The launch plan of stream mode (the loop of run_stream, run_drivers.cu:227-240, which there is one tile per
 * iteration): consecutive tiles [first_tile, first_tile + ntiles) share one projection launch and one reduction
 * after a cuStreamWaitValue32 on each of their counters. Groups are returned in the order in which they are
 * waited for: first to last rows, (*descending = 1) last to first, or for EFA_ROWS_MIXED (S/16 rows per group) in the
 * order in which a list schedule of the work items on the device's SMs completes them.
 * group_tiles > 0: groups of that many tiles (1 = the reference's schedule). group_tiles == 0: about S/8
 * rows per group and the eighth that completes last cut into S/16, S/32, S/32, so that what remains after the
 * attention kernel ends is small. *band_rows (if not NULL): the band within which the attention kernel may take
 * its work head by head instead of in strict row order, 0 = strict order: bands are used when the K and V of all
 * local heads exceed what the L2 holds, and never exceed the smallest group. Host arithmetic only.
 * Returns the number of groups (groups may be NULL to count them), -1 on error. */
typedef struct efa_stream_group { int first_tile, ntiles; } efa_stream_group;
int efa_stream_plan(const efa_params* p, efa_stream_group* groups, int capacity, int* band_rows, int* descending);
/* The order in which stream mode's attention launch takes its 256-row blocks when it is neither first-to-last nor
 * last-to-first (EFA_ROWS_MIXED): blocks[k] = index of the block taken k-th. Returns the number of blocks, 0 when the
 * order of `p` is one of the two plain ones, -1 on error. Host arithmetic only. */
int efa_stream_row_blocks(const efa_params* p, short* blocks, int capacity);

/* Host control plane of one rank. The reference uses MPI for exactly these four operations
 * (MPI_Barrier / MPI_Allreduce(MAX) / MPI_Bcast / and, new here, an all-gather of opaque bytes for
 * IPC handles); a caller supplies them over whatever it has (the bundled shared-memory shim, or
 * torch.distributed). Callbacks return 0 on success. With size == 1 they may be NULL. */
typedef struct efa_world {
    void* user;
    int   rank, size;
    int   local_device;   /* CUDA device ordinal of this rank */
    int (*barrier)(void* user);
    int (*allreduce_max_f64)(void* user, double* value);
    int (*bcast_bytes)(void* user, void* buf, size_t n, int root);
    int (*allgather_bytes)(void* user, const void* in, void* out, size_t n_each);
} efa_world;

/* Runs each callback of a world once (barrier, max, broadcast, all-gather) and checks that the
 * results agree with rank and size. Host only, no CUDA call. The reference has no counterpart: it
 * is a set-up check for callers that bring their own control plane in place of MPI
 * (MPI_Barrier / MPI_Allreduce / MPI_Bcast at run_drivers.cu:38-44, attn_main.cu:155-163). */
int efa_world_selftest(const efa_world* world);

typedef struct efa_ctx efa_ctx;   /* RunCtx (attn_defs.cuh:86-99): streams, communicators */

/* make_ctx / destroy_ctx (attn_main.cuh:43-44, attn_main.cu:180-213): one compute stream (lowest
 * priority), one projection stream and ncomm communication streams (highest priority when
 * `prioritize`), ncomm NCCL communicators over the world's ranks. Collective over the world. */
int efa_make_ctx(efa_ctx** out, const efa_world* world, int ncomm, int prioritize);
int efa_destroy_ctx(efa_ctx* ctx);

/* Output buffer for efa_run_mode with EFA_REDUCE_NVLS that the reduction can write in place: a pointer into this
 * rank's memory of the context's multicast region (fp16 [S][d]; valid until the context is destroyed or a larger
 * problem makes the region grow). The switch stores the reduced rows straight into every rank's buffer. With any
 * other output pointer the reduced rows are copied there from the region by one device-to-device copy per
 * reduction. Collective (it may create the region). The reference's callers allocate the output themselves
 * (attn_bench.cu:135-136); this is the counterpart of NCCL's registered user buffers and has none there. */
int efa_nvls_output(efa_ctx* ctx, const efa_params* p, void** output);

/* Limits of the waits that guard against a signal that never comes (the reference has none: a wrong counter
 * target blocks its cuStreamWaitValue32 forever, run_drivers.cu:228-230). device_ms: how long a kernel of this
 * context polls a tile counter, a peer's arrival flag or a barrier flag before it records a status
 * (efa_kernel_status) and returns; default 10 s. host_ms: how long efa_run_mode waits for a stream before it
 * releases the pending counter waits and returns an error; default 120 s. A value <= 0 leaves a limit as it is. */
int efa_ctx_set_wait_limit_ms(efa_ctx* ctx, double device_ms, double host_ms);

/* Device tensors of one rank: Weights (attn_main.cuh:7-12) for the fp16 data path. */
typedef struct efa_weights {
    void* Qh; void* Kh; void* Vh;   /* fp16 [H_local][S][d_h] */
    void* W_O;                      /* fp16 [d_local][d] */
} efa_weights;

/* Synthetic inputs on the HOST (fp16 bit patterns), written into caller-provided buffers:
 *   recipe 0 ("ref"):    allocate_and_fill + compute_qkv (attn_main.cu:88-153): glibc rand(),
 *                        X = U(-1,1) seeded `seed`, weights seeded seed*31+rank+1, Q/K/V = X*W in
 *                        fp32 then rounded to fp16; W_O rounded to fp16.
 *   recipe 1 ("normal"): Q, K, V ~ N(0,1), W_O ~ N(0, 1/d), keyed by (seed, tensor, global head, row,
 *                        column) so that every rank count yields the same global tensors.
 * Sizes: Q/K/V H_local*S*d_h halves each, W_O d_local*d halves. */
int efa_fill_host_inputs(const efa_params* p, int rank, int seed, int recipe,
                         uint16_t* Qh, uint16_t* Kh, uint16_t* Vh, uint16_t* W_O);

/* Timing record of one efa_run_mode call. */
typedef struct efa_run_stats {
    double wall_ms;        /* barrier -> enqueue -> sync, max over ranks (run_drivers.cu:38-44) */
    float  attn_kernel_ms; /* CUDA-event time of the attention kernel on the compute stream, this rank */
    float  proj_ms;        /* CUDA-event time of the projection kernel (megatron mode), this rank, else 0 */
    int    kernel_launches;/* kernels of this library launched inside the timed region, this rank */
} efa_run_stats;

/* run_mode (run_drivers.cuh:22-26, run_drivers.cu:277-292). `output`: fp16 [S][d] device buffer (fp32 when
 * p->proj_f32), the reduced result, identical on every rank (untouched by attn / attn_tiled). Collective. */
int efa_run_mode(efa_ctx* ctx, int mode, const efa_weights* w, void* output,
                 const efa_params* p, efa_run_stats* stats);

/* The block followed by the first step after it: output = residual + (reduced projection), with the
 * residual (fp16 [S][d] device buffer, same on every rank) added to each reduced group of rows on the
 * stream that reduced it, as soon as it has landed — per tile group in stream / overlap / sync mode, once in
 * megatron mode, after the persistent kernel with the fused reduction. One fp16 rounding on top of
 * efa_run_mode's result. The reference stops at the AllReduce output buffer (run_drivers.cuh:22-24,
 * run_drivers.cu:26-30), so this has no counterpart there. Rejected for attn, attn_tiled and comm
 * (no block output) and with skip_proj / skip_comm. Collective. */
int efa_run_mode_residual(efa_ctx* ctx, int mode, const efa_weights* w, const void* residual, void* output,
                          const efa_params* p, efa_run_stats* stats);

/* The whole block on HOST buffers: copies this rank's fp16 Q/K/V/W_O to the device, runs `mode`,
 * copies the fp16 [S][d] result back. The copies are inside wall_ms. Buffers should be pinned.
 * Device staging is allocated on the first call for a given shape and reused. In stream mode with a
 * causal mask (NCCL or NVLS reduction) the work is pipelined over row chunks: rows of chunk c
 * need only the keys of chunks 0..c, so the copy-in of the next chunk, the attention / projection /
 * AllReduce of this one and the copy-out of the previous one overlap. */
int efa_run_mode_host(efa_ctx* ctx, int mode,
                      const uint16_t* Qh, const uint16_t* Kh, const uint16_t* Vh, const uint16_t* W_O,
                      uint16_t* output, const efa_params* p, efa_run_stats* stats);

/* The same, but only rows [out_row0, out_row0 + out_rows) of the result are copied back, into `output` (which
 * holds just those rows; NULL or out_rows == 0: nothing is copied back). The reduced result is the same on every
 * rank, so with several ranks each can bring back its own share of the rows over its own PCIe link
 * instead of one rank bringing back all of them. Like efa_run_mode_host it has no counterpart in the reference,
 * whose timed region never leaves the device (run_drivers.cu:218-245). */
int efa_run_mode_host_rows(efa_ctx* ctx, int mode,
                           const uint16_t* Qh, const uint16_t* Kh, const uint16_t* Vh, const uint16_t* W_O,
                           uint16_t* output, int out_row0, int out_rows, const efa_params* p, efa_run_stats* stats);

#ifdef __cplusplus
}
#endif
#endif /* EFA_B200_H */
