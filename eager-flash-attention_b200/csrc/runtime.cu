// Problem description, rank context and synthetic inputs.
// Counterpart of make_params / attn_check_params / make_ctx / destroy_ctx / allocate_and_fill /
// compute_qkv / blocks_per_tile of eager-flash-attention (attn_main.cu:35-74, 88-153, 180-213, 275-280).
#include "runtime.h"

#include "fa_fwd_sm100.cuh"
#include "host_util.h"
#include "nccl_dyn.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace efa {

// Load the code of every kernel of the library on the current device (one function per translation unit).
int fa_preload(); int proj_preload(); int p2p_preload(); int nvls_preload(); int modes_preload();

int world_barrier(const efa_world& w)
{
    if (w.size <= 1 || !w.barrier) return 0;
    if (w.barrier(w.user)) { set_error("world barrier failed"); return 1; }
    return 0;
}

int world_max(const efa_world& w, double* v)
{
    if (w.size <= 1 || !w.allreduce_max_f64) return 0;
    if (w.allreduce_max_f64(w.user, v)) { set_error("world allreduce(max) failed"); return 1; }
    return 0;
}

int ensure_bytes(void** ptr, size_t* have, size_t want)
{
    if (*have >= want && *ptr) return 0;
    if (*ptr) { EFA_CUDA(cudaFree(*ptr)); *ptr = nullptr; *have = 0; }
    EFA_CUDA(cudaMalloc(ptr, want));
    *have = want;
    return 0;
}

int ensure_events(efa_ctx* c, size_t n)
{
    while (c->events.size() < n) {
        cudaEvent_t e;
        EFA_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        c->events.push_back(e);
    }
    return 0;
}

int ensure_trace_events(efa_ctx* c, size_t n)
{
    while (c->trace_events.size() < n) {
        cudaEvent_t e;
        EFA_CUDA(cudaEventCreate(&e));
        c->trace_events.push_back(e);
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Synthetic inputs
// ---------------------------------------------------------------------------------------------
namespace {

inline uint16_t f2h(float x)
{
    __half h = __float2half_rn(x);
    uint16_t u;
    std::memcpy(&u, &h, 2);
    return u;
}

// glibc rand() stream, U(-1, 1) * scale: the exact expression of rand_fill (attn_main.cu:88-96).
void rand_fill_host(float* dst, size_t n, float scale)
{
    for (size_t i = 0; i < n; i++)
        dst[i] = scale * (2.0f * (float)rand() / RAND_MAX - 1.0f);
}

template <class F>
void parallel_for(int n, F f)
{
    unsigned nt = std::max(1u, std::min((unsigned)n, std::thread::hardware_concurrency()));
    if (nt == 1) { for (int i = 0; i < n; i++) f(i); return; }
    std::vector<std::thread> th;
    for (unsigned t = 0; t < nt; t++)
        th.emplace_back([=]() { for (int i = (int)t; i < n; i += (int)nt) f(i); });
    for (auto& x : th) x.join();
}

// out[S][n] (as fp16) = X[S][d] * Wt[d][n] in fp32, rows in parallel.
void qkv_host(const float* X, const float* W, int S, int d, int n, uint16_t* out)
{
    parallel_for(S, [&](int s) {
        std::vector<float> acc(n);
        std::fill(acc.begin(), acc.end(), 0.f);
        const float* x = X + (size_t)s * d;
        for (int k = 0; k < d; k++) {
            const float xv = x[k];
            const float* wr = W + (size_t)k * n;
            for (int j = 0; j < n; j++) acc[j] += xv * wr[j];
        }
        for (int j = 0; j < n; j++) out[(size_t)s * n + j] = f2h(acc[j]);
    });
}

inline uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Two independent N(0,1) samples from one 64-bit key (Box-Muller on two 32-bit uniforms).
inline void normal_pair(uint64_t key, float* a, float* b)
{
    const uint64_t h = splitmix64(key);
    const double u1 = ((double)(uint32_t)(h >> 32) + 1.0) * (1.0 / 4294967296.0);   // (0, 1]
    const double u2 = (double)(uint32_t)h * (1.0 / 4294967296.0);                    // [0, 1)
    const double r = std::sqrt(-2.0 * std::log(u1));
    const double t = 6.283185307179586476925 * u2;
    *a = (float)(r * std::cos(t));
    *b = (float)(r * std::sin(t));
}

inline uint64_t normal_key(int seed, int tensor, int a, int b, int pair)
{
    uint64_t k = splitmix64((uint64_t)(uint32_t)seed * 0x100000001B3ull + (uint64_t)tensor);
    k = splitmix64(k ^ ((uint64_t)(uint32_t)a << 32 | (uint32_t)b));
    return k ^ (uint64_t)(uint32_t)pair;
}

}  // namespace

}  // namespace efa

using namespace efa;

extern "C" int efa_fill_host_inputs(const efa_params* p, int rank, int seed, int recipe,
                                    uint16_t* Qh, uint16_t* Kh, uint16_t* Vh, uint16_t* W_O)
{
    if (!p || !Qh || !Kh || !Vh || !W_O) { set_error("efa_fill_host_inputs: null argument"); return 2; }
    const int S = p->S, d = p->d, H_local = p->H_local, d_h = p->d_h, d_local = p->d_local;
    if (recipe == 0) {
        // X seeded with `seed`, identical on all ranks; weights seeded seed*31+rank+1, rank-specific;
        // fill order X, W_q, W_k, W_v, W_O with scales 1, 0.15, 0.15, 0.10, 0.05.
        std::vector<float> X((size_t)S * d);
        const size_t wn = (size_t)H_local * d * d_h;
        std::vector<float> Wq(wn), Wk(wn), Wv(wn), Wo((size_t)d_local * d);
        srand(seed);
        rand_fill_host(X.data(), X.size(), 1.0f);
        srand(seed * 31 + rank + 1);
        rand_fill_host(Wq.data(), wn, 0.15f);
        rand_fill_host(Wk.data(), wn, 0.15f);
        rand_fill_host(Wv.data(), wn, 0.10f);
        rand_fill_host(Wo.data(), Wo.size(), 0.05f);
        // Per head h: Q_h[S][d_h] = X[S][d] * W_q_h[d][d_h], then round to fp16 (compute_qkv).
        for (int h = 0; h < H_local; h++) {
            const size_t wo = (size_t)h * d * d_h, qo = (size_t)h * S * d_h;
            qkv_host(X.data(), Wq.data() + wo, S, d, d_h, Qh + qo);
            qkv_host(X.data(), Wk.data() + wo, S, d, d_h, Kh + qo);
            qkv_host(X.data(), Wv.data() + wo, S, d, d_h, Vh + qo);
        }
        for (size_t i = 0; i < Wo.size(); i++) W_O[i] = f2h(Wo[i]);
        return 0;
    }
    if (recipe == 1) {
        if (d_h % 2 != 0 || d % 2 != 0) { set_error("efa_fill_host_inputs: odd sizes"); return 2; }
        uint16_t* dst[3] = {Qh, Kh, Vh};
        for (int t = 0; t < 3; t++) {
            uint16_t* out = dst[t];
            parallel_for(H_local * S, [&, out, t](int hs) {
                const int h = hs / S, s = hs % S;
                const int gh = rank * H_local + h;
                uint16_t* row = out + ((size_t)h * S + s) * d_h;
                for (int j = 0; j < d_h; j += 2) {
                    float a, b;
                    normal_pair(normal_key(seed, t, gh, s, j >> 1), &a, &b);
                    row[j] = f2h(a);
                    row[j + 1] = f2h(b);
                }
            });
        }
        const float sigma = 1.0f / std::sqrt((float)d);
        parallel_for(d_local, [&](int r) {
            const int gr = rank * d_local + r;
            uint16_t* row = W_O + (size_t)r * d;
            for (int j = 0; j < d; j += 2) {
                float a, b;
                normal_pair(normal_key(seed, 3, gr, 0, j >> 1), &a, &b);
                row[j] = f2h(a * sigma);
                row[j + 1] = f2h(b * sigma);
            }
        });
        return 0;
    }
    set_error("efa_fill_host_inputs: unknown recipe %d", recipe);
    return 2;
}

extern "C" int efa_make_params(efa_params* out, int S, int d, int H, int tile, int nbuf, int split, int causal, int world_size)
{
    if (!out) { set_error("efa_make_params: null output"); return 2; }
    efa_params p;
    std::memset(&p, 0, sizeof(p));
    p.S = S; p.d = d; p.H = H; p.R = world_size;
    p.H_local = (world_size > 0) ? H / world_size : 0;
    p.d_h = (H > 0) ? d / H : 0;
    p.d_local = p.H_local * p.d_h;
    p.tile = tile;
    p.num_tiles = (tile > 0) ? S / tile : 0;
    p.nbuf = nbuf; p.split = split; p.causal = causal;
    p.skip_proj = 0; p.skip_comm = 0;
    p.reduce = EFA_REDUCE_NCCL;
    p.group_tiles = 0;
    p.proj_f32 = 0;
    p.row_order = EFA_ROWS_AUTO;
    p.reduce_ctas = 0; p.band_rows = 0; p.reserve_sms = 0; p.trace = 0; p.wire = EFA_WIRE_AUTO; p.debug_target_bias = 0;
    const float scale = p.d_h > 0 ? 1.0f / sqrtf((float)p.d_h) : 0.f;
    p.flash_tc = efa_flash_params{S, p.d_h, p.H_local, split, causal, scale};
    *out = p;
    return 0;
}

extern "C" const char* efa_attn_check_params(const efa_params* p)
{
    if (!p) return "null params";
    if (p->R <= 0 || p->H <= 0 || p->H % p->R != 0) return "H must be divisible by the number of ranks";
    if (p->d % p->H != 0) return "d must be divisible by H";
    if (p->tile <= 0 || p->S % p->tile != 0) return "S must be a multiple of tile";
    if (p->nbuf < 1) return "nbuf must be >= 1";
    if (p->d % 64 != 0) return "d must be a multiple of 64";
    return fa_check_params(p->flash_tc, p->tile);
}

extern "C" int efa_blocks_per_tile(const efa_params* p)
{
    // One count per finished 64-row block per (head, split).
    return (p->tile / 64) * p->H_local * p->split;
}

namespace {

// EFA_ROWS_MIXED applies to a causal problem in strict row order (no bands): otherwise it is first-to-last.
bool mixed_order(const efa_params* p)
{
    if (p->row_order != EFA_ROWS_MIXED || !p->causal || p->band_rows > 0) return false;
    const double kv_bytes = 2.0 * (double)p->H_local * p->S * p->d_h * 2.0;
    return kv_bytes <= 80e6 || p->band_rows < 0;
}

// Two 256-row blocks from the end, one from the start, and so on.
int mixed_blocks(const efa_params* p, std::vector<short>& order)
{
    const int nb = (p->S + 255) / 256;
    order.clear();
    int lo = 0, hi = nb - 1;
    while (lo <= hi) {
        for (int k = 0; k < 2 && hi >= lo; k++) order.push_back((short)hi--);
        if (lo <= hi) order.push_back((short)lo++);
    }
    return nb;
}

}  // namespace

extern "C" int efa_stream_row_blocks(const efa_params* p, short* blocks, int capacity)
{
    if (!p || p->S <= 0) { set_error("efa_stream_row_blocks: invalid params"); return -1; }
    if (!mixed_order(p)) return 0;
    std::vector<short> order;
    const int nb = mixed_blocks(p, order);
    if (nb > 32767) { set_error("efa_stream_row_blocks: too many row blocks"); return -1; }
    if (blocks) {
        if (capacity < nb) { set_error("efa_stream_row_blocks: %d blocks, room for %d", nb, capacity); return -1; }
        std::copy(order.begin(), order.end(), blocks);
    }
    return nb;
}

extern "C" int efa_stream_plan(const efa_params* p, efa_stream_group* groups, int capacity, int* band_rows, int* descending)
{
    if (!p || p->tile <= 0 || p->num_tiles <= 0) { set_error("efa_stream_plan: invalid params"); return -1; }
    const bool mixed = mixed_order(p);
    // AUTO: last rows first only where nothing has to be hidden behind the attention kernel (one rank): rows then
    // complete slowly at first and in a rush at the end, which is the wrong way round for a reduction that has to
    // keep up; with several ranks the first rows go first, as in the reference.
    const bool desc = !mixed && (p->row_order == EFA_ROWS_DESCENDING || (p->row_order == EFA_ROWS_AUTO && p->causal && p->R == 1));
    if (descending) *descending = desc ? 1 : 0;
    const bool auto_groups = p->group_tiles <= 0;
    int gt = p->group_tiles;
    if (auto_groups) { gt = (p->S / (mixed ? 16 : 8)) / p->tile; if (gt < 1) gt = 1; }
    if (gt > p->num_tiles) gt = p->num_tiles;
    int n = 0, smallest = p->num_tiles;
    // Laid out over positions 0 .. num_tiles: position x is tile x, or tile num_tiles - 1 - x (descending).
    for (int t0 = 0; t0 < p->num_tiles; n++) {
        int nt = (t0 + gt <= p->num_tiles) ? gt : p->num_tiles - t0;
        if (auto_groups && !mixed && gt >= 4 && t0 + gt >= p->num_tiles) {
            // the eighth that completes last: S/16, S/32, S/32 rows
            const int left = p->num_tiles - t0;
            nt = (left > gt / 2) ? gt / 2 : (left > gt / 4 ? left - gt / 4 : left);
            if (nt < 1) nt = left;
        }
        if (groups) {
            if (n >= capacity) { set_error("efa_stream_plan: more than %d groups", capacity); return -1; }
            groups[n].first_tile = desc ? p->num_tiles - t0 - nt : t0;
            groups[n].ntiles = nt;
        }
        if (nt < smallest) smallest = nt;
        t0 += nt;
    }
    if (mixed && groups) {
        // Order the groups as a list schedule of the work items completes them: items (one per 256-row block, head
        // and split) go to the SM that is free first, in dispatch order, and cost their number of key stages.
        std::vector<short> order;
        const int nb = mixed_blocks(p, order);
        const int per_block = p->H_local * p->split, sms = 148;
        std::vector<double> free_at(sms, 0.0), done(nb, 0.0);
        for (int k = 0; k < nb; k++) {
            const int y = order[k];
            for (int i = 0; i < per_block; i++) {
                auto it = std::min_element(free_at.begin(), free_at.end());
                *it += 2.0 * (y + 1) / p->split + 3.0;
                done[y] = std::max(done[y], *it);
            }
        }
        std::vector<std::pair<double, int>> key(n);
        for (int g = 0; g < n; g++) {
            const int r0 = groups[g].first_tile * p->tile, r1 = (groups[g].first_tile + groups[g].ntiles) * p->tile;
            double t = 0.0;
            for (int y = r0 / 256; y <= (r1 - 1) / 256 && y < nb; y++) t = std::max(t, done[y]);
            key[g] = {t, g};
        }
        std::sort(key.begin(), key.end());
        std::vector<efa_stream_group> sorted(n);
        for (int g = 0; g < n; g++) sorted[g] = groups[key[g].second];
        std::copy(sorted.begin(), sorted.end(), groups);
    }
    if (band_rows) {
        // Rows only have to complete group by group, so the attention kernel may order its work in bands no longer
        // than the smallest group (whole 256-row blocks, at most 2048 rows, none below 512). Bands exist for the L2:
        // in strict row order every local head's K and V are live at once; when they fit in the L2 anyway (half of
        // it is assumed to be available to them) there is nothing to gain and strict order is kept.
        int b = smallest * p->tile;
        if (auto_groups && b < p->S / 16) b = p->S / 16;      // the two smallest groups may complete together
        b = (b / 256) * 256;
        if (b > 2048) b = 2048;
        if (b < 512) b = 0;
        const double kv_bytes = 2.0 * (double)p->H_local * p->S * p->d_h * 2.0;
        if (kv_bytes <= 80e6) b = 0;
        if (p->band_rows > 0) b = (p->band_rows / 256) * 256;
        if (p->band_rows < 0 || mixed) b = 0;
        *band_rows = b;
    }
    return n;
}

extern "C" int efa_make_ctx(efa_ctx** out, const efa_world* world, int ncomm, int prioritize)
{
    if (!out || !world) { set_error("efa_make_ctx: null argument"); return 2; }
    if (ncomm < 1 || ncomm > EFA_MAX_COMM) { set_error("ncomm must be in [1, %d]", EFA_MAX_COMM); return 2; }
    if (world->size > 1 && (!world->barrier || !world->allreduce_max_f64 || !world->bcast_bytes)) {
        set_error("efa_make_ctx: a world of %d ranks needs barrier, allreduce_max_f64 and bcast_bytes", world->size);
        return 2;
    }
    EFA_CUDA(cudaSetDevice(world->local_device));
    cudaDeviceProp prop;
    EFA_CUDA(cudaGetDeviceProperties(&prop, world->local_device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library contains sm_100a code only", world->local_device, prop.major, prop.minor);
        return 3;
    }
    const NcclApi* nccl = nccl_api();
    if (!nccl) return 1;
    efa_ctx* c = new efa_ctx();
    c->world = *world;
    int lo = 0, hi = 0;   // numerically lower = higher priority
    EFA_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    const int side = prioritize ? hi : lo;
    EFA_CUDA(cudaStreamCreateWithPriority(&c->compute_stream, cudaStreamNonBlocking, lo));
    EFA_CUDA(cudaStreamCreateWithPriority(&c->proj_stream, cudaStreamNonBlocking, side));
    c->ncomm = ncomm;
    for (int i = 0; i < ncomm; i++) {
        EFA_CUDA(cudaStreamCreateWithPriority(&c->comm_streams[i], cudaStreamNonBlocking, side));
        ncclUniqueId id;
        std::memset(&id, 0, sizeof(id));
        if (world->rank == 0) {
            ncclResult_t r = nccl->GetUniqueId(&id);
            if (r != ncclSuccess) { set_error("ncclGetUniqueId: %s", nccl->GetErrorString(r)); return 1; }
        }
        if (world->size > 1 && world->bcast_bytes(world->user, &id, sizeof(id), 0)) {
            set_error("efa_make_ctx: broadcast of the NCCL id failed");
            return 1;
        }
        ncclResult_t r = nccl->CommInitRank(&c->nccls[i], world->size, id, world->rank);
        if (r != ncclSuccess) { set_error("ncclCommInitRank: %s", nccl->GetErrorString(r)); return 1; }
    }
    // Everything a run enqueues behind a front-end wait must be loaded before the first wait exists: a first launch
    // that has to load code may wait for the device to go idle, and a stream that waits for a counter that is not
    // coming never is. So: every kernel of this library, and NCCL's (one eight-byte AllReduce per communicator).
    if (fa_preload() || proj_preload() || p2p_preload() || nvls_preload() || modes_preload()) return 1;
    {
        float* warm = nullptr;
        EFA_CUDA(cudaMalloc(&warm, 2 * sizeof(float)));
        EFA_CUDA(cudaMemset(warm, 0, 2 * sizeof(float)));
        for (int i = 0; i < ncomm; i++) {
            ncclResult_t r = nccl->AllReduce(warm, warm, 2, ncclFloat, ncclSum, c->nccls[i], c->comm_streams[i]);
            if (r != ncclSuccess) { set_error("ncclAllReduce (warm-up): %s", nccl->GetErrorString(r)); return 1; }
            EFA_CUDA(cudaStreamSynchronize(c->comm_streams[i]));
        }
        EFA_CUDA(cudaFree(warm));
    }
    EFA_CUDA(cudaEventCreate(&c->ev_t0));
    EFA_CUDA(cudaEventCreate(&c->ev_t1));
    EFA_CUDA(cudaEventCreate(&c->ev_t2));
    EFA_CUDA(cudaEventCreate(&c->ev_t3));
    *out = c;
    return 0;
}

namespace efa { void p2p_destroy(efa_ctx* c); void nvls_destroy(efa_ctx* c); int nvls_prepare(efa_ctx* c, const efa_params& p); void* nvls_result_buf(efa_ctx* c); }

extern "C" int efa_nvls_output(efa_ctx* c, const efa_params* p, void** output)
{
    if (!c || !p || !output) { set_error("efa_nvls_output: null argument"); return 2; }
    if (nvls_prepare(c, *p)) return 1;
    *output = nvls_result_buf(c);
    return 0;
}

extern "C" int efa_ctx_set_wait_limit_ms(efa_ctx* c, double device_ms, double host_ms)
{
    if (!c) { set_error("efa_ctx_set_wait_limit_ms: null context"); return 2; }
    if (device_ms > 0.0) c->wait_limit_ns = (unsigned long long)(device_ms * 1e6);
    if (host_ms > 0.0) c->host_wait_limit_ms = host_ms;
    return 0;
}

extern "C" int efa_destroy_ctx(efa_ctx* c)
{
    if (!c) return 0;
    cudaDeviceSynchronize();
    p2p_destroy(c);
    nvls_destroy(c);
    for (int i = 0; i < c->ncomm; i++) {
        if (c->nccls[i] && nccl_api()) nccl_api()->CommDestroy(c->nccls[i]);
        if (c->comm_streams[i]) cudaStreamDestroy(c->comm_streams[i]);
    }
    if (c->h2d_stream) cudaStreamDestroy(c->h2d_stream);
    if (c->d2h_stream) cudaStreamDestroy(c->d2h_stream);
    if (c->compute_stream) cudaStreamDestroy(c->compute_stream);
    if (c->proj_stream) cudaStreamDestroy(c->proj_stream);
    for (cudaEvent_t e : c->events) cudaEventDestroy(e);
    for (cudaEvent_t e : c->trace_events) cudaEventDestroy(e);
    for (cudaEvent_t e : {c->ev_t0, c->ev_t1, c->ev_t2, c->ev_t3}) if (e) cudaEventDestroy(e);
    if (c->rescue_stream) cudaStreamDestroy(c->rescue_stream);
    for (void* q : {c->O_all, c->send_buf, (void*)c->counters, (void*)c->order_tab, (void*)c->ws_O, (void*)c->ws_m, (void*)c->ws_l,
                    c->h_Q, c->h_K, c->h_V, c->h_W, c->h_out})
        if (q) cudaFree(q);
    delete c;
    return 0;
}
