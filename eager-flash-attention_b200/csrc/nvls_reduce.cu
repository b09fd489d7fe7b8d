// Sum AllReduce of the partial sums (fp32 or fp16) through an NVLink multicast object.
//
// Stands in for allreduce() of eager-flash-attention (run_drivers.cu:26-30: ncclAllReduce, fp32 sum) on
// one NVSwitch box. Every rank owns a region of the same size and layout (symmetric memory) that is
// bound to one multicast object; a multicast address therefore names the same offset on all ranks:
//   multimem.ld_reduce [mc + x]   returns the SUM over all ranks of what each holds at x (the switch adds,
//                                 .acc::f32: fp16 inputs are accumulated in fp32 and rounded once),
//   multimem.st [mc + x], v       writes v at x on every rank,
//   multimem.red [mc + x], 1      adds 1 to the word at x on every rank.
// One call reduces a range of elements: rank r takes the r-th share of the range, loads the sums of its
// share and stores them to every rank's result buffer, so each element crosses each NVLink once in each
// direction. A call is bracketed by two barriers among the ranks, per thread block: block b of every
// rank adds 1 to flag b on all ranks and waits for its local copy to reach ranks * (barriers so far).
// Flags only grow (wrap-safe comparison), nothing is ever reset. The first barrier says "every rank's
// partial sums of this range are written" (its projection is earlier in stream order), the second
// "every rank's share has landed everywhere".
//
// Waits are bounded: on expiry the block records a status and returns without touching the data.
// The multicast here is the NVSwitch one (multimem.*). The in-switch kernel uses no TMA at all; the pulling kernel
// further down fetches with plain bulk asynchronous copies (one destination block each, no multicast qualifier).
#include "nvls_reduce.h"

#include "host_util.h"
#include "sm100_ptx.cuh"

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstddef>
#include <cstring>
#include <vector>

struct NvlsState {
    int R = 0, rank = 0;
    size_t size = 0;                 // bytes mapped (flags + partial sums + results)
    size_t data_bytes = 0;           // capacity of the result region (fp16); the partial sums have twice that (room for fp32)
    CUmemGenericAllocationHandle mem = 0, mc = 0;
    CUdeviceptr uc = 0, mcva = 0;    // this rank's memory; the multicast view of all ranks' memory
    CUdevice dev = 0;
    bool have_mem = false, have_mc = false, bound = false, uc_mapped = false, mc_mapped = false;
    unsigned seq[EFA_MAX_COMM] = {}; // barriers done per slot (same on all ranks)
    // EFA_REDUCE_PULL: fp32 partial sums in plain device memory that every rank maps (CUDA IPC)
    float* pull_send = nullptr;
    size_t pull_bytes = 0;
    float* pull_peer[8] = {};
    void*  pull_opened[8] = {};      // what cudaIpcOpenMemHandle returned, per peer
    int    pull_ctas = 0;            // grid of the pulling kernel, fixed while these buffers live (it has flags and counts of its own)
    unsigned pull_seq[EFA_MAX_COMM] = {};
};

namespace efa {

namespace {

#ifndef EFA_NV_THREADS
#define EFA_NV_THREADS 512
#endif
constexpr int    NV_THREADS   = EFA_NV_THREADS;
constexpr int    NV_MAX_CTAS  = 64;
constexpr size_t NV_FLAG_BYTES = 64 * 1024;             // two banks (in-switch, pulling) of EFA_MAX_COMM slots x NV_MAX_CTAS flags, padded

struct NvArgs {
    const char* mc_send;       // multicast view of the partial sums
    char*       mc_out;        // multicast view of the result buffers
    unsigned*   flags_mc;      // multicast view of this slot's flags
    const unsigned* flags_uc;  // this rank's copy of them
    size_t      first16, n16;  // range in units of 8 elements (16 bytes of fp16)
    int         R, rank;
    unsigned    target_start, target_end;
    unsigned long long limit_ns;
    int*        status;
};

__device__ __forceinline__ void multimem_red_add(unsigned* mc_addr, unsigned v)
{
    asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" :: "l"(mc_addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16(const char* mc_addr)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f32(const char* mc_addr)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st(char* mc_addr, const uint4& v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Thread 0 of the block: add 1 to this block's flag on every rank, then wait until all ranks did.
__device__ __forceinline__ bool block_barrier(unsigned* flags_mc, const unsigned* flags_uc, unsigned long long limit_ns,
                                              unsigned target, int site, int* abort_word)
{
    __threadfence_system();
    multimem_red_add(flags_mc + blockIdx.x, 1u);
    const unsigned long long t0 = globaltimer_ns();
    int spins = 0;
    while (true) {
        const unsigned v = ld_acquire_sys_u32(flags_uc + blockIdx.x);
        if ((int)(v - target) >= 0) return true;
        if ((++spins & 15) == 0 && globaltimer_ns() - t0 > limit_ns) { *abort_word = site; return false; }
        __nanosleep(spins < 64 ? 50 : 400);
    }
}

// The data loop. A warp works on runs of 256 elements: 512 bytes of fp16 results, one 16-byte store per lane.
//   fp16 partial sums: one 16-byte load per lane (fp32 accumulation and the rounding inside the switch).
//   WIRE_F32: the partial sums are fp32, 1 KB per run. Lane l loads bytes [16 l, 16 l + 16) and [512 + 16 l, ...):
//   every load instruction of the warp covers 512 contiguous bytes. The switch sums in fp32, the lane rounds
//   (once), and neighbouring lanes swap halves so that each again owns 16 contiguous bytes of the result: an
//   even lane l stores elements [4 l, 4 l + 8) of the run, an odd lane [128 + 4 (l - 1), ... + 8).
// LOADS 16-byte loads are in flight per thread before the first store.
#ifndef EFA_NV_LOADS
#define EFA_NV_LOADS 8
#endif
template <bool WIRE_F32>
__global__ void __launch_bounds__(NV_THREADS)
nvls_allreduce_kernel(const NvArgs a)
{
    constexpr int RUNS = WIRE_F32 ? EFA_NV_LOADS / 2 : EFA_NV_LOADS;     // runs per warp and iteration
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        block_barrier(a.flags_mc, a.flags_uc, a.limit_ns, a.target_start, 61, &abort_word);
    }
    __syncthreads();
    if (abort_word == 0) {
        // this rank's share of the range, in whole runs (32 units of 8 elements) except at the end of the range
        const size_t per = ((a.n16 + a.R - 1) / a.R + 31) / 32 * 32;
        const size_t lo = min((size_t)a.rank * per, a.n16), hi = min(lo + per, a.n16);
        const int lane = threadIdx.x & 31;
        const size_t warp = (size_t)blockIdx.x * (NV_THREADS / 32) + (threadIdx.x >> 5);
        const size_t warps = (size_t)gridDim.x * (NV_THREADS / 32);
        const int my_unit = WIRE_F32 ? ((lane & 1) ? 16 + (lane >> 1) : (lane >> 1)) : lane;   // the unit this lane stores
        for (size_t run = lo + warp * 32; run < hi; run += RUNS * warps * 32) {
            uint4 v[RUNS];
            #pragma unroll
            for (int u = 0; u < RUNS; u++) {
                const size_t base = run + (size_t)u * warps * 32;          // first unit of the run
                v[u] = make_uint4(0u, 0u, 0u, 0u);
                if (base >= hi) continue;                                  // the same for the whole warp
                const int left = (int)min((size_t)32, hi - base);          // units of this run inside the share
                if (WIRE_F32) {
                    const char* src = a.mc_send + (a.first16 + base) * 32;
                    uint4 x = make_uint4(0u, 0u, 0u, 0u), y = x;
                    if ((lane >> 1) < left)      x = multimem_ld_reduce_f32(src + lane * 16);
                    if (16 + (lane >> 1) < left) y = multimem_ld_reduce_f32(src + 512 + lane * 16);
                    v[u].x = pack_f16x2(__uint_as_float(x.x), __uint_as_float(x.y));
                    v[u].y = pack_f16x2(__uint_as_float(x.z), __uint_as_float(x.w));
                    v[u].z = pack_f16x2(__uint_as_float(y.x), __uint_as_float(y.y));
                    v[u].w = pack_f16x2(__uint_as_float(y.z), __uint_as_float(y.w));
                } else if (lane < left) {
                    v[u] = multimem_ld_reduce_f16(a.mc_send + (a.first16 + base + lane) * 16);
                }
            }
            #pragma unroll
            for (int u = 0; u < RUNS; u++) {
                const size_t base = run + (size_t)u * warps * 32;
                if (base >= hi) continue;
                const int left = (int)min((size_t)32, hi - base);
                uint4 out = v[u];
                if (WIRE_F32) {
                    // an even lane keeps its first half and takes the neighbour's first half; an odd lane the second halves
                    const bool odd = lane & 1;
                    const unsigned give0 = odd ? v[u].x : v[u].z, give1 = odd ? v[u].y : v[u].w;
                    const unsigned got0 = __shfl_xor_sync(0xffffffffu, give0, 1), got1 = __shfl_xor_sync(0xffffffffu, give1, 1);
                    out = odd ? make_uint4(got0, got1, v[u].z, v[u].w) : make_uint4(v[u].x, v[u].y, got0, got1);
                }
                if (my_unit < left) multimem_st(a.mc_out + (a.first16 + base + my_unit) * 16, out);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // Arrive even after a failed first barrier, so that the flags stay in step across ranks.
        int second = 0;
        block_barrier(a.flags_mc, a.flags_uc, a.limit_ns, a.target_end, 62, abort_word == 0 ? &abort_word : &second);
        if (abort_word != 0 && a.status != nullptr && atomicCAS(a.status, 0, (int)KS_WAIT_TIMEOUT) == 0) {
            a.status[1] = (int)blockIdx.x;
            a.status[2] = abort_word;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same reduction with the sum done on the SM: rank r fetches its share of EVERY rank's fp32 partial sums
// (its own among them) with bulk asynchronous copies into shared memory, adds them in rank order, rounds once and
// stores the fp16 result to every rank through the switch (multimem.st). A bulk copy moves 8 KB per instruction and
// a block keeps up to 192 KB in flight, so a dozen blocks fill the links, where multimem.ld_reduce (a round trip
// through the switch per 16 bytes and thread) needs some fifty. The price is wire bytes: each link carries
// (R-1)/R of the fp32 partial sums inbound instead of 1/R.
// Warp 0 issues the copies (one elected lane), warps 1-8 add and store, one unit of 8 elements per thread and chunk;
// ring of `nstage` stages, every wait bounded.
// ---------------------------------------------------------------------------------------------
constexpr int PL_CONSUMERS = 256;
constexpr int PL_THREADS = 32 + PL_CONSUMERS;
constexpr int PL_UNITS = 256;                              // units of 8 elements per chunk: 8 KB of fp32 per rank
constexpr int PL_CHUNK_BYTES = PL_UNITS * 32;
constexpr int PL_MAX_STAGES = 8;
constexpr int PL_SMEM_BUDGET = 192 * 1024;

struct PullArgs {
    const float* send_peer[8]; // every rank's partial sums (peer mappings; this rank's own at [rank])
    char*       mc_out;        // multicast view of the result buffers
    unsigned*   flags_mc;
    const unsigned* flags_uc;
    size_t      first16, n16;  // range in units of 8 elements
    int         R, rank, nstage;
    unsigned    target_start, target_end;
    unsigned long long limit_ns;
    int*        status;
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(PL_THREADS)
pull_allreduce_kernel(const PullArgs a)
{
    extern __shared__ __align__(128) unsigned char pl_smem[];
    __shared__ uint64_t full[PL_MAX_STAGES], empty[PL_MAX_STAGES];
    __shared__ int abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int s = 0; s < a.nstage; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], PL_CONSUMERS / 32); }
        mbar_fence_init();
        block_barrier(a.flags_mc, a.flags_uc, a.limit_ns, a.target_start, 63, &abort_word);
    }
    __syncthreads();
    if (abort_word == 0) {
        // this rank's share of the range, in whole chunks except at the end of the range
        const size_t per = ((a.n16 + a.R - 1) / a.R + PL_UNITS - 1) / PL_UNITS * PL_UNITS;
        const size_t lo = min((size_t)a.rank * per, a.n16), hi = min(lo + per, a.n16);
        const int nchunks = (int)((hi - lo + PL_UNITS - 1) / PL_UNITS);
        const size_t stage_bytes = (size_t)a.R * PL_CHUNK_BYTES;
        if (warp == 0) {
            if (elect_one()) {
                // the partial sums were written through the generic proxy (on this GPU and on the peers) and are read
                // through the asynchronous one
                asm volatile("fence.proxy.async;" ::: "memory");
                int it = 0, s = 0, use = 0;
                for (int k = blockIdx.x; k < nchunks; k += gridDim.x, it++) {
                    if (use > 0 && !mbar_wait(&empty[s], (uint32_t)((use - 1) & 1), &abort_word, 64, a.limit_ns)) break;
                    const size_t unit0 = lo + (size_t)k * PL_UNITS;
                    const uint32_t bytes = (uint32_t)min((size_t)PL_UNITS, hi - unit0) * 32u;
                    mbar_expect_tx(&full[s], bytes * (uint32_t)a.R);
                    unsigned char* dst = pl_smem + (size_t)s * stage_bytes;
                    for (int q = 0; q < a.R; q++) {
                        int j = a.rank + 1 + q; if (j >= a.R) j -= a.R;      // every rank starts at another peer
                        bulk_load(dst + (size_t)q * PL_CHUNK_BYTES, a.send_peer[j] + (a.first16 + unit0) * 8, bytes, &full[s]);
                    }
                    if (++s == a.nstage) { s = 0; use++; }
                }
                if (abort_word != 0) {
                    // somebody gave up: no copy may still be on its way into this block's shared memory when it exits
                    // (one limit for all stages together)
                    const unsigned long long t_drain = globaltimer_ns();
                    for (int t = 0; t < a.nstage; t++) {
                        const int uses = use + (t < s ? 1 : 0);              // copies issued into stage t so far
                        const unsigned long long spent = globaltimer_ns() - t_drain;
                        if (spent >= a.limit_ns) break;
                        int local = 0;
                        if (uses > 0) mbar_wait(&full[t], (uint32_t)((uses - 1) & 1), &local, 0, a.limit_ns - spent);
                    }
                }
            }
        } else {
            const int t = threadIdx.x - 32;
            int s = 0, use = 0;
            for (int k = blockIdx.x; k < nchunks; k += gridDim.x) {
                if (!mbar_wait(&full[s], (uint32_t)(use & 1), &abort_word, 65, a.limit_ns)) break;
                const size_t unit0 = lo + (size_t)k * PL_UNITS;
                const int units = (int)min((size_t)PL_UNITS, hi - unit0);
                const unsigned char* src = pl_smem + (size_t)s * stage_bytes;
                static_assert(PL_UNITS == PL_CONSUMERS, "one unit per adding thread and chunk");
                if (t < units) {
                    const int unit = t;
                    float4 x[8], y[8];
                    #pragma unroll
                    for (int j = 0; j < 8; j++) {                            // all loads first, then the sum in rank order
                        if (j < a.R) {
                            int q = j - a.rank - 1; if (q < 0) q += a.R;
                            const float4* p = reinterpret_cast<const float4*>(src + (size_t)q * PL_CHUNK_BYTES + (size_t)unit * 32);
                            x[j] = p[0]; y[j] = p[1];
                        }
                    }
                    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    #pragma unroll
                    for (int j = 0; j < 8; j++) {                            // rank order: the same sum whoever adds
                        if (j < a.R) {
                            acc[0] += x[j].x; acc[1] += x[j].y; acc[2] += x[j].z; acc[3] += x[j].w;
                            acc[4] += y[j].x; acc[5] += y[j].y; acc[6] += y[j].z; acc[7] += y[j].w;
                        }
                    }
                    uint4 out;
                    out.x = pack_f16x2(acc[0], acc[1]); out.y = pack_f16x2(acc[2], acc[3]);
                    out.z = pack_f16x2(acc[4], acc[5]); out.w = pack_f16x2(acc[6], acc[7]);
                    multimem_st(a.mc_out + (a.first16 + unit0 + unit) * 16, out);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                if (++s == a.nstage) { s = 0; use++; }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int second = 0;
        block_barrier(a.flags_mc, a.flags_uc, a.limit_ns, a.target_end, 66, abort_word == 0 ? &abort_word : &second);
        if (abort_word != 0 && a.status != nullptr && atomicCAS(a.status, 0, (int)KS_WAIT_TIMEOUT) == 0) {
            a.status[1] = (int)blockIdx.x;
            a.status[2] = abort_word;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// One file descriptor from rank 0 to every other rank (Unix-domain socket in the abstract namespace,
// SCM_RIGHTS): how the multicast object's shareable handle travels between the processes of one host.
// ---------------------------------------------------------------------------------------------
int send_fd(int sock, int fd)
{
    char byte = 'x';
    iovec io{&byte, 1};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_iov = &io; msg.msg_iovlen = 1;
    msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET; cm->cmsg_type = SCM_RIGHTS; cm->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(cm), &fd, sizeof(int));
    return sendmsg(sock, &msg, 0) == 1 ? 0 : 1;
}

int recv_fd(int sock, int* fd)
{
    char byte = 0;
    iovec io{&byte, 1};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_iov = &io; msg.msg_iovlen = 1;
    msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
    pollfd pf{sock, POLLIN, 0};
    if (poll(&pf, 1, 20000) != 1) return 1;
    if (recvmsg(sock, &msg, 0) != 1) return 1;
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    if (!cm || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS) return 1;
    std::memcpy(fd, CMSG_DATA(cm), sizeof(int));
    return 0;
}

socklen_t abstract_addr(sockaddr_un* addr, const char* name)
{
    std::memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    const size_t len = std::strlen(name);
    std::memcpy(addr->sun_path + 1, name, len);           // sun_path[0] == 0: abstract namespace
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + len);
}

}  // namespace

// Rank 0 passes `fd_root`; every other rank receives its own descriptor for the same object in *fd_out.
// Returns 0 on this rank's success (the caller votes over the ranks afterwards).
int share_fd(const efa_world& w, int fd_root, int* fd_out)
{
    char name[64];
    std::memset(name, 0, sizeof(name));
    int lsock = -1;
    int rc = 0;
    if (w.rank == 0) {
        static int serial = 0;
        snprintf(name, sizeof(name), "efa-nvls-%d-%d", (int)getpid(), serial++);
        lsock = socket(AF_UNIX, SOCK_STREAM, 0);
        sockaddr_un addr;
        const socklen_t alen = abstract_addr(&addr, name);
        if (lsock < 0 || bind(lsock, (sockaddr*)&addr, alen) != 0 || listen(lsock, 16) != 0) {
            if (lsock >= 0) close(lsock);
            lsock = -1;
            name[0] = '!';                                    // tells the others not to connect
            rc = 1;
        }
    }
    if (w.bcast_bytes(w.user, name, sizeof(name), 0)) return 1;
    if (name[0] == '!') return 1;
    if (w.rank == 0) {
        *fd_out = fd_root;
        for (int i = 1; i < w.size; i++) {
            pollfd pf{lsock, POLLIN, 0};
            if (poll(&pf, 1, 20000) != 1) { rc = 1; break; }
            const int s = accept(lsock, nullptr, nullptr);
            if (s < 0) { rc = 1; break; }
            if (send_fd(s, fd_root)) rc = 1;
            close(s);
        }
        close(lsock);
    } else {
        const int s = socket(AF_UNIX, SOCK_STREAM, 0);
        sockaddr_un addr;
        const socklen_t alen = abstract_addr(&addr, name);
        if (s < 0 || connect(s, (sockaddr*)&addr, alen) != 0 || recv_fd(s, fd_out)) rc = 1;
        if (s >= 0) close(s);
    }
    return rc;
}

namespace {

// Every rank learns whether all ranks succeeded (a failure on one rank must not leave the others inside
// the next collective step).
bool all_ok(const efa_world& w, bool mine)
{
    double v = mine ? 0.0 : 1.0;
    if (world_max(w, &v)) return false;
    return v == 0.0;
}

void release_pull(NvlsState* st)
{
    for (int r = 0; r < 8; r++) {
        if (st->pull_opened[r]) cudaIpcCloseMemHandle(st->pull_opened[r]);
        st->pull_opened[r] = nullptr;
        st->pull_peer[r] = nullptr;
    }
    if (st->pull_send) cudaFree(st->pull_send);
    st->pull_send = nullptr;
    st->pull_bytes = 0;
    (void)cudaGetLastError();
}

void release_local(NvlsState* st)
{
    release_pull(st);
    const DriverApi* api = driver_api();
    if (!api) return;
    if (st->mc_mapped) { api->cuMemUnmap(st->mcva, st->size); st->mc_mapped = false; }
    if (st->mcva) { api->cuMemAddressFree(st->mcva, st->size); st->mcva = 0; }
    if (st->uc_mapped) { api->cuMemUnmap(st->uc, st->size); st->uc_mapped = false; }
    if (st->uc) { api->cuMemAddressFree(st->uc, st->size); st->uc = 0; }
    if (st->bound) { api->cuMulticastUnbind(st->mc, st->dev, 0, st->size); st->bound = false; }
    if (st->have_mem) { api->cuMemRelease(st->mem); st->have_mem = false; }
    if (st->have_mc) { api->cuMemRelease(st->mc); st->have_mc = false; }
    st->size = 0; st->data_bytes = 0;
}

int create_region(efa_ctx* c, NvlsState* st, size_t data_bytes)
{
    const DriverApi* api = driver_api();
    if (!api) return 1;
    const efa_world& w = c->world;
    const int R = w.size;
    EFA_CUDA(cudaFree(nullptr));                                  // makes the runtime's context current
    bool ok = api->cuCtxGetDevice(&st->dev) == CUDA_SUCCESS;
    int supported = 0;
    if (ok) ok = api->cuDeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, st->dev) == CUDA_SUCCESS && supported;
    if (!all_ok(w, ok)) { set_error("reduce=nvls: a device of this group does not support NVLink multicast"); return 5; }

    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)R;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mp.size = NV_FLAG_BYTES + 3 * data_bytes;                     // flags, partial sums (fp32 capable), fp16 results
    CUmemAllocationProp ap;
    std::memset(&ap, 0, sizeof(ap));
    ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    ap.location.id = (int)st->dev;
    ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g_mc = 0, g_mem = 0;
    ok = api->cuMulticastGetGranularity(&g_mc, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS &&
         api->cuMemGetAllocationGranularity(&g_mem, &ap, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && g_mc && g_mem;
    if (!all_ok(w, ok)) { set_error("reduce=nvls: no multicast granularity (is the NVLink fabric set up for multicast?)"); return 5; }
    const size_t gran = g_mc > g_mem ? g_mc : g_mem;              // both are powers of two
    const size_t size = (mp.size + gran - 1) / gran * gran;
    mp.size = size;
    st->size = size;

    // the multicast object: created by rank 0, imported by the others
    int fd = -1;
    ok = true;
    if (w.rank == 0) {
        ok = api->cuMulticastCreate(&st->mc, &mp) == CUDA_SUCCESS;
        if (ok) st->have_mc = true;
        if (ok && R > 1) ok = api->cuMemExportToShareableHandle(&fd, st->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
    }
    if (!all_ok(w, ok)) { if (fd >= 0) close(fd); release_local(st); set_error("reduce=nvls: the multicast object could not be created"); return 5; }
    if (R > 1) {
        int got = -1;
        ok = share_fd(w, fd, &got) == 0;
        if (ok && w.rank != 0) {
            ok = api->cuMemImportFromShareableHandle(&st->mc, (void*)(uintptr_t)got, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
            if (ok) st->have_mc = true;
            close(got);
        }
        if (w.rank == 0 && fd >= 0) close(fd);
        if (!all_ok(w, ok)) { release_local(st); set_error("reduce=nvls: the multicast handle could not be passed to every rank"); return 5; }
    }
    ok = api->cuMulticastAddDevice(st->mc, st->dev) == CUDA_SUCCESS;
    if (!all_ok(w, ok)) { release_local(st); set_error("reduce=nvls: cuMulticastAddDevice failed"); return 5; }

    // this rank's memory, bound at offset 0 of the object
    ok = api->cuMemCreate(&st->mem, size, &ap, 0) == CUDA_SUCCESS;
    if (ok) st->have_mem = true;
    if (!all_ok(w, ok)) { release_local(st); set_error("reduce=nvls: no device memory for the symmetric region (%zu bytes)", size); return 1; }
    ok = api->cuMulticastBindMem(st->mc, 0, st->mem, 0, size, 0) == CUDA_SUCCESS;
    if (ok) st->bound = true;
    if (!all_ok(w, ok)) { release_local(st); set_error("reduce=nvls: cuMulticastBindMem failed"); return 5; }

    CUmemAccessDesc acc;
    std::memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = (int)st->dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    ok = api->cuMemAddressReserve(&st->uc, size, gran, 0, 0) == CUDA_SUCCESS;
    if (ok) { ok = api->cuMemMap(st->uc, size, 0, st->mem, 0) == CUDA_SUCCESS; st->uc_mapped = ok; }
    if (ok) ok = api->cuMemSetAccess(st->uc, size, &acc, 1) == CUDA_SUCCESS;
    if (ok) ok = api->cuMemAddressReserve(&st->mcva, size, gran, 0, 0) == CUDA_SUCCESS;
    if (ok) { ok = api->cuMemMap(st->mcva, size, 0, st->mc, 0) == CUDA_SUCCESS; st->mc_mapped = ok; }
    if (ok) ok = api->cuMemSetAccess(st->mcva, size, &acc, 1) == CUDA_SUCCESS;
    if (ok) ok = cudaMemset((void*)st->uc, 0, size) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    if (!all_ok(w, ok)) { (void)cudaGetLastError(); release_local(st); set_error("reduce=nvls: mapping the symmetric region failed"); return 5; }
    st->R = R; st->rank = w.rank; st->data_bytes = data_bytes;
    for (unsigned& s : st->seq) s = 0;
    return 0;
}

// fp32 partial sums of the pulling reduction: one plain allocation per rank, mapped by every other rank.
struct PullPacket {
    cudaIpcMemHandle_t handle;
    int ok;
};

int create_pull(efa_ctx* c, NvlsState* st, size_t bytes, int ctas)
{
    const efa_world& w = c->world;
    const int R = w.size;
    // A second bank of flags, all zero again: the pulling kernel's grid may differ from the in-switch kernel's.
    st->pull_ctas = (ctas >= 1 && ctas <= NV_MAX_CTAS) ? ctas : 12;
    for (unsigned& q : st->pull_seq) q = 0;
    // Every local failure up to the exchange travels in the packet's `ok`, so that all ranks return together; the
    // exchange is also the barrier between clearing the flags and their first use.
    bool ok = cudaMemset((unsigned*)st->uc + (size_t)EFA_MAX_COMM * NV_MAX_CTAS, 0,
                         (size_t)EFA_MAX_COMM * NV_MAX_CTAS * sizeof(unsigned)) == cudaSuccess &&
              cudaDeviceSynchronize() == cudaSuccess;
    if (ok) ok = cudaMalloc(reinterpret_cast<void**>(&st->pull_send), bytes) == cudaSuccess;
    if (ok) { st->pull_bytes = bytes; ok = cudaMemset(st->pull_send, 0, bytes) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess; }
    PullPacket mine;
    std::memset(&mine, 0, sizeof(mine));
    mine.ok = ok && cudaIpcGetMemHandle(&mine.handle, st->pull_send) == cudaSuccess;
    std::vector<PullPacket> all((size_t)R);
    if (w.allgather_bytes(w.user, &mine, all.data(), sizeof(PullPacket))) { release_pull(st); set_error("reduce=pull: handle exchange failed"); return 1; }
    bool every = true;
    for (int r = 0; r < R; r++) every = every && all[(size_t)r].ok;
    if (!every) { (void)cudaGetLastError(); release_pull(st); set_error("reduce=pull: a rank could not clear its flags, or allocate or export %zu bytes of partial sums", bytes); return 1; }
    bool opened = true;
    for (int r = 0; r < R && opened; r++) {
        if (r == w.rank) { st->pull_peer[r] = st->pull_send; continue; }
        void* ptr = nullptr;
        opened = cudaIpcOpenMemHandle(&ptr, all[(size_t)r].handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
        if (opened) { st->pull_opened[r] = ptr; st->pull_peer[r] = static_cast<float*>(ptr); }
    }
    if (!all_ok(w, opened)) { (void)cudaGetLastError(); release_pull(st); set_error("reduce=pull: a rank could not map a peer's partial sums (cudaIpcOpenMemHandle)"); return 5; }
    return 0;
}

}  // namespace

int nvls_supported(efa_ctx* c, const efa_params& p, const char** why)
{
    (void)c;
    *why = nullptr;
    if (p.R > 8) *why = "reduce=nvls handles at most 8 ranks (one NVSwitch box)";
    else if (p.proj_f32) *why = "reduce=nvls / pull write an fp16 result (proj_f32, an fp32 output, goes with the NCCL reduction)";
    return *why == nullptr;
}

int nvls_prepare(efa_ctx* c, const efa_params& p)
{
    const char* why = nullptr;
    if (!nvls_supported(c, p, &why)) { set_error("%s", why); return 5; }
    if (c->world.size > 1 && (!c->world.bcast_bytes || !c->world.allreduce_max_f64)) { set_error("reduce=nvls needs the world's callbacks"); return 2; }
    if (!c->nvls) c->nvls = new NvlsState();
    NvlsState* st = c->nvls;
    const size_t want = (size_t)p.S * p.d * sizeof(__half);
    const bool pull = p.reduce == EFA_REDUCE_PULL;
    if (pull && c->world.size > 1 && !c->world.allgather_bytes) { set_error("reduce=pull needs the world's allgather_bytes callback"); return 2; }
    // Growing is collective, so the ranks vote (they all see the same params; the vote guards against a mix-up).
    // A grid is fixed while its flags live, so an explicit reduce_ctas that differs from the grid in place rebuilds too.
    const bool asked = p.reduce_ctas >= 1 && p.reduce_ctas <= NV_MAX_CTAS;
    double vote = (st->size != 0 && st->data_bytes >= want && st->R == c->world.size &&
                   (pull || !asked || p.reduce_ctas == c->nvls_ctas)) ? 0.0 : 1.0;
    if (vote == 0.0 && pull && (st->pull_bytes < 2 * st->data_bytes || (asked && p.reduce_ctas != st->pull_ctas)))
        vote = 0.5;                                         // the region is fine, the fp32 partial sums (or their grid) are not
    if (world_max(c->world, &vote)) return 1;
    if (vote == 0.0) return 0;
    if (vote == 0.5) {
        if (world_barrier(c->world)) return 1;
        EFA_CUDA(cudaDeviceSynchronize());
        release_pull(st);
        return create_pull(c, st, 2 * st->data_bytes, p.reduce_ctas);
    }
    if (world_barrier(c->world)) return 1;
    EFA_CUDA(cudaDeviceSynchronize());
    release_local(st);
    if (world_barrier(c->world)) return 1;
    const size_t data = (want + 4095) / 4096 * 4096;
    // The grid of the reduction kernel is fixed for the life of a region (flag b counts the barriers of block b).
    c->nvls_ctas = (!pull && p.reduce_ctas >= 1 && p.reduce_ctas <= NV_MAX_CTAS) ? p.reduce_ctas : 32;
    if (create_region(c, st, data)) return 1;
    return pull ? create_pull(c, st, 2 * st->data_bytes, p.reduce_ctas) : 0;
}

void* nvls_pull_send_buf(efa_ctx* c) { return c->nvls ? (void*)c->nvls->pull_send : nullptr; }

void* nvls_send_buf(efa_ctx* c) { return c->nvls && c->nvls->size ? (void*)(c->nvls->uc + NV_FLAG_BYTES) : nullptr; }
void* nvls_result_buf(efa_ctx* c) { return c->nvls && c->nvls->size ? (void*)(c->nvls->uc + NV_FLAG_BYTES + 2 * c->nvls->data_bytes) : nullptr; }

int nvls_allreduce(efa_ctx* c, int slot, size_t first, size_t n, bool wire_f32, bool pull, cudaStream_t stream)
{
    NvlsState* st = c->nvls;
    if (!st || !st->size) { set_error("nvls_allreduce without nvls_prepare"); return 2; }
    if (slot < 0 || slot >= EFA_MAX_COMM) { set_error("nvls_allreduce: slot %d out of range", slot); return 2; }
    if ((first % 8) != 0 || (n % 8) != 0 || (first + n) * sizeof(__half) > st->data_bytes) {
        set_error("nvls_allreduce: range [%zu, %zu) not 16-byte aligned or outside the region", first, first + n);
        return 2;
    }
    if (n == 0) return 0;
    if (pull) {
        if (!st->pull_send) { set_error("nvls_allreduce: the pulling reduction was not prepared"); return 2; }
        PullArgs q;
        for (int r = 0; r < 8; r++) q.send_peer[r] = r < st->R ? st->pull_peer[r] : nullptr;
        q.mc_out = (char*)(st->mcva + NV_FLAG_BYTES + 2 * st->data_bytes);
        q.flags_mc = (unsigned*)st->mcva + (size_t)(EFA_MAX_COMM + slot) * NV_MAX_CTAS;
        q.flags_uc = (const unsigned*)st->uc + (size_t)(EFA_MAX_COMM + slot) * NV_MAX_CTAS;
        q.first16 = first / 8; q.n16 = n / 8;
        q.R = st->R; q.rank = st->rank;
        q.nstage = PL_SMEM_BUDGET / (st->R * PL_CHUNK_BYTES);
        if (q.nstage > PL_MAX_STAGES) q.nstage = PL_MAX_STAGES;
        q.target_start = (unsigned)st->R * (st->pull_seq[slot] + 1u);
        q.target_end = (unsigned)st->R * (st->pull_seq[slot] + 2u);
        st->pull_seq[slot] += 2u;
        q.limit_ns = c->wait_limit_ns;
        q.status = kernel_status_word();
        const size_t smem = (size_t)q.nstage * st->R * PL_CHUNK_BYTES;
        static bool configured = false;
        if (!configured) {
            EFA_CUDA(cudaFuncSetAttribute(pull_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PL_SMEM_BUDGET));
            configured = true;
        }
        pull_allreduce_kernel<<<st->pull_ctas, PL_THREADS, smem, stream>>>(q);
        EFA_CUDA(cudaGetLastError());
        return 0;
    }
    NvArgs a;
    a.mc_send = (const char*)(st->mcva + NV_FLAG_BYTES);
    a.mc_out = (char*)(st->mcva + NV_FLAG_BYTES + 2 * st->data_bytes);
    a.flags_mc = (unsigned*)st->mcva + (size_t)slot * NV_MAX_CTAS;
    a.flags_uc = (const unsigned*)st->uc + (size_t)slot * NV_MAX_CTAS;
    a.first16 = first / 8; a.n16 = n / 8;
    a.R = st->R; a.rank = st->rank;
    a.target_start = (unsigned)st->R * (st->seq[slot] + 1u);
    a.target_end = (unsigned)st->R * (st->seq[slot] + 2u);
    st->seq[slot] += 2u;
    a.limit_ns = c->wait_limit_ns;
    a.status = kernel_status_word();
    // The grid is the same for every call of the context: flag b counts the barriers of block b.
    if (wire_f32) nvls_allreduce_kernel<true><<<c->nvls_ctas, NV_THREADS, 0, stream>>>(a);
    else          nvls_allreduce_kernel<false><<<c->nvls_ctas, NV_THREADS, 0, stream>>>(a);
    EFA_CUDA(cudaGetLastError());
    return 0;
}

void nvls_destroy(efa_ctx* c)
{
    if (!c->nvls) return;
    if (c->nvls->size) {
        // Nobody may unbind while a peer can still issue multimem operations on the object.
        world_barrier(c->world);
        cudaDeviceSynchronize();
        world_barrier(c->world);
        release_local(c->nvls);
        world_barrier(c->world);
    }
    delete c->nvls;
    c->nvls = nullptr;
}


namespace {
template <class K> int touch_kernel(K kernel)
{
    cudaFuncAttributes attr;
    EFA_CUDA(cudaFuncGetAttributes(&attr, kernel));
    return 0;
}
}  // namespace

int nvls_preload() { return touch_kernel(nvls_allreduce_kernel<true>) || touch_kernel(nvls_allreduce_kernel<false>) || touch_kernel(pull_allreduce_kernel); }

}  // namespace efa
