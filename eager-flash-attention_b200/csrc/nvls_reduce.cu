// Sum AllReduce of the fp16 partial sums through an NVLink multicast object.
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
// No TMA, no cluster multicast; the multicast here is the NVSwitch one (multimem.*).
#include "nvls_reduce.h"

#include "host_util.h"
#include "sm100_ptx.cuh"

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstddef>
#include <cstring>

struct NvlsState {
    int R = 0, rank = 0;
    size_t size = 0;                 // bytes mapped (flags + partial sums + results)
    size_t data_bytes = 0;           // capacity of the result region (fp16); the partial sums have twice that (room for fp32)
    CUmemGenericAllocationHandle mem = 0, mc = 0;
    CUdeviceptr uc = 0, mcva = 0;    // this rank's memory; the multicast view of all ranks' memory
    CUdevice dev = 0;
    bool have_mem = false, have_mc = false, bound = false, uc_mapped = false, mc_mapped = false;
    unsigned seq[EFA_MAX_COMM] = {}; // barriers done per slot (same on all ranks)
};

namespace efa {

namespace {

constexpr int    NV_THREADS   = 512;
constexpr int    NV_MAX_CTAS  = 64;
constexpr size_t NV_FLAG_BYTES = 64 * 1024;             // EFA_MAX_COMM slots x NV_MAX_CTAS flags, padded

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
__device__ __forceinline__ bool block_barrier(const NvArgs& a, unsigned target, int site, int* abort_word)
{
    __threadfence_system();
    multimem_red_add(a.flags_mc + blockIdx.x, 1u);
    const unsigned long long t0 = globaltimer_ns();
    int spins = 0;
    while (true) {
        const unsigned v = ld_acquire_sys_u32(a.flags_uc + blockIdx.x);
        if ((int)(v - target) >= 0) return true;
        if ((++spins & 15) == 0 && globaltimer_ns() - t0 > a.limit_ns) { *abort_word = site; return false; }
        __nanosleep(spins < 64 ? 50 : 400);
    }
}

// WIRE_F32: the partial sums are fp32 (two 16-byte loads per 8 elements, summed in fp32 by the switch, rounded here,
// once); otherwise fp16 (one load per 8 elements, fp32 accumulation and the rounding inside the switch).
template <bool WIRE_F32>
__global__ void __launch_bounds__(NV_THREADS)
nvls_allreduce_kernel(const NvArgs a)
{
    constexpr int UNROLL = WIRE_F32 ? 4 : 8;              // 16-byte loads in flight per thread: 8
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        block_barrier(a, a.target_start, 61, &abort_word);
    }
    __syncthreads();
    if (abort_word == 0) {
        // this rank's share of the range
        const size_t per = (a.n16 + a.R - 1) / a.R;
        const size_t lo = min((size_t)a.rank * per, a.n16), hi = min(lo + per, a.n16);
        const size_t stride = (size_t)gridDim.x * NV_THREADS;
        for (size_t i = lo + (size_t)blockIdx.x * NV_THREADS + threadIdx.x; i < hi; i += UNROLL * stride) {
            uint4 v[UNROLL];
            #pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const size_t e = a.first16 + i + u * stride;
                if (i + u * stride < hi) {
                    if (WIRE_F32) {
                        const uint4 x = multimem_ld_reduce_f32(a.mc_send + e * 32);
                        const uint4 y = multimem_ld_reduce_f32(a.mc_send + e * 32 + 16);
                        v[u].x = pack_f16x2(__uint_as_float(x.x), __uint_as_float(x.y));
                        v[u].y = pack_f16x2(__uint_as_float(x.z), __uint_as_float(x.w));
                        v[u].z = pack_f16x2(__uint_as_float(y.x), __uint_as_float(y.y));
                        v[u].w = pack_f16x2(__uint_as_float(y.z), __uint_as_float(y.w));
                    } else {
                        v[u] = multimem_ld_reduce_f16(a.mc_send + e * 16);
                    }
                }
            }
            #pragma unroll
            for (int u = 0; u < UNROLL; u++)
                if (i + u * stride < hi) multimem_st(a.mc_out + (a.first16 + i + u * stride) * 16, v[u]);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // Arrive even after a failed first barrier, so that the flags stay in step across ranks.
        int second = 0;
        block_barrier(a, a.target_end, 62, abort_word == 0 ? &abort_word : &second);
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

void release_local(NvlsState* st)
{
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

}  // namespace

int nvls_supported(efa_ctx* c, const efa_params& p, const char** why)
{
    (void)c;
    *why = nullptr;
    if (p.R > 8) *why = "reduce=nvls handles at most 8 ranks (one NVSwitch box)";
    else if (p.proj_f32) *why = "reduce=nvls sums fp16 partial sums (proj_f32 goes with the NCCL reduction)";
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
    // Growing is collective, so the ranks vote (they all see the same params; the vote guards against a mix-up).
    double vote = (st->size != 0 && st->data_bytes >= want && st->R == c->world.size) ? 0.0 : 1.0;
    if (world_max(c->world, &vote)) return 1;
    if (vote == 0.0) return 0;
    if (world_barrier(c->world)) return 1;
    EFA_CUDA(cudaDeviceSynchronize());
    release_local(st);
    if (world_barrier(c->world)) return 1;
    const size_t data = (want + 4095) / 4096 * 4096;
    // The grid of the reduction kernel is fixed for the life of a region (flag b counts the barriers of block b).
    c->nvls_ctas = (p.reduce_ctas >= 1 && p.reduce_ctas <= NV_MAX_CTAS) ? p.reduce_ctas : 16;
    return create_region(c, st, data);
}

void* nvls_send_buf(efa_ctx* c) { return c->nvls && c->nvls->size ? (void*)(c->nvls->uc + NV_FLAG_BYTES) : nullptr; }
void* nvls_result_buf(efa_ctx* c) { return c->nvls && c->nvls->size ? (void*)(c->nvls->uc + NV_FLAG_BYTES + 2 * c->nvls->data_bytes) : nullptr; }

int nvls_allreduce(efa_ctx* c, int slot, size_t first, size_t n, bool wire_f32, cudaStream_t stream)
{
    NvlsState* st = c->nvls;
    if (!st || !st->size) { set_error("nvls_allreduce without nvls_prepare"); return 2; }
    if (slot < 0 || slot >= EFA_MAX_COMM) { set_error("nvls_allreduce: slot %d out of range", slot); return 2; }
    if ((first % 8) != 0 || (n % 8) != 0 || (first + n) * sizeof(__half) > st->data_bytes) {
        set_error("nvls_allreduce: range [%zu, %zu) not 16-byte aligned or outside the region", first, first + n);
        return 2;
    }
    if (n == 0) return 0;
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

int nvls_preload() { return touch_kernel(nvls_allreduce_kernel<true>) || touch_kernel(nvls_allreduce_kernel<false>); }

}  // namespace efa
