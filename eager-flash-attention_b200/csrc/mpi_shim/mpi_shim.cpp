// Shared-memory implementation of the MPI subset in mpi.h (one host, a handful of ranks).
//
// All collectives go through one segment: a sense-reversing barrier and a per-rank slot area.
// A collective is: every rank writes its slot, barrier, every rank reads what it needs, barrier.
// Waits time out (EFA_SHIM_TIMEOUT_S, default 300 s) and turn into an abort, so a rank that died
// cannot leave the others spinning forever.
#include "mpi.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

constexpr int kMaxRanks = 16;
constexpr size_t kSlotBytes = 4096;

struct Segment {
    std::atomic<int> arrived;
    std::atomic<int> generation;
    std::atomic<int> aborted;
    std::atomic<int> attached;
    alignas(64) unsigned char slots[kMaxRanks][kSlotBytes];
};

Segment* g_seg = nullptr;
int g_rank = 0, g_size = 1;
char g_name[128] = "";
double g_timeout_s = 300.0;

double wall()
{
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

[[noreturn]] void die(int code)
{
    if (g_seg) g_seg->aborted.store(1);
    fflush(stdout);
    fflush(stderr);
    _exit(code ? code : 1);
}

void barrier()
{
    if (g_size == 1) return;
    const int gen = g_seg->generation.load();
    if (g_seg->arrived.fetch_add(1) + 1 == g_size) {
        g_seg->arrived.store(0);
        g_seg->generation.fetch_add(1);
        return;
    }
    const double t0 = wall();
    long spins = 0;
    while (g_seg->generation.load() == gen) {
        if ((++spins & 255) == 0) {
            if (g_seg->aborted.load()) die(1);
            if (wall() - t0 > g_timeout_s) {
                fprintf(stderr, "mpi_shim: rank %d timed out in a barrier after %.0f s\n", g_rank, g_timeout_s);
                die(1);
            }
            if (spins > (1 << 16)) usleep(50);
        }
    }
}

size_t type_size(MPI_Datatype t)
{
    switch (t) {
        case MPI_BYTE: return 1;
        case MPI_INT: return 4;
        case MPI_FLOAT: return 4;
        case MPI_DOUBLE: return 8;
    }
    return 0;
}

template <class T>
void reduce_into(T* out, int count, MPI_Op op)
{
    for (int i = 0; i < count; i++) {
        T acc;
        std::memcpy(&acc, g_seg->slots[0] + i * sizeof(T), sizeof(T));
        for (int r = 1; r < g_size; r++) {
            T v;
            std::memcpy(&v, g_seg->slots[r] + i * sizeof(T), sizeof(T));
            if (op == MPI_MAX) acc = v > acc ? v : acc;
            else if (op == MPI_MIN) acc = v < acc ? v : acc;
            else acc = acc + v;
        }
        out[i] = acc;
    }
}

}  // namespace

extern "C" {

int MPI_Init_thread(int*, char***, int required, int* provided)
{
    if (provided) *provided = required;
    const char* r = getenv("EFA_SHIM_RANK");
    const char* s = getenv("EFA_SHIM_SIZE");
    const char* n = getenv("EFA_SHIM_NAME");
    if (const char* t = getenv("EFA_SHIM_TIMEOUT_S")) g_timeout_s = atof(t);
    if (!r || !s || !n || atoi(s) <= 1) { g_rank = 0; g_size = 1; return MPI_SUCCESS; }
    g_rank = atoi(r);
    g_size = atoi(s);
    if (g_size > kMaxRanks || g_rank < 0 || g_rank >= g_size) {
        fprintf(stderr, "mpi_shim: bad rank/size %d/%d\n", g_rank, g_size);
        return MPI_ERR_OTHER;
    }
    snprintf(g_name, sizeof(g_name), "%s", n);
    // The launcher creates and sizes the segment before starting the ranks.
    int fd = shm_open(g_name, O_RDWR, 0600);
    if (fd < 0) { perror("mpi_shim: shm_open"); return MPI_ERR_OTHER; }
    void* p = mmap(nullptr, sizeof(Segment), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) { perror("mpi_shim: mmap"); return MPI_ERR_OTHER; }
    g_seg = static_cast<Segment*>(p);
    g_seg->attached.fetch_add(1);
    barrier();
    return MPI_SUCCESS;
}

int MPI_Init(int* argc, char*** argv) { int p; return MPI_Init_thread(argc, argv, 0, &p); }

int MPI_Comm_rank(MPI_Comm, int* rank) { *rank = g_rank; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm, int* size) { *size = g_size; return MPI_SUCCESS; }

int MPI_Barrier(MPI_Comm) { barrier(); return MPI_SUCCESS; }

int MPI_Bcast(void* buf, int count, MPI_Datatype type, int root, MPI_Comm)
{
    if (g_size == 1) return MPI_SUCCESS;
    const size_t bytes = (size_t)count * type_size(type);
    if (type_size(type) == 0) return MPI_ERR_OTHER;
    unsigned char* b = static_cast<unsigned char*>(buf);
    for (size_t off = 0; off < bytes; off += kSlotBytes) {
        const size_t n = bytes - off < kSlotBytes ? bytes - off : kSlotBytes;
        if (g_rank == root) std::memcpy(g_seg->slots[0], b + off, n);
        barrier();
        if (g_rank != root) std::memcpy(b + off, g_seg->slots[0], n);
        barrier();
    }
    return MPI_SUCCESS;
}

int MPI_Allreduce(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op, MPI_Comm)
{
    const size_t bytes = (size_t)count * type_size(type);
    if (type_size(type) == 0 || type == MPI_BYTE || bytes > kSlotBytes) return MPI_ERR_OTHER;
    if (g_size == 1) { if (recv != send) std::memcpy(recv, send, bytes); return MPI_SUCCESS; }
    std::memcpy(g_seg->slots[g_rank], send, bytes);
    barrier();
    if (type == MPI_INT) reduce_into(static_cast<int*>(recv), count, op);
    else if (type == MPI_FLOAT) reduce_into(static_cast<float*>(recv), count, op);
    else reduce_into(static_cast<double*>(recv), count, op);
    barrier();
    return MPI_SUCCESS;
}

int MPI_Allgather(const void* send, int scount, MPI_Datatype stype, void* recv, int, MPI_Datatype, MPI_Comm)
{
    const size_t bytes = (size_t)scount * type_size(stype);
    if (type_size(stype) == 0 || bytes > kSlotBytes) return MPI_ERR_OTHER;
    if (g_size == 1) { std::memcpy(recv, send, bytes); return MPI_SUCCESS; }
    std::memcpy(g_seg->slots[g_rank], send, bytes);
    barrier();
    for (int r = 0; r < g_size; r++)
        std::memcpy(static_cast<unsigned char*>(recv) + (size_t)r * bytes, g_seg->slots[r], bytes);
    barrier();
    return MPI_SUCCESS;
}

double MPI_Wtime(void) { return wall(); }

int MPI_Abort(MPI_Comm, int code)
{
    fprintf(stderr, "mpi_shim: rank %d aborts with code %d\n", g_rank, code);
    die(code);
}

int MPI_Finalize(void)
{
    if (g_seg) {
        barrier();
        munmap(g_seg, sizeof(Segment));
        g_seg = nullptr;
    }
    return MPI_SUCCESS;
}

}  // extern "C"

// Size of the segment, for the launcher.
extern "C" unsigned long efa_shim_segment_bytes(void) { return (unsigned long)sizeof(Segment); }
