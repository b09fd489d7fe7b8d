/* A ten-function subset of MPI for single-host runs, one process per GPU, when no MPI
 * installation exists: exactly the calls the attention-block drivers make (initialisation, rank and
 * size, barrier, broadcast of bytes, max/min all-reduce of a scalar, wall clock, abort, finalise).
 * Backed by a POSIX shared-memory segment; ranks are started by efa_launch, which sets
 * EFA_SHIM_RANK, EFA_SHIM_SIZE and EFA_SHIM_NAME. Without those variables the process is a world
 * of one rank. Only host buffers are supported.
 */
#ifndef EFA_MPI_SHIM_H
#define EFA_MPI_SHIM_H

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;

#define MPI_COMM_WORLD      0
#define MPI_SUCCESS         0
#define MPI_ERR_OTHER       15
#define MPI_THREAD_MULTIPLE 3

#define MPI_BYTE   1
#define MPI_INT    2
#define MPI_DOUBLE 3
#define MPI_FLOAT  4

#define MPI_MAX 1
#define MPI_MIN 2
#define MPI_SUM 3

int    MPI_Init_thread(int* argc, char*** argv, int required, int* provided);
int    MPI_Init(int* argc, char*** argv);
int    MPI_Comm_rank(MPI_Comm comm, int* rank);
int    MPI_Comm_size(MPI_Comm comm, int* size);
int    MPI_Barrier(MPI_Comm comm);
int    MPI_Bcast(void* buf, int count, MPI_Datatype type, int root, MPI_Comm comm);
int    MPI_Allreduce(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op, MPI_Comm comm);
int    MPI_Allgather(const void* send, int scount, MPI_Datatype stype, void* recv, int rcount, MPI_Datatype rtype, MPI_Comm comm);
double MPI_Wtime(void);
int    MPI_Abort(MPI_Comm comm, int code);
int    MPI_Finalize(void);

#ifdef __cplusplus
}
#endif
#endif
