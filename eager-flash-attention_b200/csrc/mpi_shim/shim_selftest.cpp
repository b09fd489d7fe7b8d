// shim_selftest: exercises the shared-memory MPI subset without a GPU (start with efa_launch -n R shim_selftest).
//   (no flag)          barrier, broadcast, max and min reductions, all-gather; every rank checks the results
//   --absent RANK      that rank leaves before the first barrier: the others must time out of it
//                      (EFA_SHIM_TIMEOUT_S) and exit non-zero instead of spinning forever
#include <mpi.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

int main(int argc, char** argv)
{
    int provided = 0, rank = 0, size = 1;
    if (MPI_Init_thread(&argc, &argv, MPI_THREAD_MULTIPLE, &provided) != MPI_SUCCESS) return 2;
    MPI_Comm_rank(MPI_COMM_WORLD, &rank);
    MPI_Comm_size(MPI_COMM_WORLD, &size);
    for (int i = 1; i + 1 < argc; i++)
        if (std::strcmp(argv[i], "--absent") == 0 && std::atoi(argv[i + 1]) == rank) {
            printf("rank %d leaves before the barrier\n", rank);
            fflush(stdout);
            _Exit(0);
        }
    MPI_Barrier(MPI_COMM_WORLD);
    int word = rank == 0 ? 1234567 : 0;
    MPI_Bcast(&word, 1, MPI_INT, 0, MPI_COMM_WORLD);
    double mine = 10.0 + rank, hi = 0.0;
    MPI_Allreduce(&mine, &hi, 1, MPI_DOUBLE, MPI_MAX, MPI_COMM_WORLD);
    int ok = (word == 1234567) && (hi == 10.0 + size - 1), all_ok = 0;
    unsigned char me = (unsigned char)(rank * 3 + 1), everyone[16];
    MPI_Allgather(&me, 1, MPI_BYTE, everyone, 1, MPI_BYTE, MPI_COMM_WORLD);
    for (int r = 0; r < size; r++) ok = ok && everyone[r] == (unsigned char)(r * 3 + 1);
    MPI_Allreduce(&ok, &all_ok, 1, MPI_INT, MPI_MIN, MPI_COMM_WORLD);
    if (rank == 0) printf("shim selftest %s on %d ranks\n", all_ok ? "passed" : "FAILED", size);
    MPI_Finalize();
    return all_ok ? 0 : 1;
}
