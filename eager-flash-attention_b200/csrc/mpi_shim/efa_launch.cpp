// efa_launch -n R [--] program args... : start R copies of a program on this host as ranks of the
// shared-memory MPI subset (mpi.h). Plays the part srun plays for eager-flash-attention
// (bench_sweep.py:42-63, perlmutter/tests.sbatch). Exit code: the first non-zero exit code of a
// rank, else 0. When one rank fails the others are told through the segment and then signalled.
#include <fcntl.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

extern "C" unsigned long efa_shim_segment_bytes(void);

int main(int argc, char** argv)
{
    int n = 1;
    int i = 1;
    while (i < argc) {
        if (std::strcmp(argv[i], "-n") == 0 && i + 1 < argc) { n = std::atoi(argv[i + 1]); i += 2; }
        else if (std::strcmp(argv[i], "--") == 0) { i++; break; }
        else break;
    }
    if (i >= argc || n < 1 || n > 16) {
        fprintf(stderr, "usage: %s -n R [--] program [args...]   (1 <= R <= 16)\n", argv[0]);
        return 2;
    }
    char name[64];
    snprintf(name, sizeof(name), "/efa_shim_%d", (int)getpid());
    int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) { perror("efa_launch: shm_open"); return 1; }
    const unsigned long bytes = efa_shim_segment_bytes();
    if (ftruncate(fd, (off_t)bytes) != 0) { perror("efa_launch: ftruncate"); shm_unlink(name); return 1; }
    void* seg = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (seg == MAP_FAILED) { perror("efa_launch: mmap"); shm_unlink(name); return 1; }
    std::memset(seg, 0, bytes);

    std::vector<pid_t> pids;
    for (int r = 0; r < n; r++) {
        pid_t pid = fork();
        if (pid < 0) { perror("efa_launch: fork"); break; }
        if (pid == 0) {
            setenv("EFA_SHIM_RANK", std::to_string(r).c_str(), 1);
            setenv("EFA_SHIM_SIZE", std::to_string(n).c_str(), 1);
            setenv("EFA_SHIM_NAME", name, 1);
            execvp(argv[i], argv + i);
            perror("efa_launch: execvp");
            _exit(127);
        }
        pids.push_back(pid);
    }
    int rc = ((int)pids.size() == n) ? 0 : 1;
    size_t left = pids.size();
    while (left > 0) {
        int st = 0;
        pid_t done = wait(&st);
        if (done < 0) break;
        left--;
        int code = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + (WIFSIGNALED(st) ? WTERMSIG(st) : 0);
        if (code != 0 && rc == 0) {
            rc = code;
            // third int of the segment is the abort flag read by every waiting rank
            reinterpret_cast<volatile int*>(seg)[2] = 1;
            sleep(2);
            for (pid_t p : pids) if (p != done) kill(p, SIGTERM);
        }
    }
    munmap(seg, bytes);
    shm_unlink(name);
    return rc;
}
