// Exercises the threads-as-ranks MPI stand-in under ThreadSanitizer: point-to-point in both blocking and
// non-blocking forms, the collectives the reference uses, and communicator splitting.  A data race in the
// mailboxes or barriers makes ThreadSanitizer end the program with a non-zero exit code.
#include <cstdio>
#include <vector>

#include "mpi.h"

static int g_bad = 0;

static void rank_main(int, int, void*) {
  int rank, P;
  MPI_Comm_rank(MPI_COMM_WORLD, &rank);
  MPI_Comm_size(MPI_COMM_WORLD, &P);
  for (int iter = 0; iter < 20; iter++) {
    // ring exchange, non-blocking
    std::vector<int> out(64, rank * 1000 + iter), in(64, -1);
    MPI_Request rq[2];
    MPI_Irecv(in.data(), 64, MPI_INT, (rank + P - 1) % P, iter, MPI_COMM_WORLD, &rq[0]);
    MPI_Isend(out.data(), 64, MPI_INT, (rank + 1) % P, iter, MPI_COMM_WORLD, &rq[1]);
    MPI_Waitall(2, rq, MPI_STATUSES_IGNORE);
    if (in[0] != ((rank + P - 1) % P) * 1000 + iter) __atomic_fetch_add(&g_bad, 1, __ATOMIC_RELAXED);
    // pairwise, blocking
    int peer = rank ^ 1, got = -1, mine = rank + iter;
    if (peer < P) {
      MPI_Sendrecv(&mine, 1, MPI_INT, peer, 77, &got, 1, MPI_INT, peer, 77, MPI_COMM_WORLD, MPI_STATUS_IGNORE);
      if (got != peer + iter) __atomic_fetch_add(&g_bad, 1, __ATOMIC_RELAXED);
    }
    // collectives
    int mx = 0;
    MPI_Allreduce(&mine, &mx, 1, MPI_INT, MPI_MAX, MPI_COMM_WORLD);
    if (mx != P - 1 + iter) __atomic_fetch_add(&g_bad, 1, __ATOMIC_RELAXED);
    std::vector<int> a2a_s(P), a2a_r(P, -1);
    for (int i = 0; i < P; i++) a2a_s[i] = rank * P + i;
    MPI_Alltoall(a2a_s.data(), 1, MPI_INT, a2a_r.data(), 1, MPI_INT, MPI_COMM_WORLD);
    for (int i = 0; i < P; i++)
      if (a2a_r[i] != i * P + rank) __atomic_fetch_add(&g_bad, 1, __ATOMIC_RELAXED);
    // sub-communicators, as the two-layer algorithms make them
    MPI_Comm sub;
    MPI_Comm_split(MPI_COMM_WORLD, rank / 2, rank, &sub);
    int sr, ss, sum = 0;
    MPI_Comm_rank(sub, &sr);
    MPI_Comm_size(sub, &ss);
    MPI_Allreduce(&rank, &sum, 1, MPI_INT, MPI_SUM, sub);
    int base = (rank / 2) * 2, want = 0;
    for (int i = 0; i < ss; i++) want += base + i;
    if (sum != want) __atomic_fetch_add(&g_bad, 1, __ATOMIC_RELAXED);
    MPI_Comm_free(&sub);
    MPI_Barrier(MPI_COMM_WORLD);
  }
}

int main() {
  shim_run(6, rank_main, nullptr);
  std::printf("bad %d\n", g_bad);
  return g_bad ? 1 : 0;
}
