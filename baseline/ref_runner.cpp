// Timing / checking harness for the UNMODIFIED reference library (its src/*.cpp compiled against
// the MPI stand-in in mpi_shim/).  Calls the reference's public entry points exactly as its own
// drivers do (examples/rbruckv_example.cpp:96-131): per iteration a barrier, MPI_Wtime around the
// call on every rank, MPI_Allreduce(MAX) of the elapsed time.  The result is checked byte for byte
// against a direct-copy expectation after the last iteration.
//
// usage: ref_runner <algo> <P> <type_size> <counts_file> <iters> <warmup> [n r r2 b b2]
//   counts_file: P x P whitespace-separated integers, row s = elements rank s sends to each rank.
// Output: one JSON line on stdout (mean, median and minimum of the per-iteration maxima over ranks).
// With REF_SEND_DIR / REF_RECV_DIR in the environment rank r takes its (packed) send buffer from
// <REF_SEND_DIR>/send_<r>.bin and writes its receive buffer to <REF_RECV_DIR>/recv_<r>.bin, so that a test can
// compare the reference's receive bytes with another implementation's.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "rbruckv.h"  // the reference's header (pulls <mpi.h> = the stand-in)

namespace {

struct Job {
  std::string algo;
  int P = 0, ts = 4, iters = 10, warmup = 3;
  int n = 0, r = 2, r2 = 0, b = 0, b2 = 0;
  std::vector<int> counts;  // P*P
  // results
  std::vector<double> times;  // per timed iteration, max over ranks (seconds)
  std::vector<long long> errors;
  int rc = 0;
};

inline unsigned char pattern(int s, int d, size_t k) {
  unsigned x = (unsigned)s * 2654435761u ^ (unsigned)d * 40503u ^ (unsigned)k * 2246822519u;
  x ^= x >> 15;
  return (unsigned char)(x * 2654435761u >> 24);
}

int call(const Job& J, char* sb, int* sc, int* sd, char* rb, int* rc, int* rd, MPI_Datatype t) {
  const std::string& a = J.algo;
  MPI_Comm c = MPI_COMM_WORLD;
  if (a == "rbruck") return twophase_rbruck_alltoallv(J.r, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "rbruck_om") return twophase_rbruck_alltoallv_om(J.r, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "tuna") return tuna_algorithm(J.r, J.b, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "tuna2") return tuna2_algorithm(J.r, J.b, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "ttpl") return TTPL_rbruck_alltoallv(J.n, J.r, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "ttpl_bt") return TTPL_BT_alltoallv(J.n, J.r, J.b, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "ttpl_bt_s1") return TTPL_BT_alltoallv_s1(J.n, J.r, J.b, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "scattered") return MPICH_intra_scattered(J.b, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "linear") return ompi_alltoallv_intra_basic_linear(sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "pairwise") return ompi_alltoallv_intra_pairwise(sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "xor") return exclisive_or_alltoallv(sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "twolayer_linear") return twolayer_communicator_linear(J.n, sb, sc, sd, t, rb, rc, rd, t, c);
  if (a == "twolayer_linear_s2") {
    int e = twolayer_communicator_linear_s2(J.n, J.b, J.b2, sb, sc, sd, t, rb, rc, rd, t, c);
    return e;
  }
  if (a == "mpi_alltoallv") return MPI_Alltoallv(sb, sc, sd, t, rb, rc, rd, t, c);
  return -99;
}

void rank_main(int rank, int P, void* arg) {
  Job& J = *static_cast<Job*>(arg);
  const int ts = J.ts;
  // the reference moves MPI_CHAR bytes and uses the type only for its size; pick a type of that size
  MPI_Datatype t = ts == 1 ? MPI_CHAR : ts == 4 ? MPI_INT : ts == 8 ? MPI_UNSIGNED_LONG_LONG : MPI_CHAR;
  const int mult = (t == MPI_CHAR) ? ts : 1;  // element sizes without a matching type travel as bytes
  std::vector<int> sc(P), sd(P), rc(P), rd(P);
  long long stot = 0, rtot = 0;
  for (int i = 0; i < P; i++) {
    sc[i] = J.counts[(size_t)rank * P + i] * mult;
    rc[i] = J.counts[(size_t)i * P + rank] * mult;
    sd[i] = (int)stot; rd[i] = (int)rtot;
    stot += sc[i]; rtot += rc[i];
  }
  const size_t esz = (t == MPI_CHAR) ? 1 : (size_t)ts;
  std::vector<char> sb((size_t)stot * esz + 64), rb((size_t)rtot * esz + 64, (char)0xA5);
  for (int d = 0; d < P; d++) {
    size_t n = (size_t)sc[d] * esz, o = (size_t)sd[d] * esz;
    for (size_t k = 0; k < n; k++) sb[o + k] = (char)pattern(rank, d, k);
  }
  const char* send_dir = std::getenv("REF_SEND_DIR");
  const char* recv_dir = std::getenv("REF_RECV_DIR");
  if (send_dir) {
    std::ifstream f(std::string(send_dir) + "/send_" + std::to_string(rank) + ".bin", std::ios::binary);
    f.read(sb.data(), (std::streamsize)((size_t)stot * esz));
  }
  const bool twolayer_s2 = (J.algo == "twolayer_linear_s2");
  for (int it = 0; it < J.warmup + J.iters; it++) {
    MPI_Barrier(MPI_COMM_WORLD);
    double t0 = MPI_Wtime();
    int e = call(J, sb.data(), sc.data(), sd.data(), rb.data(), rc.data(), rd.data(), t);
    double el = MPI_Wtime() - t0, mx = 0;
    if (e != 0 && rank == 0) J.rc = e;
    MPI_Allreduce(&el, &mx, 1, MPI_DOUBLE, MPI_MAX, MPI_COMM_WORLD);
    if (twolayer_s2) {
      // the reference allocates iteration_time in every call and leaves freeing to the caller
      MPI_Barrier(MPI_COMM_WORLD);
      if (rank == 0 && iteration_time) { free(iteration_time); iteration_time = nullptr; }
      MPI_Barrier(MPI_COMM_WORLD);
    }
    if (rank == 0 && it >= J.warmup) J.times.push_back(mx);
  }
  long long bad = 0;
  if (!send_dir)
    for (int s = 0; s < P; s++) {
      size_t n = (size_t)rc[s] * esz, o = (size_t)rd[s] * esz;
      for (size_t k = 0; k < n; k++) bad += ((unsigned char)rb[o + k] != pattern(s, rank, k));
    }
  if (recv_dir) {
    std::ofstream f(std::string(recv_dir) + "/recv_" + std::to_string(rank) + ".bin", std::ios::binary);
    f.write(rb.data(), (std::streamsize)((size_t)rtot * esz));
  }
  J.errors[rank] = bad;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 7) {
    std::fprintf(stderr, "usage: %s <algo> <P> <type_size> <counts_file> <iters> <warmup> [n r r2 b b2]\n", argv[0]);
    return 2;
  }
  Job J;
  J.algo = argv[1];
  J.P = std::atoi(argv[2]);
  J.ts = std::atoi(argv[3]);
  J.iters = std::atoi(argv[5]);
  J.warmup = std::atoi(argv[6]);
  if (argc > 7) J.n = std::atoi(argv[7]);
  if (argc > 8) J.r = std::atoi(argv[8]);
  if (argc > 9) J.r2 = std::atoi(argv[9]);
  if (argc > 10) J.b = std::atoi(argv[10]);
  if (argc > 11) J.b2 = std::atoi(argv[11]);
  std::ifstream in(argv[4]);
  J.counts.resize((size_t)J.P * J.P);
  for (auto& v : J.counts)
    if (!(in >> v)) { std::fprintf(stderr, "bad counts file\n"); return 2; }
  J.errors.assign(J.P, 0);
  // The reference's TuNA loops forever for P <= 2 (radix clamped to 1, src/tuna.cpp:20,28).
  if ((J.algo == "tuna" || J.algo == "tuna2") && J.P <= 2) {
    std::printf("{\"impl\": \"reference\", \"algo\": \"%s\", \"P\": %d, \"unavailable\": \"reference TuNA does not terminate for P <= 2\"}\n",
                J.algo.c_str(), J.P);
    return 0;
  }
  shim_run(J.P, rank_main, &J);
  long long bad = 0, bytes = 0;
  for (auto e : J.errors) bad += e;
  for (auto c : J.counts) bytes += (long long)c * J.ts;
  std::vector<double> t = J.times;
  std::sort(t.begin(), t.end());
  double sum = 0;
  for (double v : J.times) sum += v;
  double mean = t.empty() ? 0 : sum / t.size(), med = t.empty() ? 0 : t[t.size() / 2], mn = t.empty() ? 0 : t[0];
  std::printf("{\"impl\": \"reference\", \"transport\": \"mpi_shim_threads\", \"algo\": \"%s\", \"P\": %d, \"type_size\": %d, "
              "\"iters\": %d, \"warmup\": %d, \"n\": %d, \"r\": %d, \"b\": %d, \"rc\": %d, \"mismatched_bytes\": %lld, "
              "\"total_bytes\": %lld, \"mean_us\": %.3f, \"median_us\": %.3f, \"min_us\": %.3f, \"sum_s\": %.9f}\n",
              J.algo.c_str(), J.P, J.ts, J.iters, J.warmup, J.n, J.r, J.b, J.rc, bad, bytes, mean * 1e6, med * 1e6,
              mn * 1e6, sum);
  return 0;
}
