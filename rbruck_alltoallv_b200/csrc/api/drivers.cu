// Native benchmark driver over the C API, shaped like the reference's example programs
// (examples/rbruckv_example.cpp, twophaseLayer_example.cpp, twophaseLayer_example2.cpp, twolayer_example.cpp,
// twophaseLayer_example4.cpp): sweep the block size n = nmin, 2 nmin, ... nmax, fill the send buffers with
// `dest + 10 * src` as 8-byte elements, call one collective through its reference-shaped entry point once per
// local rank, time it on the device, run check_errors on the result and print one line per measurement with the
// reference's tags ("[Rbruckv] P, n, b, base, seconds").  Differences on purpose: counts come from a seeded
// generator instead of the wall clock, the time is a CUDA-event time of the device work (the reference's
// MPI_Wtime span also contains its mallocs), and every call is also checked byte-exactly by the Python tests.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "api/ctx_internal.h"
#include "rbv/rbruckv.h"

namespace {

struct Lcg {  // small seeded generator: the drivers must be reproducible
  unsigned long long s;
  explicit Lcg(unsigned long long seed) : s(seed * 6364136223846793005ull + 1442695040888963407ull) {}
  unsigned next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (unsigned)(s >> 33); }
};

// counts[s][d] for all ranks; mode 0: constant n (shuffled order is irrelevant for constants), 1: n * (k % 100) / 100
void make_counts(std::vector<int>& c, int P, int n, int mode, unsigned long long seed) {
  c.assign((size_t)P * P, n);
  if (mode == 1) {
    Lcg g(seed);
    for (auto& v : c) v = (int)((long long)n * (g.next() % 100) / 100);
  }
}

typedef int (*CallFn)(const char* algo, int n_group, int radix, int b, int b2, char* sb, int* sc, int* sd, char* rb,
                      int* rc, int* rd, rbv_comm_t comm);

int call_algo(const char* algo, int ng, int r, int b, int b2, char* sb, int* sc, int* sd, char* rb, int* rc, int* rd,
              rbv_comm_t comm) {
  const rbv_datatype t = RBV_UNSIGNED_LONG_LONG;
  std::string a(algo);
  if (a == "tuna2") return tuna2_algorithm(r, b, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "tuna") return tuna_algorithm(r, b, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "rbruck") return twophase_rbruck_alltoallv(r, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "rbruck_om") return twophase_rbruck_alltoallv_om(r, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "scattered") return MPICH_intra_scattered(b, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "linear") return ompi_alltoallv_intra_basic_linear(sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "pairwise") return ompi_alltoallv_intra_pairwise(sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "xor") return exclisive_or_alltoallv(sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "spreadout") { spreadout_alltoallv(sb, sc, sd, t, rb, rc, rd, t, comm); return 0; }
  if (a == "ttpl") return TTPL_rbruck_alltoallv(ng, r, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "ttpl_bt") return TTPL_BT_alltoallv(ng, r, b, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "ttpl_bt_s1") return TTPL_BT_alltoallv_s1(ng, r, b, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "ttpl_bt_s2") return TTPL_BT_alltoallv_s2(ng, r, b, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "twolayer_linear") return twolayer_communicator_linear(ng, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "twolayer_linear_s2") return twolayer_communicator_linear_s2(ng, b, b2, sb, sc, sd, t, rb, rc, rd, t, comm);
  if (a == "twolayer_linear_s3") return twolayer_communicator_linear_s3(ng, b, b2, sb, sc, sd, t, rb, rc, rd, t, comm);
  return -99;
}

}  // namespace

// tag: printed in brackets, e.g. "Rbruckv", "MPICH_scattered", "TTPL_S1".  Returns the number of failed checks,
// or a negative value when a call was refused.  Lines go to `out` (stdout when null).
extern "C" int rbv_driver_sweep(rbv_ctx_t ctx, const char* tag, const char* algo, int loop_count, int warmup,
                                int n_group, int radix, int b, int b2, int nmin, int nmax, int count_mode,
                                unsigned long long seed, const char* out_path) {
  rbv::Context& c = *ctx->c;
  const int P = c.P(), L = c.L(), first = c.proc() * L;
  FILE* out = out_path && out_path[0] ? std::fopen(out_path, "a") : stdout;
  if (!out) return -1;
  int failures = 0;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (int n = nmin; n <= nmax; n *= 2) {
    std::vector<int> counts;
    make_counts(counts, P, n, count_mode, seed + (unsigned long long)n);
    // per local rank: host arrays (elements), device buffers
    std::vector<std::vector<int>> sc(L), sd(L), rc(L), rd(L);
    std::vector<char*> sb(L, nullptr), rb(L, nullptr);
    std::vector<std::vector<long long>> host_send(L);
    std::vector<long long> rtot(L, 0);
    bool alloc_ok = true;
    for (int lr = 0; lr < L; lr++) {
      const int me = first + lr;
      sc[lr].resize(P); sd[lr].resize(P); rc[lr].resize(P); rd[lr].resize(P);
      long long so = 0, ro = 0;
      for (int i = 0; i < P; i++) {
        sc[lr][i] = counts[(size_t)me * P + i]; rc[lr][i] = counts[(size_t)i * P + me];
        sd[lr][i] = (int)so; rd[lr][i] = (int)ro;
        so += sc[lr][i]; ro += rc[lr][i];
      }
      rtot[lr] = ro;
      host_send[lr].assign((size_t)so + 1, 0);
      for (int i = 0; i < P; i++)
        for (int k = 0; k < sc[lr][i]; k++) host_send[lr][(size_t)sd[lr][i] + k] = i + 10ll * me;
      if (cudaMalloc(&sb[lr], (size_t)(so + 1) * 8) != cudaSuccess) alloc_ok = false;
      rb[lr] = static_cast<char*>(rbv_symm_alloc(ctx, (size_t)(ro + 1) * 8));
      if (!rb[lr]) alloc_ok = false;
      if (alloc_ok) cudaMemcpy(sb[lr], host_send[lr].data(), (size_t)so * 8, cudaMemcpyHostToDevice);
    }
    if (!alloc_ok) { std::fprintf(out, "[%s] allocation failed at n = %d\n", tag, n); failures++; }
    double best = 1e30, sum = 0;
    int rcode = 0;
    for (int it = 0; alloc_ok && it < warmup + loop_count; it++) {
      for (int lr = 0; lr < L; lr++) cudaMemsetAsync(rb[lr], 0, (size_t)rtot[lr] * 8, ctx->stream);
      cudaEventRecord(e0, ctx->stream);
      for (int lr = 0; lr < L; lr++) {
        int e = call_algo(algo, n_group, radix, b, b2, sb[lr], sc[lr].data(), sd[lr].data(), rb[lr], rc[lr].data(),
                          rd[lr].data(), rbv_comm(ctx, lr));
        if (e) rcode = e;
      }
      cudaEventRecord(e1, ctx->stream);
      if (rcode) break;
      cudaEventSynchronize(e1);
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      if (it >= warmup) { sum += ms * 1e-3; if (ms * 1e-3 < best) best = ms * 1e-3; }
    }
    if (rcode) {
      std::fprintf(out, "[%s] %d, %d, %d, %d, refused with code %d: %s\n", tag, P, n, b, radix, rcode, rbv_last_error());
      failures = failures ? failures : -1;
    } else if (alloc_ok) {
      rbv_status st;
      int code = rbv_ctx_status(ctx, &st);
      int errors = 0;
      for (int lr = 0; lr < L; lr++) {
        std::vector<long long> h((size_t)rtot[lr] + 1);
        cudaMemcpy(h.data(), rb[lr], (size_t)rtot[lr] * 8, cudaMemcpyDeviceToHost);
        errors += check_errors(rc[lr].data(), h.data(), first + lr, P);
      }
      if (code || errors) {
        failures++;
        std::fprintf(out, "[%s] %d %d has errors (%d bad elements, device status %d)\n", tag, P, n, errors, code);
      }
      // the reference prints: tag, nprocs, n, block count, base, max time in seconds
      std::fprintf(out, "[%s] %d, %d, %d, %d, %.9f\n", tag, P, n, b, radix, loop_count > 0 ? sum / loop_count : 0.0);
    }
    for (int lr = 0; lr < L; lr++) {
      if (sb[lr]) cudaFree(sb[lr]);
      if (rb[lr]) rbv_symm_free(ctx, rb[lr]);
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (out != stdout) std::fclose(out);
  return failures;
}
