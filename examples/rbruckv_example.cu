// C++ usage of the library through its C API, shaped like the reference's examples/rbruckv_example.cpp:
// for n = 2, 4, ... elements per block, run tuna2_algorithm (b = 1) for every radix given on the command line,
// check the result with check_errors and print "[Rbruckv] P, n, b, base, seconds".
//
//   ./rbruckv_example <loop-count> <nranks> <base-list...>
//
// All `nranks` logical ranks live in this one process on GPU 0; every rank makes its own call, exactly like the
// ranks of an SPMD program would (the kernel starts when the last local rank has called).  With one process per
// GPU the same code runs with rbv_ctx_create(nranks, nproc, proc, ...) and an exchange of IPC handles.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "rbv/rbruckv.h"

int main(int argc, char** argv) {
  if (argc < 4) {
    std::printf("Usage: %s <loop-count> <nranks> <base-list>\n", argv[0]);
    return 1;
  }
  const int loops = std::atoi(argv[1]), P = std::atoi(argv[2]);
  std::vector<int> bases;
  for (int i = 3; i < argc; i++) bases.push_back(std::atoi(argv[i]));

  rbv_ctx_t ctx = rbv_ctx_create(P, /*nproc=*/1, /*proc=*/0, /*device=*/0, /*user bytes=*/256u << 20, /*arena=*/16u << 20);
  if (!ctx) { std::printf("context: %s\n", rbv_last_error()); return 1; }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  int failures = 0;

  for (int n = 2; n <= 2048; n *= 2) {
    // every rank sends n elements to every rank; payload of block (src -> dst): dst + 10 * src
    std::vector<int> counts(P, n), displs(P);
    for (int i = 0; i < P; i++) displs[i] = i * n;
    std::vector<char*> sb(P), rb(P);
    for (int r = 0; r < P; r++) {
      std::vector<long long> h((size_t)P * n);
      for (int d = 0; d < P; d++)
        for (int k = 0; k < n; k++) h[(size_t)d * n + k] = d + 10ll * r;
      cudaMalloc(&sb[r], h.size() * 8);
      cudaMemcpy(sb[r], h.data(), h.size() * 8, cudaMemcpyHostToDevice);
      rb[r] = static_cast<char*>(rbv_symm_alloc(ctx, h.size() * 8));
    }
    for (int base : bases) {
      double total = 0;
      for (int it = 0; it < loops; it++) {
        cudaEventRecord(e0, 0);
        for (int r = 0; r < P; r++) {
          int rc = tuna2_algorithm(base, 1, sb[r], counts.data(), displs.data(), RBV_UNSIGNED_LONG_LONG, rb[r],
                                   counts.data(), displs.data(), RBV_UNSIGNED_LONG_LONG, rbv_comm(ctx, r));
          if (rc) { std::printf("tuna2_algorithm returned %d: %s\n", rc, rbv_last_error()); return 1; }
        }
        cudaEventRecord(e1, 0);
        cudaEventSynchronize(e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        total += ms * 1e-3;
      }
      rbv_status st;
      if (rbv_ctx_status(ctx, &st)) { std::printf("device status %d\n", st.code); failures++; }
      for (int r = 0; r < P; r++) {
        std::vector<long long> h((size_t)P * n);
        cudaMemcpy(h.data(), rb[r], h.size() * 8, cudaMemcpyDeviceToHost);
        int err = check_errors(counts.data(), h.data(), r, P);
        if (err) { std::printf("[Rbruckv] %d %d has errors\n", base, n); failures++; }
      }
      std::printf("[Rbruckv] %d, %d, %d, %d, %.9f\n", P, n, 1, base, total / loops);
    }
    for (int r = 0; r < P; r++) { cudaFree(sb[r]); rbv_symm_free(ctx, rb[r]); }
  }
  rbv_ctx_destroy(ctx);
  return failures ? 1 : 0;
}
