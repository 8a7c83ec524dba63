// Runs every algorithm of the plan compiler and the CPU executor on small ragged problems.  Built with
// -fsanitize=address,undefined by tests/test_sanitizers.py: any out-of-bounds access, leak or undefined
// behaviour in the host code ends the program with a non-zero exit code.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "rbv/plan.h"

using namespace rbv;

static int run_one(const AlgoSpec& spec, int ts, unsigned seed) {
  Plan plan = build_plan(spec);
  if (plan.err) return 0;   // argument errors are a valid outcome; they must not touch memory either
  const int P = spec.P;
  std::mt19937 rng(seed);
  std::vector<int> counts((size_t)P * P);
  for (auto& c : counts) c = plan.uniform ? 5 : (int)(rng() % 9);
  std::vector<std::vector<char>> send(P), recv(P), want(P);
  std::vector<long long> sd((size_t)P * P), rd((size_t)P * P);
  for (int s = 0; s < P; s++) {
    long long off = 0;
    for (int d = 0; d < P; d++) { sd[(size_t)s * P + d] = off; off += counts[(size_t)s * P + d]; }
    send[s].resize((size_t)off * ts + 1);
    for (auto& b : send[s]) b = (char)(rng() & 0xff);
  }
  for (int d = 0; d < P; d++) {
    long long off = 0;
    for (int s = 0; s < P; s++) { rd[(size_t)d * P + s] = off; off += counts[(size_t)s * P + d]; }
    recv[d].assign((size_t)off * ts + 1, (char)0x5a);
    want[d] = recv[d];
    for (int s = 0; s < P; s++)
      std::memcpy(want[d].data() + rd[(size_t)d * P + s] * ts, send[s].data() + sd[(size_t)s * P + d] * ts,
                  (size_t)counts[(size_t)s * P + d] * ts);
  }
  std::vector<const char*> sp(P);
  std::vector<char*> rp(P);
  for (int i = 0; i < P; i++) { sp[i] = send[i].data(); rp[i] = recv[i].data(); }
  int rc = host_execute(plan, ts, sp.data(), rp.data(), counts.data(), sd.data(), rd.data());
  if (rc) { std::printf("executor rc %d for algo %d P %d\n", rc, (int)spec.algo, P); return 1; }
  for (int d = 0; d < P; d++)
    if (recv[d] != want[d]) { std::printf("mismatch algo %d P %d rank %d\n", (int)spec.algo, P, d); return 1; }
  return 0;
}

int main() {
  int bad = 0, ran = 0;
  for (int algo = 0; algo < ALG_COUNT; algo++)
    for (int P : {1, 2, 3, 6, 8, 12})
      for (int n : {1, 2, 3, 4})
        for (int r : {1, 2, 3, 9})
          for (int b : {0, 1, 3}) {
            AlgoSpec s{};
            s.algo = (Algo)algo; s.P = P; s.n = n; s.r = r; s.r2 = r; s.b = b; s.b2 = b;
            bad += run_one(s, 1 + (ran % 3) * 3, 1234u + ran);
            ran++;
          }
  std::printf("ran %d cases, %d bad\n", ran, bad);
  return bad ? 1 : 0;
}
