// C ABI over the host-only parts (plan compiler, CPU executor, integer helpers) for ctypes.
#include <cstring>
#include <vector>

#include "rbv/plan.h"

using namespace rbv;

extern "C" {

void* rbv_plan_create(int algo, int P, int n, int r, int r2, int b, int b2) {
  AlgoSpec s;
  s.algo = algo; s.P = P; s.n = n; s.r = r; s.r2 = r2; s.b = b; s.b2 = b2;
  return new Plan(build_plan(s));
}
void rbv_plan_destroy(void* p) { delete static_cast<Plan*>(p); }
int rbv_plan_err(void* p) { return static_cast<Plan*>(p)->err; }
const char* rbv_plan_errmsg(void* p) { return static_cast<Plan*>(p)->errmsg.c_str(); }
int rbv_plan_ncells(void* p) { return static_cast<Plan*>(p)->ncells; }
long long rbv_plan_nops(void* p) { return (long long)static_cast<Plan*>(p)->ops.size(); }
const void* rbv_plan_ops(void* p) { return static_cast<Plan*>(p)->ops.data(); }
int rbv_plan_uniform(void* p) { return static_cast<Plan*>(p)->uniform ? 1 : 0; }
int rbv_plan_inplace_ok(void* p) { return static_cast<Plan*>(p)->inplace_ok ? 1 : 0; }
// out[0..6] = w, K, w2, K2, max_blocks_per_round, phases, hops (low 31 bits)
void rbv_plan_stats(void* p, long long* out) {
  const PlanStats& s = static_cast<Plan*>(p)->stats;
  out[0] = s.w; out[1] = s.K; out[2] = s.w2; out[3] = s.K2;
  out[4] = s.max_blocks_per_round; out[5] = s.phases; out[6] = s.hops;
}
// out[0..6] = algo, P, n, r, r2, b, b2 after clamping
void rbv_plan_spec(void* p, int* out) {
  const AlgoSpec& s = static_cast<Plan*>(p)->spec;
  out[0] = s.algo; out[1] = s.P; out[2] = s.n; out[3] = s.r; out[4] = s.r2; out[5] = s.b; out[6] = s.b2;
}
const char* rbv_algo_name(int algo) { return algo_name(algo); }
int rbv_algo_from_name(const char* name) { return algo_from_name(name); }
int rbv_algo_count() { return ALG_COUNT; }

int rbv_host_alltoallv(void* plan, int type_size, const char* const* sendbufs, char* const* recvbufs,
                       const int* sendcounts, const long long* sdispls, const long long* rdispls) {
  Plan* pl = static_cast<Plan*>(plan);
  if (pl->err) return pl->err;
  return host_execute(*pl, type_size, sendbufs, recvbufs, sendcounts, sdispls, rdispls);
}

int rbv_ipow(int x, unsigned p) { return ipow(x, p); }
int rbv_ndigits(int v, int r) { return ndigits(v, r); }
int rbv_to_base(int w, int N, int b, int* out) {
  std::vector<int> v = to_base(w, N, b);
  for (size_t i = 0; i < v.size(); i++) out[i] = v[i];
  return (int)v.size();
}

}  // extern "C"
