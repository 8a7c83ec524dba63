// Schedule compiler: turns (algorithm, P, n, r, b, ...) into the ordered op list described in
// rbv/plan.h.  Pure host C++, no CUDA dependency, so it is unit-tested on machines without a GPU.
#include "rbv/plan.h"

#include <algorithm>
#include <array>
#include <cstring>
#include <map>

namespace rbv {

static const char* kAlgoNames[ALG_COUNT] = {
    "linear",          "spreadout",        "scattered",        "pairwise",
    "xor",             "twolayer_linear",  "twolayer_linear_s2", "twolayer_linear_s3",
    "twolayer_linear_s4", "rbruck",        "rbruck_om",        "tuna",
    "tuna2",           "ttpl",             "ttpl_bt",          "ttpl_bt_s1",
    "ttpl_bt_s2",      "uniform_spreadout_twolayer", "uniform_isplit_rbruck",
    "merge",           "simple_merge",     "split"};

const char* algo_name(int algo) {
  return (algo >= 0 && algo < ALG_COUNT) ? kAlgoNames[algo] : "unknown";
}
int algo_from_name(const char* name) {
  for (int i = 0; i < ALG_COUNT; i++)
    if (std::strcmp(name, kAlgoNames[i]) == 0) return i;
  return -1;
}

int ipow(int x, unsigned p) {
  long long res = 1, base = x;
  while (p) {
    if (p & 1) res *= base;
    base *= base;
    p >>= 1;
  }
  return (int)res;
}

int ndigits(int v, int r) {
  int w = 0;
  while (v > 0) { w++; v /= r; }
  return w;
}

std::vector<int> to_base(int w, int N, int b) {
  std::vector<int> v(w > 0 ? w : 0, 0);
  int i = 0;
  while (N && i < w) { v[i++] = N % b; N /= b; }
  return v;
}

namespace {

inline int mod(int a, int m) { int x = a % m; return x < 0 ? x + m : x; }

struct TmpOp { Op op; uint64_t order; };

struct Builder {
  Plan& pl;
  int P;
  std::vector<TmpOp> tmp;
  std::map<std::array<int, 4>, int> cells;
  explicit Builder(Plan& p) : pl(p), P(p.spec.P) {}

  int cell(int a, int b, int c, int d) {
    std::array<int, 4> k{a, b, c, d};
    auto it = cells.find(k);
    if (it != cells.end()) return it->second;
    int id = (int)cells.size();
    cells[k] = id;
    return id;
  }
  // phase: coarse stage (0 self copy, 1 intra / flat rounds, 2 inter, 3 trailing self copy);
  // step: round or batch index inside the phase; sub: order inside one step.
  void emit(int phase, int step, uint32_t sub, int src, int dst, int S, int D, int sc, int dc,
            uint32_t flags = 0) {
    TmpOp t;
    t.op.src = (uint16_t)src; t.op.dst = (uint16_t)dst;
    t.op.origin = (uint16_t)S; t.op.dest = (uint16_t)D;
    t.op.src_cell = sc; t.op.dst_cell = dc;
    t.op.key = ((uint32_t)phase << 24) | (uint32_t)(step & 0xffffff);
    t.op.flags = flags;
    t.order = ((uint64_t)t.op.key << 32) | sub;
    tmp.push_back(t);
  }
  void self_copy(int R, int phase = 0) { emit(phase, 0, 0, R, R, R, R, -1, -1, 1u); }
  void direct(int phase, int step, uint32_t sub, int R, int T) {
    if (R == T) emit(phase, step, sub, R, R, R, R, -1, -1, 1u);
    else emit(phase, step, sub, R, T, R, T, -1, -1);
  }
  void finish() {
    std::stable_sort(tmp.begin(), tmp.end(),
                     [](const TmpOp& a, const TmpOp& b) { return a.order < b.order; });
    pl.ops.reserve(tmp.size());
    for (auto& t : tmp) {
      if (pl.keys.empty() || pl.keys.back() != t.op.key) pl.keys.push_back(t.op.key);
      t.op.flags = (t.op.flags & 0xffffu) | ((uint32_t)(pl.keys.size() - 1) << 16);
      pl.ops.push_back(t.op);
      if (!(t.op.flags & 1u)) pl.stats.hops++;
    }
    pl.stats.phases = (int)pl.keys.size();
    pl.ncells = (int)cells.size();
    check_coverage();
  }
  // Every (origin, destination) pair must leave its origin exactly once per call (in `nparts` slices when the
  // block is split), and every rank copies its own block exactly once.
  void check_coverage() {
    if (pl.keys.size() > 65535u) { pl.err = -13; pl.errmsg = "too many distinct issue keys"; return; }
    std::vector<int> seen((size_t)P * P, 0), want((size_t)P * P, 1);
    for (const Op& o : pl.ops) {
      if (o.src_cell >= 0) continue;
      if (o.origin != o.src) { pl.err = -13; pl.errmsg = "first hop executed by a rank that is not the origin"; return; }
      const size_t i = (size_t)o.origin * P + o.dest;
      seen[i]++;
      if (op_nparts(o)) want[i] = (int)op_nparts(o);
    }
    for (size_t i = 0; i < seen.size(); i++)
      if (seen[i] != want[i]) {
        pl.err = -13;
        pl.errmsg = "schedule does not send block " + std::to_string(i / P) + " -> " + std::to_string(i % P) +
                    " exactly once";
        return;
      }
  }
};

struct Round { int x, z; };

// Rounds of a radix-r Bruck over m members, low digit first; z*r^x < m keeps only the top-digit
// values that occur (the reference's K = w(r-1) - d, src/tuna.cpp:28-31, in integer arithmetic).
std::vector<Round> bruck_rounds(int m, int r, bool high_to_low) {
  std::vector<Round> rs;
  if (m <= 1) return rs;
  int w = ndigits(m - 1, r);
  for (int x = 0; x < w; x++)
    for (int z = 1; z < r; z++)
      if ((long long)z * ipow(r, x) < m) rs.push_back({x, z});
  if (high_to_low) std::reverse(rs.begin(), rs.end());
  return rs;
}

inline int digit(int j, int x, int r) { return (j / ipow(r, x)) % r; }
inline int top_digit_pos(int v, int r) {  // position of the highest non-zero digit, -1 for 0
  int p = -1, x = 0;
  while (v) { if (v % r) p = x; v /= r; x++; }
  return p;
}
inline int low_digit_pos(int v, int r) {  // position of the lowest non-zero digit, -1 for 0
  int x = 0;
  if (!v) return -1;
  while (v % r == 0) { v /= r; x++; }
  return x;
}

// State of relative block j when a member executes round (x, z) with digit_x(j) == z.
struct Hop {
  int L;         // distance already travelled (toward lower member ids)
  bool first;    // block still sits at its origin
  bool final_;   // this hop reaches the block's last member
  int prev;      // digit position of the hop that delivered the block here (when !first)
};
inline Hop hop_state(int j, int x, int r, bool high_to_low) {
  Hop h;
  int px = ipow(r, x);
  if (!high_to_low) {
    h.L = j % px;
    h.final_ = (j / px) / r == 0;
    h.prev = top_digit_pos(h.L, r);
  } else {
    int hi = (j / px / r) * px * r;
    h.L = hi;
    h.final_ = (j % px) == 0;
    h.prev = low_digit_pos(hi, r);
  }
  h.first = (h.L == 0);
  return h;
}

int blocks_in_round(int m, int r, int x, int z) {
  int c = 0;
  for (int j = 1; j < m; j++) if (digit(j, x, r) == z) c++;
  return c;
}

// ---------------------------------------------------------------------------------------------
// Flat radix-r Bruck family (reference: src/twophase_tunable_rbruckv.cpp, -om.cpp, tuna.cpp,
// tuna2.cpp).  Relative block j on member q was sent by S = q + L and is bound for D = S - j; one
// hop of round (x, z) moves it to q - z*r^x.  The relative index is preserved across hops.
// ---------------------------------------------------------------------------------------------
void build_flat_bruck(Builder& B, int r, bool high_to_low, int batch, bool interleave) {
  const int P = B.P;
  for (int R = 0; R < P; R++) B.self_copy(R);
  auto rounds = bruck_rounds(P, r, high_to_low);
  B.pl.stats.w = P > 1 ? ndigits(P - 1, r) : 0;
  B.pl.stats.K = (int)rounds.size();
  // step index of every round: one step per round (batch == 0) or one per batch of `batch` rounds
  // of the same digit (TuNA, src/tuna.cpp:69-72).
  std::vector<int> step(rounds.size());
  {
    int s = -1, curx = -2, inb = 0;
    for (size_t i = 0; i < rounds.size(); i++) {
      if (batch <= 0) { step[i] = (int)i; continue; }
      if (rounds[i].x != curx || inb == batch) { s++; inb = 0; curx = rounds[i].x; }
      step[i] = s; inb++;
    }
  }
  for (size_t ri = 0; ri < rounds.size(); ri++) {
    const int x = rounds[ri].x, z = rounds[ri].z;
    const int sp = z * ipow(r, x);
    B.pl.stats.max_blocks_per_round =
        std::max(B.pl.stats.max_blocks_per_round, blocks_in_round(P, r, x, z));
    for (int q = 0; q < P; q++) {
      const int t = mod(q - sp, P);
      int i = 0;
      for (int j = 1; j < P; j++) {
        if (digit(j, x, r) != z) continue;
        Hop h = hop_state(j, x, r, high_to_low);
        int S = mod(q + h.L, P), D = mod(S - j, P);
        int sc = h.first ? -1 : B.cell(0, j, h.prev, 0);
        int dc = h.final_ ? -1 : B.cell(0, j, x, 0);
        uint32_t sub = interleave ? ((uint32_t)i << 12 | (uint32_t)z) : ((uint32_t)z << 16 | (uint32_t)i);
        B.emit(1, step[ri], sub, q, t, S, D, sc, dc);
        i++;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Hierarchical family (reference: src/twophase_twolayer_rbruck.cpp, src/twolayer_rbruck.cpp).
// Intra phase: Bruck over the n members of a group that carries, per relative index j, one block
// for every destination group g.  Afterwards rank (gid, q) holds, for every (g, lr), the block
// from (gid, lr) bound for (g, q).  The inter phase moves it along the "rail" to (g, q).
// ---------------------------------------------------------------------------------------------
struct Hier { int n, G, r; };

void build_intra(Builder& B, const Hier& H) {
  const int n = H.n, G = H.G, r = H.r;
  auto rounds = bruck_rounds(n, r, false);
  B.pl.stats.w = n > 1 ? ndigits(n - 1, r) : 0;
  B.pl.stats.K = (int)rounds.size();
  for (size_t ri = 0; ri < rounds.size(); ri++) {
    const int x = rounds[ri].x, z = rounds[ri].z;
    const int sp = z * ipow(r, x);
    B.pl.stats.max_blocks_per_round =
        std::max(B.pl.stats.max_blocks_per_round, G * blocks_in_round(n, r, x, z));
    for (int gid = 0; gid < G; gid++)
      for (int q = 0; q < n; q++) {
        const int me = gid * n + q, t = gid * n + mod(q - sp, n);
        uint32_t sub = 0;
        for (int g = 0; g < G; g++)
          for (int j = 1; j < n; j++) {
            if (digit(j, x, r) != z) continue;
            Hop h = hop_state(j, x, r, false);
            int Sl = mod(q + h.L, n), Dl = mod(Sl - j, n);
            int S = gid * n + Sl, D = g * n + Dl;
            int sc = h.first ? -1 : B.cell(1, g, j, h.prev);
            int dc = (h.final_ && g == gid) ? -1 : B.cell(1, g, j, x);
            B.emit(1, (int)ri, sub++, me, t, S, D, sc, dc);
          }
      }
  }
}

// Where the block from (gid, lr) bound for (g, q) rests on rank (gid, q) after the intra phase.
int intra_result_cell(Builder& B, const Hier& H, int q, int g, int lr) {
  if (lr == q) return -1;  // still in the send buffer
  int j = mod(lr - q, H.n);
  return B.cell(1, g, j, top_digit_pos(j, H.r));
}

void build_inter_direct(Builder& B, const Hier& H, int algo, int bblock) {
  const int n = H.n, G = H.G, P = n * G;
  const bool coalesced = (algo == ALG_TTPL_BT || algo == ALG_UNIFORM_SPREADOUT_TWOLAYER);
  if (coalesced) { if (bblock <= 0 || bblock > G) bblock = G; }
  else           { if (bblock <= 0 || bblock > P) bblock = P; }
  for (int gid = 0; gid < G; gid++)
    for (int q = 0; q < n; q++) {
      const int me = gid * n + q;
      if (coalesced) {
        // one message per destination group = its n blocks back to back
        // (src/twophase_twolayer_rbruck.cpp:430-453)
        for (int i = 0; i < G; i++) {
          int nd = mod(gid - i, G);
          if (nd == gid) continue;  // own group: delivered by the intra phase already
          for (int lr = 0; lr < n; lr++)
            B.emit(2, i / bblock, (uint32_t)(i * n + lr), me, nd * n + q, gid * n + lr, nd * n + q,
                   intra_result_cell(B, H, q, nd, lr), -1);
        }
      } else {
        // one message per (group, source local rank), flat index over all P
        // (src/twophase_twolayer_rbruck.cpp:634-671)
        for (int f = 0; f < P; f++) {
          int gi = f / n, lr = f % n, nd = mod(gid - gi, G);
          if (nd == gid) continue;
          B.emit(2, f / bblock, (uint32_t)f, me, nd * n + q, gid * n + lr, nd * n + q,
                 intra_result_cell(B, H, q, nd, lr), -1);
        }
      }
    }
}

// Inter-group Bruck on super-blocks of n blocks (completes what
// src/twophase_twolayer_rbruck.cpp:178-227 starts; also the inter phase of
// src/twolayer_rbruck.cpp:243-274).
void build_inter_bruck(Builder& B, const Hier& H, int r2) {
  const int n = H.n, G = H.G;
  auto rounds = bruck_rounds(G, r2, false);
  B.pl.stats.w2 = G > 1 ? ndigits(G - 1, r2) : 0;
  B.pl.stats.K2 = (int)rounds.size();
  for (size_t ri = 0; ri < rounds.size(); ri++) {
    const int x = rounds[ri].x, z = rounds[ri].z;
    const int sp = z * ipow(r2, x);
    for (int gq = 0; gq < G; gq++)
      for (int q = 0; q < n; q++) {
        const int me = gq * n + q, t = mod(gq - sp, G) * n + q;
        uint32_t sub = 0;
        for (int jg = 1; jg < G; jg++) {
          if (digit(jg, x, r2) != z) continue;
          Hop h = hop_state(jg, x, r2, false);
          int Sg = mod(gq + h.L, G), Dg = mod(Sg - jg, G);
          for (int lr = 0; lr < n; lr++) {
            int sc = h.first ? intra_result_cell(B, H, q, Dg, lr) : B.cell(2, lr, jg, h.prev);
            int dc = h.final_ ? -1 : B.cell(2, lr, jg, x);
            B.emit(2, (int)ri, sub++, me, t, Sg * n + lr, Dg * n + q, sc, dc);
          }
        }
      }
  }
}

void build_hier(Builder& B, const AlgoSpec& s) {
  Hier H{s.n, s.P / s.n, s.r};
  const bool self_last = (s.algo == ALG_TTPL_BT_S2);
  if (!self_last) for (int R = 0; R < s.P; R++) B.self_copy(R);
  build_intra(B, H);
  switch (s.algo) {
    case ALG_TTPL:
      build_inter_bruck(B, H, std::max(2, std::min(s.r, H.G)));
      break;
    case ALG_UNIFORM_ISPLIT_RBRUCK:
      build_inter_bruck(B, H, s.r2);
      break;
    default:
      build_inter_direct(B, H, s.algo, s.b);
  }
  if (self_last) for (int R = 0; R < s.P; R++) B.self_copy(R, 3);
}

// ---------------------------------------------------------------------------------------------
// Direct (single hop) family.
// ---------------------------------------------------------------------------------------------
void build_direct(Builder& B, const AlgoSpec& s) {
  const int P = s.P;
  switch (s.algo) {
    case ALG_LINEAR:  // self copy, then destinations in rank order (src/OpenMPI_basic_linear.cpp:28-63)
      for (int R = 0; R < P; R++) {
        B.self_copy(R);
        for (int T = 0; T < P; T++) if (T != R) B.direct(1, 0, (uint32_t)T, R, T);
      }
      break;
    case ALG_SPREADOUT:  // i-th send goes to rank - i, everything posted at once (benchmarks/common.cpp:10-37)
      for (int R = 0; R < P; R++)
        for (int i = 0; i < P; i++) B.direct(1, 0, (uint32_t)i, R, mod(R - i, P));
      break;
    case ALG_SCATTERED:  // spread-out order in batches of bblock (src/MPICH_scattered.cpp:38-70)
      for (int R = 0; R < P; R++)
        for (int i = 0; i < P; i++) B.direct(1, i / s.b, (uint32_t)i, R, mod(R - i, P));
      break;
    case ALG_PAIRWISE:  // step s sends to rank + s (src/OpenMPI_pairwise.cpp:32-58)
      for (int R = 0; R < P; R++)
        for (int st = 0; st < P; st++) B.direct(1, st, 0, R, mod(R + st, P));
      break;
    case ALG_XOR:  // step s exchanges with rank ^ s (src/exclusive_or_alltoallv.cpp:40-46)
      for (int R = 0; R < P; R++)
        for (int st = 0; st < P; st++) B.direct(1, st, 0, R, R ^ st);
      break;
    default: break;
  }
}

void build_twolayer_linear(Builder& B, const AlgoSpec& s) {
  const int P = s.P, n = s.n, G = P / n;
  for (int R = 0; R < P; R++) {
    const int gid = R / n, q = R % n;
    switch (s.algo) {
      case ALG_TWOLAYER_LINEAR:  // src/twolayer_communicator_linear.cpp:13-87
        for (int i = 0; i < n; i++) B.direct(1, 0, (uint32_t)i, R, gid * n + mod(q - i, n));
        for (int i = 1; i < G; i++)
          for (int j = 0; j < n; j++) B.direct(2, 0, (uint32_t)(i * n + j), R, mod(gid + i, G) * n + j);
        break;
      case ALG_TWOLAYER_LINEAR_S2:  // :91-192
      case ALG_TWOLAYER_LINEAR_S4:  // declared only in the reference; same schedule as _s2 here
        for (int i = 0; i < n; i++) B.direct(1, i / s.b, (uint32_t)i, R, gid * n + mod(q - i, n));
        for (int f = 1; f < P; f++) {
          int gi = f / n, gr = f % n, nd = mod(gid + gi, G);
          if (nd == gid) continue;
          B.direct(2, (f - 1) / s.b2, (uint32_t)f, R, nd * n + gr);
        }
        break;
      case ALG_TWOLAYER_LINEAR_S3:  // :196-317 (the self block, which the reference forgets, is copied)
        B.self_copy(R);
        for (int i = 1; i < n; i++) B.direct(1, (i - 1) / s.b, (uint32_t)i, R, gid * n + mod(q - i, n));
        for (int i = 1; i < G; i++)
          for (int j = 0; j < n; j++)
            B.direct(2, 0, (uint32_t)(i * n + j), R, mod(gid + i, G) * n + mod(j - q, n));
        break;
      default: break;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Leader-routed exchanges (reference: benchmarks/merge_benchmark.cpp:155-332 and
// benchmarks/simple_merge_benchmark.cpp:138-210).  The ranks of a group hand their blocks to one
// leader, the leaders exchange them, and each leader hands the blocks to their destinations:
//   S -> leader(group of S) -> leader(group of D) -> D,
// where a hop is dropped when both ends are the same rank.  In the "merge" scheme local rank 0 of
// every group is the rank with the large messages: it neither gathers nor is gathered (it talks to
// the other groups' rank 0 and leaders directly) and local rank 1 is the leader of the small-message
// ranks.  The reference stops before the hand-out to the destinations (its scatter is commented out);
// here it is done.  In the "simple merge" scheme local rank 0 is the leader of everybody.
// Keys: phase 1 gather, phase 2 exchange between holders (spread-out order over the holder index),
// phase 3 hand-out, so the three stages can be timed separately, like the reference's
// gather_time / ata_time / scatter_time.
// ---------------------------------------------------------------------------------------------
void build_leader_routed(Builder& B, int n, int leader_lr, int exempt_lr) {
  const int P = B.P, G = P / n;
  auto holder = [&](int R) { return (R % n == exempt_lr) ? R : (R / n) * n + leader_lr; };
  // index of a holder among the ranks that take part in the exchange stage (for the spread-out order)
  auto hidx = [&](int H) { return (H / n) * 2 + ((H % n == leader_lr) ? 1 : 0); };
  for (int R = 0; R < P; R++) B.self_copy(R);
  for (int S = 0; S < P; S++)
    for (int D = 0; D < P; D++) {
      if (S == D) continue;
      const int h1 = holder(S), h2 = holder(D);
      int cur = S, cell = -1;
      if (h1 != cur) {                                  // gather
        const int dc = (h1 == D) ? -1 : B.cell(3, 1, S % n, D);
        B.emit(1, 0, (uint32_t)(S % n) * P + D, cur, h1, S, D, cell, dc);
        cur = h1; cell = dc;
      }
      if (cur != D && h2 != cur) {                      // exchange between holders
        const int dc = (h2 == D) ? -1 : B.cell(3, 2, S, D % n);
        const int dist = mod(hidx(cur) - hidx(h2), 2 * G);
        B.emit(2, 0, (uint32_t)dist * P * P + (uint32_t)S * P + D, cur, h2, S, D, cell, dc);
        cur = h2; cell = dc;
      }
      if (cur != D) B.emit(3, 0, (uint32_t)(D % n) * P + S, cur, D, S, D, cell, -1);   // hand-out
    }
}

// Spread-out exchange in which the block from rank 0 to rank P - 1 (the one huge block of the reference's
// benchmark) travels as `parts` separate messages, all posted together with the other blocks
// (benchmarks/split_benchmark.cpp:147-205; the reference drops count % P elements, here the last part
// takes them).
void build_split(Builder& B, int parts) {
  const int P = B.P;
  for (int R = 0; R < P; R++)
    for (int i = 0; i < P; i++) {
      const int T = mod(R - i, P);
      if (R == 0 && T == P - 1 && P > 1 && parts > 1) {
        for (int p = 0; p < parts; p++) {
          B.emit(1, 0, (uint32_t)i * 256 + p, R, T, R, T, -1, -1, ((uint32_t)p << 2) | ((uint32_t)parts << 9));
        }
      } else {
        B.direct(1, 0, (uint32_t)i * 256, R, T);
      }
    }
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

Plan build_plan(const AlgoSpec& in) {
  Plan pl;
  pl.spec = in;
  AlgoSpec& s = pl.spec;
  auto fail = [&](int code, const char* msg) { pl.err = code; pl.errmsg = msg; return pl; };
  if (s.P < 1 || s.P > 65535) return fail(-1, "rank count out of range");
  if (s.algo < 0 || s.algo >= ALG_COUNT) return fail(-1, "unknown algorithm");
  const int P = s.P;
  pl.uniform = (s.algo == ALG_UNIFORM_SPREADOUT_TWOLAYER || s.algo == ALG_UNIFORM_ISPLIT_RBRUCK);
  pl.inplace_ok = (s.algo == ALG_TTPL_BT_S2);
  Builder B(pl);

  const bool hier = (s.algo >= ALG_TTPL && s.algo <= ALG_UNIFORM_ISPLIT_RBRUCK);
  const bool tl_linear = (s.algo >= ALG_TWOLAYER_LINEAR && s.algo <= ALG_TWOLAYER_LINEAR_S4);
  const bool leader = (s.algo == ALG_MERGE || s.algo == ALG_SIMPLE_MERGE);

  // Argument rules of the reference (return codes and clamps), evaluated before the P == 1 shortcut
  // so that an invalid radix is reported for every P.
  switch (s.algo) {
    case ALG_RBRUCK: case ALG_RBRUCK_OM:
      if (s.r < 2) return fail(-1, "radix must be >= 2");       // src/twophase_tunable_rbruckv.cpp:16
      if (s.r > P) s.r = std::max(2, P);                         // :22
      break;
    case ALG_TUNA: case ALG_TUNA2:
      if (s.r < 2) s.r = 2;                                      // src/tuna.cpp:13
      if (s.r > P - 1) s.r = std::max(2, P - 1);                 // :20 (P <= 2 would give r = 1 and hang there)
      if (s.b <= 0 || s.b > P) s.b = P;                          // :21
      break;
    case ALG_SCATTERED:
      if (s.b <= 0 || s.b > P) s.b = P;                          // src/MPICH_scattered.cpp:32
      break;
    case ALG_XOR:
      if (!is_pow2(P)) return fail(-1, "XOR exchange needs a power-of-two rank count");  // src/exclusive_or_alltoallv.cpp:31
      break;
    case ALG_SPLIT:
      if (s.b <= 0 || s.b > kMaxOpParts) s.b = std::min(P, kMaxOpParts);   // one message per rank, as the reference
      break;
    default: break;
  }
  if (leader) {
    if (s.n < 1) return fail(-1, "group size must be >= 1");
    if (s.n > P) s.n = P;
    if (P % s.n != 0) return fail(-1, "group size must divide the rank count");
  }
  if (hier || tl_linear) {
    if (hier && s.algo != ALG_UNIFORM_ISPLIT_RBRUCK && s.r < 2) return fail(-1, "radix must be >= 2");
    if (P > 1) {
      if (s.n < 1) return fail(-1, "group size must be >= 1");
      // The uniform and the linear two-layer variants abort when n >= P
      // (src/twolayer_rbruck.cpp:18-22, src/twolayer_communicator_linear.cpp:23-27).
      const bool aborts = tl_linear || pl.uniform;
      if (aborts && s.n >= P) return fail(-2, "the process count should be divided by the process count of a group");
      if (s.n > P) s.n = P;
      if (P % s.n != 0) return fail(-1, "group size must divide the rank count");
    } else {
      s.n = 1;
    }
    if (hier) {
      if (s.r < 2) s.r = 2;
      if (s.r > s.n) s.r = std::max(2, s.n);                     // src/twophase_twolayer_rbruck.cpp:248
      const int G = P / s.n;
      if (s.algo == ALG_UNIFORM_ISPLIT_RBRUCK) {
        // The reference overwrites r2 with the group count (src/twolayer_rbruck.cpp:158); a valid
        // r2 is honoured here, anything else falls back to that behaviour.
        if (s.r2 < 2 || s.r2 > G) s.r2 = std::max(2, G);
      }
    } else {
      if (s.b <= 0 || s.b > s.n) s.b = s.n;                      // bblock1
      if (s.b2 <= 0 || s.b2 > P) s.b2 = P;                       // bblock2
    }
  }

  if (P == 1) {
    B.self_copy(0);
    B.finish();
    return pl;
  }

  switch (s.algo) {
    case ALG_RBRUCK:    build_flat_bruck(B, s.r, true, 0, false); break;
    case ALG_RBRUCK_OM: build_flat_bruck(B, s.r, false, 0, false); break;
    case ALG_TUNA:      build_flat_bruck(B, s.r, false, s.b, false); break;
    case ALG_TUNA2:     build_flat_bruck(B, s.r, false, s.b, true); break;
    case ALG_MERGE:        build_leader_routed(B, s.n, s.n >= 2 ? 1 : 0, s.n >= 2 ? 0 : -1); break;
    case ALG_SIMPLE_MERGE: build_leader_routed(B, s.n, 0, -1); break;
    case ALG_SPLIT:        build_split(B, s.b); break;
    default:
      if (hier) build_hier(B, s);
      else if (tl_linear) build_twolayer_linear(B, s);
      else build_direct(B, s);
  }
  B.finish();
  return pl;
}

std::vector<Op> ops_for_ranks(const Plan& plan, const std::vector<int>& ranks) {
  std::vector<char> mine(plan.spec.P, 0);
  for (int r : ranks) if (r >= 0 && r < plan.spec.P) mine[r] = 1;
  std::vector<Op> out;
  for (const Op& o : plan.ops) if (mine[o.src]) out.push_back(o);
  return out;
}

int host_execute(const Plan& plan, int ts, const char* const* sendbufs, char* const* recvbufs,
                 const int* sendcounts, const long long* sdispls, const long long* rdispls) {
  const int P = plan.spec.P;
  long long M = 0;
  for (long long i = 0; i < (long long)P * P; i++) M = std::max<long long>(M, sendcounts[i]);
  const size_t stride = (size_t)M * ts;
  std::vector<std::vector<char>> stage(P);
  std::vector<std::vector<char>> state(P);
  for (int p = 0; p < P; p++) {
    stage[p].resize(stride * plan.ncells + 1);
    state[p].assign(plan.ncells + 1, 0);
  }
  for (const Op& o : plan.ops) {
    if (o.src >= P || o.dst >= P || o.origin >= P || o.dest >= P) return -12;
    long long first = 0, cnt = 0;
    op_slice(o, sendcounts[(size_t)o.origin * P + o.dest], &first, &cnt);
    if (op_nparts(o) && (o.src_cell >= 0 || o.dst_cell >= 0)) return -12;   // slices travel in one hop only
    const size_t bytes = (size_t)cnt * ts;
    const char* src;
    if (o.src_cell < 0) {
      if (o.src != o.origin) return -12;
      src = sendbufs[o.src] + (sdispls[(size_t)o.src * P + o.dest] + first) * ts;
    } else {
      if (o.src_cell >= plan.ncells) return -12;
      if (state[o.src][o.src_cell] != 1) return -10;
      state[o.src][o.src_cell] = 2;
      src = stage[o.src].data() + stride * o.src_cell;
    }
    char* dst;
    if (o.dst_cell < 0) {
      if (o.dst != o.dest) return -12;
      dst = recvbufs[o.dst] + (rdispls[(size_t)o.dst * P + o.origin] + first) * ts;
    } else {
      if (o.dst_cell >= plan.ncells) return -12;
      if (state[o.dst][o.dst_cell] != 0) return -11;
      state[o.dst][o.dst_cell] = 1;
      dst = stage[o.dst].data() + stride * o.dst_cell;
    }
    if (bytes) std::memmove(dst, src, bytes);
  }
  return 0;
}

}  // namespace rbv
