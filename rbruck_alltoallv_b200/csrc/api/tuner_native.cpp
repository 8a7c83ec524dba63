// Algorithm selection for the C API: reads the table of measured winners that the sweep writes
// (parallel/tuner.py keeps the file; the format is a JSON object of
//   "P<ranks>-G<processes>-c<size class>[-s<skew class>]": {"choice": {"algo": "...", "n": .., "r": .., "b": ..,
//   "protocol": "eager" | "rendezvous"}, "us": <microseconds>})
// and answers with the same rules as the Python side: size class = floor(log2(mean block bytes)), skew class 1
// when the coefficient of variation of the block sizes is 0.5 or more, neighbouring classes stand in for classes
// that were not measured, and the built-in rule (spread-out; eager up to 64 KB blocks) when the table has nothing.
// The reference has no selection logic beyond the hard-coded batch limits of its driver
// (examples/twophaseLayer_example2.cpp:136-152); its ML_benchmark entry point is declared and never defined.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "rbv/plan.h"
#include "rbv/rbruckv.h"

namespace {

struct Entry { rbv_choice c; double us; };
std::map<std::string, Entry> g_table;
std::string g_path, g_loaded_from;
std::mutex g_mutex;
bool g_loaded = false;

// ---- a reader for exactly the shape above (objects, strings, numbers) ----
struct Reader {
  const char* p;
  const char* e;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r' || *p == ',' || *p == ':')) p++; }
  bool str(std::string* out) {
    ws();
    if (p >= e || *p != '"') return false;
    const char* q = ++p;
    while (p < e && *p != '"') p++;
    if (p >= e) return false;
    out->assign(q, p);
    p++;
    return true;
  }
  bool num(double* out) {
    ws();
    char* end = nullptr;
    *out = std::strtod(p, &end);
    if (end == p) return false;
    p = end;
    return true;
  }
  bool open() { ws(); if (p < e && *p == '{') { p++; return true; } return false; }
  bool close() { ws(); if (p < e && *p == '}') { p++; return true; } return false; }
  // skips one value of any kind
  void skip() {
    ws();
    if (p >= e) return;
    if (*p == '"') { std::string s; str(&s); return; }
    if (*p == '{' || *p == '[') {
      int depth = 0;
      do { if (*p == '{' || *p == '[') depth++; else if (*p == '}' || *p == ']') depth--; p++; } while (p < e && depth > 0);
      return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') p++;
  }
};

void parse_choice(Reader& r, rbv_choice* c) {
  std::memset(c, 0, sizeof *c);
  c->algo = rbv::ALG_SPREADOUT;
  c->r = 2;
  if (!r.open()) return;
  std::string k, v;
  double d;
  while (!r.close() && r.p < r.e) {
    if (!r.str(&k)) { r.p = r.e; return; }
    if (k == "algo") { r.str(&v); int a = rbv::algo_from_name(v.c_str()); if (a >= 0) c->algo = a; }
    else if (k == "protocol") { r.str(&v); c->eager = (v == "eager"); }
    else if (r.num(&d)) {
      if (k == "n") c->n = (int)d; else if (k == "r") c->r = (int)d; else if (k == "r2") c->r2 = (int)d;
      else if (k == "b") c->b = (int)d; else if (k == "b2") c->b2 = (int)d;
    } else r.skip();
  }
}

void load_locked() {
  std::string path = g_path;
  if (path.empty()) if (const char* e = std::getenv("RBV_TUNER_CACHE")) path = e;
  if (g_loaded && path == g_loaded_from) return;
  g_table.clear();
  g_loaded = true;
  g_loaded_from = path;
  if (path.empty()) return;
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) return;
  std::string text;
  char buf[4096];
  size_t n;
  while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
  std::fclose(f);
  Reader r{text.data(), text.data() + text.size()};
  if (!r.open()) return;
  std::string key, k;
  while (!r.close() && r.p < r.e) {
    if (!r.str(&key) || !r.open()) return;
    Entry en{};
    en.c.algo = rbv::ALG_SPREADOUT;
    while (!r.close() && r.p < r.e) {
      if (!r.str(&k)) return;
      if (k == "choice") parse_choice(r, &en.c);
      else if (k == "us") r.num(&en.us);
      else r.skip();
    }
    g_table[key] = en;
  }
}

int size_class(double mean) { return mean <= 1.0 ? 0 : (int)std::floor(std::log2(mean)); }

}  // namespace

extern "C" {

void rbv_tuner_set_table(const char* path) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_path = path ? path : "";
  g_loaded = false;
}

int rbv_tuner_entries(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  load_locked();
  return (int)g_table.size();
}

// Returns 1 when the answer comes from the table, 0 when it is the built-in rule.
int rbv_tuner_choose(int P, int nproc, double mean_block_bytes, double cv, rbv_choice* out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  load_locked();
  const int cls = size_class(mean_block_bytes), sk = cv >= 0.5 ? 1 : 0;
  const int classes[3] = {cls, cls - 1, cls + 1};
  for (int c : classes)
    for (int s : {sk, 1 - sk}) {
      char key[64];
      if (s) std::snprintf(key, sizeof key, "P%d-G%d-c%d-s%d", P, nproc, c, s);
      else std::snprintf(key, sizeof key, "P%d-G%d-c%d", P, nproc, c);
      auto it = g_table.find(key);
      if (it != g_table.end()) { *out = it->second.c; return 1; }
    }
  std::memset(out, 0, sizeof *out);
  out->algo = rbv::ALG_SPREADOUT;
  out->r = 2;
  out->eager = mean_block_bytes <= 64.0 * 1024;
  return 0;
}

}  // extern "C"
