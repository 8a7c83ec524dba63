// Definitions behind the opaque handles of the C API, shared by the translation units that implement it.
#pragma once
#include <memory>
#include <vector>

#include "rbv/context.h"
#include "rbv/rbruckv.h"

using rbv::AlgoSpec;
using rbv::Context;

struct rbv_comm_s {
  rbv_ctx_s* ctx;
  int local;
};

struct rbv_ctx_s {
  std::unique_ptr<Context> c;
  cudaStream_t stream = nullptr;
  int grid = 0;
  size_t chunk = 0;
  unsigned long long eager = 0;   // cell payload bytes of the eager protocol for the following calls (0: off)
  bool allow_static = true;       // persistent calls with host-side counts may run the static kernel
  std::vector<void*> recv_mirror; // for the next rbv_prepare*: where the received blocks are wanted in the end
  double plan_build_s = 0;        // host time spent compiling the schedule of the latest call (0: it was cached)
  // per-rank entry points: the resolved call of the previous collective, reused when the next one has the same
  // arguments (a loop over one collective then costs one kernel launch per iteration)
  void* cached = nullptr;
  int last_rc = 0;                // return code of the latest rbv_prepare*
  bool automatic = false;         // the collective being collected asked for the automatic choice
  rbv_choice last_choice{};       // what the latest automatic call resolved to
  double hint_mean = -1, hint_cv = 0;   // what the caller said about the whole exchange (automatic entry points)
  std::vector<char> cached_key;
  std::vector<rbv_comm_s> comms;
  // calls of the local ranks collected until all L have arrived
  int pend = 0;
  AlgoSpec spec;
  int ts = 0;
  unsigned flags = 0;
  std::vector<char> seen;
  std::vector<const void*> sendbufs;
  std::vector<void*> recvbufs;
  std::vector<int> sc, rc;
  std::vector<long long> sd, rd;
};

