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

