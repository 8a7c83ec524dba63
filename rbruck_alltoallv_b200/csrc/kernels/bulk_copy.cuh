// Bulk-copy engine for large, 16-byte aligned chunks: the copy engine of the SM (the untiled form of TMA)
// moves the data, one thread drives it.
//
//   global (this GPU: send buffer or staging cell)  --cp.async.bulk-->  shared-memory tile
//   shared-memory tile                              --cp.async.bulk-->  global (this GPU or a peer over NVLink)
//
// Each warp owns a ring of S (2 or 3) tiles of kBulkTile bytes and one mbarrier per tile.  The loads of tiles
// i + 1 .. i + S - 1 are in flight while tile i is stored, so a warp keeps loads and a store outstanding with
// one issuing thread and no registers spent on payload.  No load uses cluster multicast, and loads only ever read this
// GPU's memory; the stores are what crosses NVLink.  The wait on a tile's mbarrier is bounded like every
// other wait of the library.  Stands where `memcpy` stands in the reference's pack / unpack / forward steps
// (e.g. src/tuna2.cpp:134-150).
#pragma once
#include <cstdint>

#include "kernels/primitives.cuh"

namespace rbv {
namespace dev {

constexpr int kBulkTile = 4096;
constexpr int kBulkMaxStages = 3;        // tiles per warp: stages - 1 loads run ahead of the store
constexpr size_t kBulkMinBytes = 1024;   // shorter chunks go through the vector path

// Per-warp state; `it` counts tiles over the whole kernel so that mbarrier phases carry over between chunks.
struct BulkPipe {
  uint32_t tiles;    // shared-memory address of the warp's first tile
  uint32_t bars;     // shared-memory address of the warp's first mbarrier
  unsigned it;
  unsigned stages;
};

__host__ __device__ constexpr size_t bulk_smem_bytes(int warps, int stages) {
  return (size_t)warps * stages * (kBulkTile + 8);
}

__device__ __forceinline__ void bulk_pipe_init(BulkPipe& bp, unsigned char* region, int warp, int warps, int lane,
                                               int stages) {
  unsigned char* tiles = region + (size_t)warp * stages * kBulkTile;
  unsigned char* bars = region + (size_t)warps * stages * kBulkTile + (size_t)warp * stages * 8;
  bp.tiles = static_cast<uint32_t>(__cvta_generic_to_shared(tiles));
  bp.bars = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
  bp.it = 0;
  bp.stages = (unsigned)stages;
  if (lane == 0) {
    for (int s = 0; s < stages; s++)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bp.bars + 8u * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ bool bulk_bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

__device__ __forceinline__ WaitResult bulk_bar_wait(uint32_t bar, uint32_t parity, const WaitCfg& cfg) {
  if (bulk_bar_try(bar, parity)) return WAIT_OK;
  const unsigned long long t0 = globaltimer();
  unsigned n = 0;
  for (;;) {
    if (bulk_bar_try(bar, parity)) return WAIT_OK;
    if ((++n & 63u) == 0) {
      if (ld_relaxed_sys(cfg.abort_flag)) return WAIT_ABORTED;
      if (globaltimer() - t0 > cfg.timeout_ns) return WAIT_TIMEOUT;
    }
  }
}

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const char* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store(char* dst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_src), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// All but the newest `N` store groups of this thread have finished READING shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// All store groups of this thread are complete: their writes are performed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Copies n bytes (a multiple of 16; dst and src 16-byte aligned; src in this GPU's memory).  ONE thread calls
// it.  On return with WAIT_OK every byte has been written at the destination and a release by the same thread
// publishes it.  On a time-out the stores already issued are drained before returning.
//
// Tile g (counted over the whole kernel) lives in stage g mod S.  Loads run S - 1 tiles ahead: after tile i has
// been handed to the store, tile i + S - 1 is loaded into the stage that tile i - 1 used, so only the store
// before the newest one must have left shared memory.
__device__ __forceinline__ WaitResult bulk_copy(char* dst, const char* src, size_t n, BulkPipe& bp, const WaitCfg& cfg) {
  const unsigned ntiles = (unsigned)((n + kBulkTile - 1) / kBulkTile);
  const unsigned S = bp.stages, first = bp.it;
  // Data that other threads (or peers) wrote with ordinary stores is about to be read by the copy engine.
  fence_proxy_async();
  auto tile_len = [&](unsigned t) -> uint32_t {
    const size_t o = (size_t)t * kBulkTile;
    return (uint32_t)((n - o < (size_t)kBulkTile) ? (n - o) : (size_t)kBulkTile);
  };
  auto load = [&](unsigned t) {
    const unsigned st = (first + t) % S;
    bulk_load(bp.tiles + st * kBulkTile, src + (size_t)t * kBulkTile, tile_len(t), bp.bars + 8u * st);
  };
  // every store of earlier chunks is complete (each copy ends with a full wait), so all stages are free
  unsigned loaded = 0;
  for (; loaded < ntiles && loaded + 1 < S; loaded++) load(loaded);
  WaitResult res = WAIT_OK;
  for (unsigned i = 0; i < ntiles; i++) {
    const unsigned g = first + i, st = g % S;
    res = bulk_bar_wait(bp.bars + 8u * st, (g / S) & 1u, cfg);
    if (res != WAIT_OK) break;
    bulk_store(dst + (size_t)i * kBulkTile, bp.tiles + st * kBulkTile, tile_len(i));
    if (loaded < ntiles) {
      if (i > 0) bulk_wait_read<1>();   // the store of tile i - 1 has left its stage; tile i's may still be reading
      load(loaded++);
    }
  }
  bp.it = first + loaded;
  if (res != WAIT_OK) {
    // Loads still in flight complete their barrier phases; give each one more bounded wait so that shared
    // memory is quiet when the kernel leaves (a completed phase answers at once).
    for (unsigned j = (loaded > S ? loaded - S : 0); j < loaded; j++) {
      const unsigned g = first + j;
      (void)bulk_bar_wait(bp.bars + 8u * (g % S), (g / S) & 1u, cfg);
    }
  }
  bulk_wait_all();
  fence_proxy_async();
  return res;
}

}  // namespace dev
}  // namespace rbv
