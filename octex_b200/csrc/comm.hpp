// NCCL communicator of a sharded or replicated index, one process per GPU.
//
// The reference drives all GPUs from one process and lets kernels read the other GPUs' memory
// through peer pointers (hpdic/octex, cpp/src/neighbors/octex/load.cu:187-202,
// search.cu:738-753,909-919). Here every GPU has its own process; the two places where data of
// one GPU is needed on another — the kept lists after the first round of a sharded index, and the
// gathering of the per-rank results — go through NCCL send / receive and all-gather on the
// library's own stream. NCCL is loaded at run time (libnccl.so.2), so a single-GPU process needs
// no NCCL at all.
#pragma once

#include "common.hpp"

#include <cstddef>
#include <cstdint>

namespace octex_b200::detail {

constexpr size_t kUniqueIdBytes = 128;  // sizeof(ncclUniqueId)

class communicator {
 public:
  /// Every rank calls this with the same id (made by unique_id() on one of them).
  communicator(const void* unique_id, int rank, int world, int device);
  communicator(communicator const&) = delete;
  ~communicator();
  static void unique_id(void* out128);

  [[nodiscard]] auto rank() const -> int { return rank_; }
  [[nodiscard]] auto world() const -> int { return world_; }

  void group_start();
  void group_end();
  void send(const void* buf, size_t bytes, int peer, cudaStream_t s);
  void recv(void* buf, size_t bytes, int peer, cudaStream_t s);
  /// recv [world, bytes_per_rank] <- send [bytes_per_rank] of every rank.
  void all_gather(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t s);

 private:
  void* comm_ = nullptr;
  int rank_ = 0, world_ = 1, device_ = 0;
};

}  // namespace octex_b200::detail
