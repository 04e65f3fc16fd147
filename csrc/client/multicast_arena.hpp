// Symmetric device arena with an NVSwitch multicast (NVLS) view.
//
// Every rank allocates the same number of bytes through the CUDA virtual-memory API (cuMemCreate), maps the other
// ranks' allocations into its address space (handles travel as file descriptors over Unix-domain sockets), and all
// ranks bind their allocation at offset 0 of one multicast object.  Through the multicast mapping `mc_base + off`
// a single `multimem.ld_reduce` instruction returns the sum of the word at `off` in every rank's arena, reduced
// inside the switch, and a single `multimem.st` writes that word on every rank - the NVSwitch form of the
// reduce-scatter and broadcast that the push kernel otherwise does with one load / store per peer.
//
// Used by the NVLINK transport when GeePsConfig::use_multicast is set and every device reports multicast support;
// any failure before the first bind makes all ranks fall back to the cudaMalloc + CUDA IPC arena together.
//
// No counterpart in the reference (its transport is ZeroMQ over TCP).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace geeps_b200 {

class MulticastArena {
 public:
  ~MulticastArena();
  // Does this device support multicast objects at all (CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED)?
  static bool device_supported(int device);
  // Step 1 (local): allocate `bytes` (rounded up to the multicast granularity) on `device` and map it.
  bool allocate(size_t bytes, int device, std::string* err);
  // Step 2 (collective; the caller brackets it with its own host barriers where the comments say so):
  //   open a Unix-domain listener named after (tag, rank);
  bool listen(const std::string& tag, int rank, std::string* err);
  //   after a barrier: send this rank's allocation to every peer (rank 0 also creates and sends the multicast object);
  bool send_handles(const std::string& tag, int rank, int world, std::string* err);
  //   receive the peers' allocations (and the multicast object), map the peers, add this device to the team;
  bool receive_and_map(int rank, int world, std::string* err);
  //   after a barrier (every device added): bind this rank's memory and map the multicast view.
  bool bind_and_map(std::string* err);
  // Unbind / unmap / release everything (idempotent).  Call only after the ranks agreed that no kernel uses the
  // multicast view any more.
  void release();

  char* base() const { return reinterpret_cast<char*>(local_va_); }
  char* peer(int r) const { return reinterpret_cast<char*>(peer_va_[r]); }
  char* multicast_base() const { return reinterpret_cast<char*>(mc_va_); }
  size_t bytes() const { return bytes_; }
  bool bound() const { return bound_; }

 private:
  int device_ = 0, listen_fd_ = -1;
  size_t bytes_ = 0;
  unsigned long long mem_ = 0, mc_ = 0;          // CUmemGenericAllocationHandle
  unsigned long long local_va_ = 0, mc_va_ = 0;  // CUdeviceptr
  std::vector<unsigned long long> peer_mem_, peer_va_;
  bool bound_ = false, mc_added_ = false;
};

}  // namespace geeps_b200
