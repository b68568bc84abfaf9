// Symmetric heap on CUDA virtual-memory management: one physical allocation per rank, exported as a POSIX file
// descriptor, imported and mapped by every peer, plus (where the fabric has NVLS) one multicast object bound to all
// ranks' allocations and mapped once more. This is the allocation layer under the fused tensor-parallel, collective
// and expert-parallel kernels; everything that happens in the memory afterwards is this library's kernels.
// The file descriptors travel between the rank processes over a side channel the caller owns (the Python layer sends
// them through AF_UNIX sockets with SCM_RIGHTS); this class only turns descriptors into mappings.
// No counterpart in the reference, which has no multi-device memory at all.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace b2 {
namespace symm {

constexpr int kMaxRanks = 8;

class HeapSegment {
 public:
  HeapSegment() = default;
  ~HeapSegment();
  HeapSegment(const HeapSegment&) = delete;
  HeapSegment& operator=(const HeapSegment&) = delete;

  // Allocate `bytes` (rounded up to the allocation and, with `multicast`, the multicast granularity) on `device` for a
  // group of `world` ranks of which this is `rank`, and map it at this rank's slot. Returns an empty string or an error.
  std::string create(int device, int rank, int world, size_t bytes, bool multicast);
  // A new descriptor for this rank's allocation (the caller sends it to the peers and closes its copy).
  int export_fd(std::string* err);
  // Map the allocation behind a descriptor received from rank `peer` (the descriptor is closed here).
  std::string map_peer(int peer, int fd);
  // Multicast object: rank 0 creates it and exports a descriptor; the others import it; every rank adds its device;
  // after ALL ranks have added theirs, every rank binds its allocation and maps the object.
  bool multicast_supported() const { return mc_supported_; }
  int mc_create(std::string* err);
  std::string mc_import(int fd);
  std::string mc_add_device();
  std::string mc_bind_and_map();

  size_t bytes() const { return bytes_; }
  uint64_t ptr(int rank) const { return rank >= 0 && rank < kMaxRanks ? va_[rank] : 0; }
  uint64_t mc_ptr() const { return mc_va_; }
  void close();

 private:
  int device_ = -1, rank_ = 0, world_ = 1;
  size_t bytes_ = 0, gran_ = 0;
  bool mc_supported_ = false, mc_bound_ = false, have_local_ = false, have_mc_ = false;
  uint64_t local_handle_ = 0, mc_handle_ = 0;
  uint64_t peer_handle_[kMaxRanks] = {};
  bool peer_mapped_[kMaxRanks] = {};
  uint64_t va_[kMaxRanks] = {};
  uint64_t mc_va_ = 0;
};

}  // namespace symm
}  // namespace b2
