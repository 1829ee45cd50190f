// Native rank launcher for the stand-alone C++ programs: one forked process per rank, an anonymous
// shared mapping for rendezvous, a host barrier that gives up when a peer has failed or is late, a
// handle exchange table (for cudaIpc handles or any small blob), a results table and heartbeats.
//
// CUDA must not be initialised before fork(): the device count is probed in a throw-away child.
// Failure model (host side only): a rank that calls fail(), exits, or never arrives makes every
// barrier() on the other ranks return false within the time-out, instead of hanging them.
//
// Reference parity: comm_comp/ipc_multiproc.cuh:43-171 (probe_device_count, ShmBarrier, Shm,
// MultiProc::init / barrier / fail / wait_children / exchange).  The Python layer uses torchrun
// and the torch.distributed store instead; this is the zero-dependency path.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>

namespace tcl {
namespace rt {

constexpr int kMaxWorld = 8;
constexpr int kMaxSlots = 8;
constexpr int kSlotBytes = 128;
constexpr int kResultsPerRank = 16;

struct SharedBlob {
  std::atomic<int> arrived;
  std::atomic<int> generation;
  std::atomic<int> failed;        // 0 = healthy, else 1 + rank that raised it
  char failed_why[120];
  unsigned char slots[kMaxSlots][kMaxWorld][kSlotBytes];
  double results[kMaxWorld][kResultsPerRank];
  std::atomic<long long> heartbeat_ms[kMaxWorld];
};

class Launcher {
 public:
  // Forks world - 1 children; the caller becomes rank 0.  Returns this process's rank, or -1.
  int init(int world);
  int rank() const { return rank_; }
  int world() const { return world_; }
  SharedBlob* shm() { return blob_; }

  // Sense-reversing barrier over the shared blob.  false: a peer failed or the wait ran out
  // (then this rank marks the job failed too, so that nobody else keeps waiting).
  bool barrier(double timeout_s = 30.0);
  // Marks the job failed; every barrier() in flight or later returns false.
  void fail(const char* why);
  bool failed() const;
  // All ranks deposit `bytes` (<= kSlotBytes) in `slot`; `all` receives world * bytes.
  bool exchange(int slot, const void* mine, size_t bytes, void* all, double timeout_s = 30.0);
  void beat();                                   // heartbeat of this rank
  long long ms_since_beat(int rank) const;       // age of a peer's heartbeat
  // Rank 0 only: waits for the children, returns the worst exit status (signals count as 128+n).
  int wait_children(double timeout_s = 60.0);

  // Device count as seen by a throw-away child process (keeps this process CUDA-free before fork).
  static int probe_device_count();

 private:
  SharedBlob* blob_ = nullptr;
  int rank_ = 0, world_ = 1;
  int local_gen_ = 0;
  int children_[kMaxWorld] = {0};
};

}  // namespace rt
}  // namespace tcl
