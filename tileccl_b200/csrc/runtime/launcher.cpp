#include "launcher.hpp"

#include <cuda_runtime.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>

namespace tcl {
namespace rt {

static long long now_ms() {
  using namespace std::chrono;
  return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

int Launcher::probe_device_count() {
  int fds[2];
  if (pipe(fds) != 0) return 0;
  pid_t pid = fork();
  if (pid < 0) return 0;
  if (pid == 0) {
    close(fds[0]);
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) n = 0;
    ssize_t w = write(fds[1], &n, sizeof(n));
    (void)w;
    _exit(0);
  }
  close(fds[1]);
  int n = 0;
  if (read(fds[0], &n, sizeof(n)) != static_cast<ssize_t>(sizeof(n))) n = 0;
  close(fds[0]);
  int st;
  waitpid(pid, &st, 0);
  return n;
}

int Launcher::init(int world) {
  if (world < 1 || world > kMaxWorld) return -1;
  void* p = mmap(nullptr, sizeof(SharedBlob), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) return -1;
  blob_ = new (p) SharedBlob();
  std::memset(static_cast<void*>(blob_), 0, sizeof(SharedBlob));
  world_ = world;
  rank_ = 0;
  for (int r = 1; r < world; ++r) {
    pid_t pid = fork();
    if (pid < 0) { fail("fork failed"); return -1; }
    if (pid == 0) { rank_ = r; break; }
    children_[r] = pid;
  }
  beat();
  return rank_;
}

bool Launcher::failed() const { return blob_->failed.load(std::memory_order_acquire) != 0; }

void Launcher::fail(const char* why) {
  int expected = 0;
  if (blob_->failed.compare_exchange_strong(expected, 1 + rank_, std::memory_order_acq_rel)) {
    std::snprintf(blob_->failed_why, sizeof(blob_->failed_why), "%s", why ? why : "");
  }
}

bool Launcher::barrier(double timeout_s) {
  if (failed()) return false;
  const int gen = local_gen_;
  const long long deadline = now_ms() + static_cast<long long>(timeout_s * 1000);
  if (blob_->arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == world_) {
    blob_->arrived.store(0, std::memory_order_relaxed);
    blob_->generation.store(gen + 1, std::memory_order_release);
  } else {
    unsigned spins = 0;
    while (blob_->generation.load(std::memory_order_acquire) == gen) {
      if (failed()) return false;
      if (now_ms() > deadline) { fail("barrier timed out: a rank never arrived"); return false; }
      if (++spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  local_gen_ = gen + 1;
  beat();
  return !failed();
}

bool Launcher::exchange(int slot, const void* mine, size_t bytes, void* all, double timeout_s) {
  if (slot < 0 || slot >= kMaxSlots || bytes > static_cast<size_t>(kSlotBytes)) { fail("bad exchange slot or size"); return false; }
  std::memcpy(blob_->slots[slot][rank_], mine, bytes);
  if (!barrier(timeout_s)) return false;
  for (int r = 0; r < world_; ++r) std::memcpy(static_cast<unsigned char*>(all) + r * bytes, blob_->slots[slot][r], bytes);
  return barrier(timeout_s);   // nobody overwrites the slot before everyone has read it
}

void Launcher::beat() { blob_->heartbeat_ms[rank_].store(now_ms(), std::memory_order_release); }
long long Launcher::ms_since_beat(int rank) const { return now_ms() - blob_->heartbeat_ms[rank].load(std::memory_order_acquire); }

int Launcher::wait_children(double timeout_s) {
  if (rank_ != 0) return 0;
  int worst = 0;
  const long long deadline = now_ms() + static_cast<long long>(timeout_s * 1000);
  for (int r = 1; r < world_; ++r) {
    if (children_[r] <= 0) continue;
    int st = 0;
    for (;;) {
      pid_t w = waitpid(children_[r], &st, WNOHANG);
      if (w == children_[r]) break;
      if (w < 0) { st = 0x7f00; break; }
      if (now_ms() > deadline) {
        // A child that does not leave on its own is ended by its exact pid.
        kill(children_[r], SIGKILL);
        waitpid(children_[r], &st, 0);
        break;
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    int code = WIFEXITED(st) ? WEXITSTATUS(st) : WIFSIGNALED(st) ? 128 + WTERMSIG(st) : 1;
    if (code > worst) worst = code;
  }
  return worst;
}

}  // namespace rt
}  // namespace tcl
