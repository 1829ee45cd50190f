// launcher_selftest: exercises the native rank launcher on the host only (no GPU needed).
//   --mode ok          every rank runs barriers and an all-to-all exchange, checks what it got
//   --mode fail        one rank calls fail() mid-run: the others' barrier returns false, nobody hangs
//   --mode exit-early  one rank exits without joining: the others time out of the barrier
//   --mode slow        one rank arrives late but within the time-out: the job still succeeds
// Exit code 0 = the scenario behaved as specified.
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>

#include "../runtime/launcher.hpp"

using tcl::rt::Launcher;

int main(int argc, char** argv) {
  int world = 4, bad_rank = 1;
  std::string mode = "ok";
  double timeout = 1.0;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "--world" && i + 1 < argc) world = std::atoi(argv[++i]);
    else if (a == "--mode" && i + 1 < argc) mode = argv[++i];
    else if (a == "--bad-rank" && i + 1 < argc) bad_rank = std::atoi(argv[++i]);
    else if (a == "--timeout" && i + 1 < argc) timeout = std::atof(argv[++i]);
    else if (a == "--probe-devices") { std::printf("devices: %d\n", Launcher::probe_device_count()); return 0; }
    else { std::printf("usage: %s [--world N] [--mode ok|fail|exit-early|slow] [--bad-rank R] [--timeout S] [--probe-devices]\n", argv[0]); return 1; }
  }
  Launcher L;
  const int rank = L.init(world);
  if (rank < 0) { std::fprintf(stderr, "launcher init failed\n"); return 2; }
  int rc = 0;
  bool saw_failure = false;
  for (int round = 0; round < 20; ++round) {
    if (mode == "fail" && rank == bad_rank && round == 5) { L.fail("injected failure"); saw_failure = true; break; }
    if (mode == "exit-early" && rank == bad_rank && round == 5) _exit(7);
    if (mode == "slow" && rank == bad_rank && round == 5) std::this_thread::sleep_for(std::chrono::milliseconds(200));
    int mine[2] = {rank * 1000 + round, round};
    int all[2 * tcl::rt::kMaxWorld];
    if (!L.exchange(round % tcl::rt::kMaxSlots, mine, sizeof(mine), all, timeout)) { saw_failure = true; break; }
    for (int r = 0; r < world; ++r)
      if (all[2 * r] != r * 1000 + round || all[2 * r + 1] != round) { std::fprintf(stderr, "rank %d: bad payload from %d\n", rank, r); rc = 4; }
    L.shm()->results[rank][0] = round;
  }
  const bool expect_failure = mode == "fail" || mode == "exit-early";
  if (expect_failure != saw_failure) rc = 5;       // a hang would have been caught by the caller's time-out
  if (expect_failure && rank != bad_rank && !L.failed()) rc = 6;
  if (rank != 0) _exit(rc);
  const int worst = L.wait_children(10.0);
  if (mode == "exit-early") {
    // the bad rank left with 7; everyone else must have returned 0
    if (worst != 7) rc = 8;
  } else if (worst != 0) rc = worst;
  std::printf("launcher_selftest mode=%s world=%d: %s (failed flag %d: %s)\n", mode.c_str(), world, rc == 0 ? "PASS" : "FAIL", L.shm()->failed.load(),
              L.shm()->failed_why);
  return rc;
}
