"""CPU ranks (gloo): one rank leaves between steps, or goes silent; the others notice on the host
before their next step instead of entering a collective with it."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tileccl_b200.parallel import group as G  # noqa: E402
from tileccl_b200.parallel.health import PeerFailure, PeerHealth  # noqa: E402


def main():
    mode = sys.argv[1]
    rank, world, _ = G.init(backend="gloo")
    h = PeerHealth()
    dist.barrier()
    detected = None
    for step in range(6):
        if rank == 1 and step == 3:
            if mode == "leave":
                h.leave("injected departure at step 3")
            # mode "silent": just stop beating and stop taking part
            time.sleep(3.0 if mode == "silent" else 0.5)
            os._exit(0)
        if step >= 3:
            # give the notice / the silence time to show; a live rank keeps beating meanwhile
            for _ in range(2 if mode == "leave" else 9):
                time.sleep(0.2)
                h.beat()
        try:
            h.check(timeout_s=1.0)
        except PeerFailure as e:
            detected = e
            break
        t = torch.ones(1)
        dist.all_reduce(t)                # the "step": only entered when every peer is known alive
        h.beat()
    ok = detected is not None and detected.rank == 1 and step == 3
    print(f"rank {rank}: detected={detected} at step {step} -> {'HEALTH_OK' if ok else 'HEALTH_FAIL'}", flush=True)
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
