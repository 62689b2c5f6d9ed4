import json
import sys
import time

import torch
import torch.distributed as dist

from chronicals_b200.parallel.bootstrap import init_distributed
from chronicals_b200.parallel.watchdog import PeerFailure, watchdog_from_process_group


def main():
    out = sys.argv[1]
    rank, _, world = init_distributed("gloo", timeout_s=8)
    wd = watchdog_from_process_group(timeout=5.0, interval=0.2).start()
    steps = 0
    try:
        for step in range(10):
            wd.check(step)                                   # before any collective of this step
            if rank == 1 and step == 2:
                raise RuntimeError("simulated data-loader failure")
            t = torch.ones(4)
            try:
                dist.all_reduce(t)
            except RuntimeError:
                # the peer left after our check: the short process-group timeout ended the collective;
                # the watchdog now says who it was
                time.sleep(0.5)
                wd.check(step)
                raise
            steps += 1
            time.sleep(0.3)
    except PeerFailure as e:
        if rank == 0:
            with open(out, "w") as f:
                json.dump({"detected_rank": e.rank, "steps_done": steps, "reason": e.reason}, f)
    except RuntimeError as e:
        if rank == 1:
            wd.report_failure(e)
            time.sleep(12.0)                                  # outlive the peer's collective timeout
        else:
            raise
    finally:
        wd.stop()
    # no destroy_process_group barrier: the peers may already be gone


if __name__ == "__main__":
    main()
