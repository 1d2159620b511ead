"""Worker for the failure-detection tests (gloo CPU ranks). Not collected.
argv: mode ("bye" | "silent" | "pgtimeout"), out dir"""
import json
import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=timedelta(seconds=3 if mode == "pgtimeout" else 60))
    from idrak_b200.cluster.heartbeat import Heartbeat, RankLeft
    from idrak_b200.cluster.sim import RankTimeout
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.1, timeout=1.0)
    hb.wait_all_alive()
    report = {"rank": rank, "steps": 0, "error": None}
    try:
        for step in range(6):
            if mode != "pgtimeout":
                hb.check()                                  # before launching anything that waits on a peer
            if rank == world - 1 and step == 2:             # this rank leaves between steps, nothing in flight
                if mode == "bye":
                    hb.bye("test says so")
                elif mode == "silent":
                    hb.close()
                report["error"] = "left"
                time.sleep(1.5)                             # the sockets stay open while the peers look at the store
                break
            t = torch.ones(4) * rank
            dist.all_reduce(t)
            report["steps"] = step + 1
            if rank != world - 1 or step != 1:
                time.sleep(0.4)                             # "loading the next batch": the leaver is gone before the check
            if mode == "silent" and step >= 1:
                time.sleep(0.6)                             # give a stale heartbeat time to show
    except (RankLeft, RankTimeout) as e:
        report["error"] = f"{type(e).__name__}: {e}"
    except RuntimeError as e:                               # the process group's own timeout
        report["error"] = f"RuntimeError: {str(e)[:200]}"
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(report, f)
    hb.close()
    os._exit(0)                                             # no orderly shutdown: peers may be gone


if __name__ == "__main__":
    main()
