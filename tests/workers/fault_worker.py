"""One rank of a failure-detection test. All failures are made on the host: a rank that exits, never
joins, is slow, or aborts. Prints one line 'RESULT <what>' that the test reads."""
import argparse
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from dccl_b200 import Communicator, DcclError  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True)
    ap.add_argument("--victim", type=int, default=1)
    args = ap.parse_args()
    t0 = time.time()
    try:
        comm = Communicator()
    except DcclError as e:
        print("RESULT init_failed code=%d after=%.1f" % (e.code, time.time() - t0))
        return
    rank, world = comm.rank, comm.world
    x = np.ones(1 << 16, dtype=np.float32)
    try:
        for it in range(200):
            if args.mode in ("exit_mid_run", "exit_then_shrink") and rank == args.victim and it == 50:
                os._exit(9)             # dies without leaving the group
            if args.mode == "abort_local" and rank == args.victim and it == 50:
                comm.abort()
            if args.mode == "stall" and rank == args.victim and it == 50:
                time.sleep(3.0)         # longer than the transfer timeout the test sets
            comm.all_reduce(x.copy())
        code, msg = comm.last_error()
        print("RESULT completed code=%d" % code)
        comm.finalize()
    except DcclError as e:
        code, msg = comm.last_error()
        if args.mode == "exit_then_shrink":
            # the survivors go on as a smaller group: dense ranks in the old order, collectives work again
            new = comm.shrink()
            y = np.full(1000, float(rank), dtype=np.float64)
            new.all_reduce(y)
            alive = [r for r in range(world) if r != args.victim]
            ok = new.world == world - 1 and new.rank == alive.index(rank) and bool(np.all(y == float(sum(alive))))
            lst = np.zeros(new.world, dtype=np.int32)
            new.all_gather(np.array([rank], dtype=np.int32), lst)
            ok = ok and list(lst) == alive
            print("RESULT shrunk ok=%d world=%d rank=%d first_error=%d" % (int(ok), new.world, new.rank, e.code))
            new.finalize()
            comm.finalize()
            return
        print("RESULT error code=%d async=%d after=%.1f msg=%s" % (e.code, code, time.time() - t0, msg))
        # a failed group is not finalized collectively; just leave


if __name__ == "__main__":
    main()
