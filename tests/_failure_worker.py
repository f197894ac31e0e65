"""Worker for the host-side failure tests (gloo ranks on CPU).  Mode ``leave``: rank 1 leaves between steps without a
collective in flight; rank 0's next collective must end with an error inside the short process-group timeout, and
rank 0 must find out on the host (store heartbeat) which peer is gone."""

import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=4))
    store = dist.distributed_c10d._get_default_store()
    x = torch.ones(4)
    dist.all_reduce(x)  # step 1: everyone is here
    assert x[0].item() == world
    store.set(f"alive/{rank}", "1")
    if mode == "leave":
        if rank == 1:
            store.set("alive/1", "0")  # announce, then leave between steps
            print("RANK1_LEFT", flush=True)
            os._exit(0)
        time.sleep(1.0)
        gone = [r for r in range(world) if store.get(f"alive/{r}") == b"0"]
        assert gone == [1], gone
        t0 = time.time()
        try:
            dist.all_reduce(x)  # nobody on the other side
            print("UNEXPECTED_SUCCESS", flush=True)
        except Exception as e:  # noqa: BLE001
            assert time.time() - t0 < 30
            print(f"RANK0_SAW_FAILURE after {time.time() - t0:.1f}s: {type(e).__name__}", flush=True)
        os._exit(0)


if __name__ == "__main__":
    main()
