"""Child of tests/test_failure_detection_on_cpu.py: gloo ranks, rank 1 leaves between two steps; the survivors learn of it
through the store heartbeat before their next collective, or through the collective's short timeout."""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=4))
    t = torch.ones(1)
    dist.all_reduce(t)  # step 1: everyone is there
    assert t.item() == world
    store.set(f"alive/{rank}", "1")
    dist.barrier()
    if rank == 1:
        store.set("alive/1", "0")  # leaves between steps, with nothing in flight
        os._exit(0)
    time.sleep(0.5)
    if mode == "heartbeat":
        dead = [r for r in range(world) if store.get(f"alive/{r}") == b"0"]
        if dead:
            print(f"DETECTED heartbeat dead={dead}", flush=True)
            os._exit(0)
    try:
        dist.all_reduce(torch.ones(1))  # step 2 without rank 1: the short timeout ends it with an error
        print("NOT_DETECTED", flush=True)
    except Exception as e:
        print(f"DETECTED timeout {type(e).__name__}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
