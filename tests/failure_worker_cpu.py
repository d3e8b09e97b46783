"""Child of test_failure_detection_cpu.py: one gloo rank of a job in which a failure is made on the host.

``silent_rank``  three ranks publish heartbeats in a TCP store; the last one stops publishing (it stays alive and keeps its
                 process group). The others must learn of it from the store before their next collective, name the rank,
                 and carry on among themselves on a group built from the survivors.
``absent_rank``  two ranks; one never joins an all-reduce. The other's collective must end with an error after the
                 process group's (short) time limit instead of waiting forever.
"""

import datetime
import os
import sys
import time

import torch
import torch.distributed as dist


def main() -> None:
    rank, world, mode = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), sys.argv[1]
    from phyai_b200.parallel import PeerLostError
    from phyai_b200.parallel.health import Heartbeat

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=rank == 0,
                          timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3 if mode == "absent_rank" else 60))
    if mode == "silent_rank":
        hb = Heartbeat(store, rank, world, interval_s=0.05).start()
        dist.barrier()
        hb.check_peers(2.0)                                # everyone is there
        dist.barrier()
        victim = world - 1
        if rank == victim:
            hb.stop()                                      # the failure: this rank goes silent, nothing else changes
            assert hb.stale_peers(1.0) == []               # it still sees the others
        lost, deadline = None, time.time() + 10
        if rank != victim:
            while time.time() < deadline:                  # what a scheduler does before each launch
                try:
                    hb.check_peers(0.5)
                except PeerLostError as e:
                    lost = str(e)
                    break
                time.sleep(0.05)
            assert lost is not None and f"[{victim}]" in lost, lost
            print(f"[rank {rank}] LOST {victim}", flush=True)
        survivors = [r for r in range(world) if r != victim]
        group = dist.new_group(survivors)                  # every rank takes part in creating it, members use it
        if rank != victim:
            x = torch.tensor([float(rank + 1)])
            dist.all_reduce(x, group=group)
            assert x.item() == sum(r + 1 for r in survivors)
            print(f"[rank {rank}] RECOVERED {x.item():.0f}", flush=True)
        hb.stop()
    elif mode == "absent_rank":
        dist.barrier()
        if rank == 0:
            t0 = time.time()
            try:
                dist.all_reduce(torch.ones(1))             # the partner never issues its half
                print("[rank 0] NO_ERROR", flush=True)
            except Exception as e:  # noqa: BLE001 - the backend's timeout error type varies between versions
                print(f"[rank 0] TIMED_OUT after {time.time() - t0:.1f} s: {type(e).__name__}", flush=True)
            store.set("release", "1")
        else:
            store.wait(["release"], datetime.timedelta(seconds=30))   # the failure: this rank sits out the collective
            print("[rank 1] RELEASED", flush=True)
    else:
        raise SystemExit(f"unknown mode {mode}")
    # leave in order: the rank that hosts the store goes last, or the others' last reads find the server gone
    sys.stdout.flush()
    if rank != 0:
        store.set(f"bye/{rank}", "1")
    else:
        store.wait([f"bye/{r}" for r in range(1, world)], datetime.timedelta(seconds=30))
    os._exit(0)      # a process group that saw a timeout may not tear down cleanly: leave without the collective shutdown


if __name__ == "__main__":
    main()
