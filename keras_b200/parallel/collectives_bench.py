"""All-reduce benchmark: this package's peer-memory kernel against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29556 \\
        -m keras_b200.parallel.collectives_bench [--mbytes 102] [--iters 20]

Rank 0 prints one JSON line per implementation: device time (CUDA events, max over ranks, median), algorithm bandwidth
(bytes / time) and bus bandwidth (algorithm bandwidth x 2 (N-1)/N).
"""

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    return statistics.median(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbytes", type=float, default=102.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    import keras_b200 as keras
    from keras_b200.parallel.collectives import P2PAllReducer

    keras.distribution.initialize()
    rank, world = dist.get_rank(), dist.get_world_size()
    n = int(args.mbytes * 1e6 / 4) // 4 * 4
    red = P2PAllReducer(n)
    red.flat.normal_()
    other = torch.randn(n, device="cuda")
    rows = []
    for name, fn in (("peer-memory two-shot all-reduce (this package)", lambda: red.all_reduce(scale=1.0 / world)),
                     ("NCCL all-reduce", lambda: dist.all_reduce(other))):
        ms = _time(fn, args.iters, args.warmup)
        alg = n * 4 / ms / 1e6
        rows.append({"kernel": name, "world": world, "mbytes": n * 4 / 1e6, "ms": ms, "algbw_gbs": alg, "busbw_gbs": alg * 2 * (world - 1) / world})
    red.check(wait=True)
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.barrier()
    red.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
