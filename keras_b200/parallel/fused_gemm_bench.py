"""Benchmark of the fused tensor-parallel GEMMs against NCCL + cuBLAS.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29555 \\
        -m keras_b200.parallel.fused_gemm_bench [--tokens 16384] [--d 4096] [--ffn 14336] [--iters 20]

For a column-parallel projection (all-gather -> GEMM) and a row-parallel projection (GEMM -> reduce-scatter) of a
transformer MLP sharded over the N ranks, rank 0 prints one JSON line per kernel and baseline: device time (CUDA
events, max over ranks, median of ``--iters``), TFLOP/s per GPU and the fraction of the roofline, which is the slower of
the rank's FLOPs at the measured bf16 GEMM peak and the bytes the rank must move over NVLink at 770 GB/s.
"""

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    times = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    return statistics.median(times)


def single(args):
    """World size 1: the all-gather has no remote slices and the reduce-scatter reduces the rank's own staged tiles, so the
    launch exercises the tcgen05 pipeline, the staging stores and the in-kernel reduction without any peer."""
    torch.cuda.set_device(0)
    from keras_b200.parallel.fused_gemm import FusedGemmContext

    fused = FusedGemmContext()
    M, D, F = args.tokens // 128 * 128, args.d, args.ffn // 8 * 8
    x = torch.randn(M, D, device="cuda").bfloat16()
    w_up = (torch.randn(D, F, device="cuda") * 0.02).bfloat16()
    h = torch.randn(M, F, device="cuda").bfloat16()
    w_down = (torch.randn(F, D, device="cuda") * 0.02).bfloat16()
    y, _ = fused.all_gather_gemm(x, w_up)
    z = fused.gemm_reduce_scatter(h, w_down)
    torch.cuda.synchronize()
    fused.check()
    e1 = float((y.float() - x.float() @ w_up.float()).abs().max())
    e2 = float((z.float() - h.float() @ w_down.float()).abs().max())
    print(json.dumps({"single_rank": True, "tokens": M, "d": D, "ffn": F, "max_abs_err_allgather_gemm": e1, "max_abs_err_gemm_reduce_scatter": e2}))
    fused.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--copy-ctas", type=int, default=0)
    ap.add_argument("--single", action="store_true",
                    help="one process, one rank, no torch.distributed: one launch of each fused kernel (for a profiler capture of the kernel itself)")
    args = ap.parse_args()
    if args.single:
        return single(args)
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    import keras_b200 as keras
    from keras_b200.kernels.microbench import _peaks
    from keras_b200.parallel.fused_gemm import FusedGemmContext

    keras.distribution.initialize()
    rank, world = dist.get_rank(), dist.get_world_size()
    fused = FusedGemmContext(copy_ctas=args.copy_ctas)
    M, D = args.tokens, args.d
    F = args.ffn // world // 8 * 8
    Ms = M // world // 128 * 128
    M = Ms * world
    peak_tf, _, src = _peaks()
    x_rows = torch.randn(Ms, D, device="cuda").bfloat16()
    w_up = (torch.randn(D, F, device="cuda") * 0.02).bfloat16()
    h = torch.randn(M, F, device="cuda").bfloat16()
    w_down = (torch.randn(F, D, device="cuda") * 0.02).bfloat16()
    xg = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    y_rows = torch.empty(Ms, D, device="cuda", dtype=torch.bfloat16)
    yfull = torch.randn(M, D, device="cuda").bfloat16()

    def nccl_ag_gemm():
        dist.all_gather_into_tensor(xg, x_rows)
        return torch.matmul(xg, w_up)

    def nccl_gemm_rs():
        dist.reduce_scatter_tensor(y_rows, torch.matmul(h, w_down))
        return y_rows

    from keras_b200.kernels import gemm as kgemm

    rows = []
    cases = [
        ("GEMM only, gathered operand (this package)", lambda: kgemm.gemm(xg, w_up, 0, 1, M, F, D), 2.0 * M * D * F, 0),
        ("GEMM only, gathered operand (cuBLAS)", lambda: torch.matmul(xg, w_up), 2.0 * M * D * F, 0),
        ("all-gather only (NCCL)", lambda: dist.all_gather_into_tensor(xg, x_rows), 0.0, (world - 1) * Ms * D * 2),
        ("GEMM only, partial product (this package)", lambda: kgemm.gemm(h, w_down, 0, 1, M, D, F), 2.0 * M * D * F, 0),
        ("reduce-scatter only (NCCL)", lambda: dist.reduce_scatter_tensor(y_rows, yfull), 0.0, (world - 1) * Ms * D * 2),
        ("all-gather -> GEMM (fused kernel)", lambda: fused.all_gather_gemm(x_rows, w_up), 2.0 * M * D * F, (world - 1) * Ms * D * 2),
        ("all-gather -> GEMM (NCCL + cuBLAS)", nccl_ag_gemm, 2.0 * M * D * F, (world - 1) * Ms * D * 2),
        ("GEMM -> reduce-scatter (fused kernel)", lambda: fused.gemm_reduce_scatter(h, w_down), 2.0 * M * D * F, (world - 1) * Ms * D * 2),
        ("GEMM -> reduce-scatter (NCCL + cuBLAS)", nccl_gemm_rs, 2.0 * M * D * F, (world - 1) * Ms * D * 2),
    ]
    for name, fn, flops, link_bytes in cases:
        ms = _time(fn, args.iters, args.warmup)
        t_c = flops / (peak_tf * 1e12) * 1e3
        t_l = link_bytes / (LINK_GBS * 1e9) * 1e3
        rows.append({"kernel": name, "world": world, "tokens": M, "d": D, "ffn_local": F, "ms": ms, "tflops_per_gpu": flops / ms / 1e9,
                     "roofline_ms": max(t_c, t_l), "roofline_bound": "compute" if t_c >= t_l else "nvlink", "frac_of_roofline": max(t_c, t_l) / ms,
                     "peak": src})
    fused.check()
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
