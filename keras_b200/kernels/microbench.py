"""Kernel micro-benchmarks with CUDA-event timing and roofline fractions.

    python -m keras_b200.kernels.microbench gemm --m 8192 --n 8192 --k 8192
    python -m keras_b200.kernels.microbench gemm_fp8 --m 8192 --n 8192 --k 8192
    python -m keras_b200.kernels.microbench attention --batch 16 --seq 1024 --heads 12 --head-dim 64
    python -m keras_b200.kernels.microbench optim --tensors 32 --rows 4096 --channels 1024
    python -m keras_b200.kernels.microbench bn --rows 802816 --channels 256
    python -m keras_b200.kernels.microbench pool --batch 256
    python -m keras_b200.kernels.microbench norm --rows 16384 --channels 768
    python -m keras_b200.kernels.microbench xent --rows 16384 --channels 50257
    python -m keras_b200.kernels.microbench conv --batch 256            (every ResNet-50 convolution shape)
    python -m keras_b200.kernels.microbench conv --batch 32 --case 5    (one shape)

Each prints one JSON line per case: time (median of ``--iters`` after ``--warmup``), achieved TFLOP/s or GB/s and the
fraction of the measured peak (``MEASURED_PEAKS.json`` beside the package's parent directory when present, else the
fall-back 1590 TFLOP/s / 6650 GB/s).  A buffer larger than L2 is written between iterations so inputs come from HBM.
With ``--once`` exactly one launch of the kernel under test is made after set-up (for profiler captures of a single launch).
"""

import argparse
import json
import os
import statistics

import torch


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.add_(1.0)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def bench_gemm(args, flush):
    from keras_b200.kernels import gemm

    M, N, K = args.m, args.n, args.k
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    ours = lambda: gemm.gemm(a, b, False, True, M, N, K)
    lib = lambda: torch.matmul(a, b)
    if args.once:
        ours()
        torch.cuda.synchronize()
        return []
    ref = torch.matmul(a.float()[:256], b.float())
    err = float((ours()[:256].float() - ref).abs().max() / ref.abs().max())
    t_ours, t_lib = _time(ours, args.iters, args.warmup, flush), _time(lib, args.iters, args.warmup, flush)
    tf, _, src = _peaks()
    flops = 2.0 * M * N * K
    return [{"kernel": "kb200_gemm_bf16 (tcgen05)", "shape": [M, N, K], "ms": t_ours, "tflops": flops / t_ours / 1e9, "frac_of_peak": flops / t_ours / 1e9 / tf,
             "peak": src, "rel_err_vs_fp32": err},
            {"kernel": "torch.matmul (cuBLAS)", "shape": [M, N, K], "ms": t_lib, "tflops": flops / t_lib / 1e9, "frac_of_peak": flops / t_lib / 1e9 / tf, "peak": src}]


def bench_gemm_fp8(args, flush):
    """e4m3 x e4m3 product of the float8 policy: quantisation kernels timed separately from the GEMM."""
    from keras_b200.kernels import fp8

    M, N, K = args.m, args.n, args.k
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    sa, sb = torch.tensor(0.01, device="cuda"), torch.tensor(0.01, device="cuda")
    qa, _, _ = fp8.quantize(a, sa, False)
    _, qbt, _ = fp8.quantize(b, sb, False, row_major=False, transposed=True)
    alpha = (sa * sb).reshape(1)
    ours = lambda: fp8.gemm(qa, qbt, alpha, M, N, K)
    if args.once:
        ours()
        torch.cuda.synchronize()
        return []
    ref = (qa[:256, :K].view(torch.float8_e4m3fn).float() @ qbt[:, :K].view(torch.float8_e4m3fn).float().t()) * float(alpha)
    err = float((ours()[:256].float() - ref).abs().max() / ref.abs().max())
    t = _time(ours, args.iters, args.warmup, flush)
    t_q = _time(lambda: fp8.quantize(a, sa, False, row_major=True, transposed=True), args.iters, args.warmup, flush)
    tf, bw, src = _peaks()
    flops = 2.0 * M * N * K
    return [{"kernel": "kb200_gemm_fp8 (tcgen05 kind::f8f6f4)", "shape": [M, N, K], "ms": t, "tflops": flops / t / 1e9,
             "x_measured_bf16_peak": flops / t / 1e9 / tf, "frac_of_nominal_fp8_peak": flops / t / 1e9 / 4500.0, "peak": src, "rel_err_vs_fp32": err},
            {"kernel": "kb200_fp8_quantize (row-major + transposed + amax)", "shape": [M, K], "ms": t_q, "gbs": M * K * 4 / t_q / 1e6,
             "frac_of_peak": M * K * 4 / t_q / 1e6 / bw, "peak": src}]


def bench_attention(args, flush):
    """Causal self-attention forward, [B, T, H, D] layout: this package's tcgen05 kernel against the library's fused attention."""
    import torch.nn.functional as F

    from keras_b200.kernels import attention

    B, T, H, D = args.batch, args.seq, args.heads, args.head_dim
    q, k, v = (torch.randn(B, T, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    scale = D ** -0.5
    ours = lambda: attention.forward(q, k, v, scale, True)
    lib = lambda: F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, scale=scale)
    if args.once:
        ours()
        torch.cuda.synchronize()
        return []
    err = float((ours()[0].float() - lib().transpose(1, 2).float()).abs().max())
    t_ours, t_lib = _time(ours, args.iters, args.warmup, flush), _time(lib, args.iters, args.warmup, flush)
    tf, _, src = _peaks()
    flops = 4.0 * B * H * T * T * D / 2
    return [{"kernel": "flash_fwd_kernel (tcgen05)", "shape": [B, T, H, D], "causal": True, "ms": t_ours, "tflops": flops / t_ours / 1e9,
             "frac_of_peak": flops / t_ours / 1e9 / tf, "peak": src, "max_abs_diff_vs_library": err},
            {"kernel": "F.scaled_dot_product_attention (library)", "shape": [B, T, H, D], "causal": True, "ms": t_lib, "tflops": flops / t_lib / 1e9,
             "frac_of_peak": flops / t_lib / 1e9 / tf, "peak": src}]


def bench_optim(args, flush):
    """Fused multi-tensor AdamW step (update, decay, bf16 shadow write, gradient zeroing) over `--tensors` parameters of
    `--rows` x `--channels` floats, against the library's fused AdamW."""
    from keras_b200.kernels import ops as kops

    n, numel = args.tensors, args.rows * args.channels
    params = [torch.randn(numel, device="cuda") for _ in range(n)]
    grads = [torch.randn(numel, device="cuda") for _ in range(n)]
    m = [torch.zeros(numel, device="cuda") for _ in range(n)]
    v = [torch.zeros(numel, device="cuda") for _ in range(n)]
    shadows = [torch.empty(numel, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    plan = kops.OptimizerPlan(params, grads, m, v, shadows, [0.1] * n)
    ours = lambda: plan.adam(3e-4, 0.9, 0.999, 1e-8, lr=3e-4, grad_scale=1.0, zero_grad=True)
    if args.once:
        ours()
        torch.cuda.synchronize()
        return []
    for p_ in params:
        p_.grad = torch.randn_like(p_)
    ref = torch.optim.AdamW(params, lr=3e-4, weight_decay=0.1, fused=True)
    t_ours, t_lib = _time(ours, args.iters, args.warmup, flush), _time(ref.step, args.iters, args.warmup, flush)
    _, bw, src = _peaks()
    ob = n * numel * (4 * 8 + 2)  # read p, g, m, v; write p, m, v and g := 0 (fp32); write the bf16 shadow
    lb = n * numel * 4 * 7
    return [{"kernel": "kb200_fused_adam (update + decay + bf16 shadow + zero grad)", "tensors": n, "numel": numel, "ms": t_ours, "gbs": ob / t_ours / 1e6,
             "frac_of_peak": ob / t_ours / 1e6 / bw, "peak": src},
            {"kernel": "torch.optim.AdamW(fused=True)", "tensors": n, "numel": numel, "ms": t_lib, "gbs": lb / t_lib / 1e6,
             "frac_of_peak": lb / t_lib / 1e6 / bw, "peak": src}]


def bench_bn(args, flush):
    from keras_b200.kernels import ops as kops

    M, C = args.rows, args.channels
    x = torch.randn(M, C, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    gamma = torch.ones(C, device="cuda", requires_grad=True)
    beta = torch.zeros(C, device="cuda", requires_grad=True)
    mm, mv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    fwd = lambda: kops.FusedBatchNormAct.apply(x, gamma, beta, None, mm, mv, 0.99, 1e-3, True, None)
    if args.once:
        fwd()
        torch.cuda.synchronize()
        return []
    y = fwd()
    dy = torch.randn_like(y)
    bwd = lambda: torch.autograd.grad(fwd(), (x, gamma, beta), dy)
    t_f = _time(lambda: fwd(), args.iters, args.warmup, flush)
    t_fb = _time(bwd, args.iters, args.warmup, flush)
    _, bw, src = _peaks()
    nbytes = M * C * 2
    fwd_bytes = 3 * nbytes + nbytes // 16          # stats read + apply read/write + mask write
    bwd_bytes = 5 * nbytes + 2 * (nbytes // 16)    # reduce reads dy,x ; apply reads dy,x writes dx ; mask twice
    return [{"kernel": "bn forward (stats+apply+relu)", "shape": [M, C], "ms": t_f, "gbs": fwd_bytes / t_f / 1e6, "frac_of_peak": fwd_bytes / t_f / 1e6 / bw, "peak": src},
            {"kernel": "bn forward+backward", "shape": [M, C], "ms": t_fb, "gbs": (fwd_bytes + bwd_bytes) / t_fb / 1e6,
             "frac_of_peak": (fwd_bytes + bwd_bytes) / t_fb / 1e6 / bw, "peak": src}]


def bench_pool(args, flush):
    from keras_b200.kernels import dispatch

    x = torch.randn(args.batch, 112, 112, 64, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    fwd = lambda: dispatch.max_pool2d(x, (3, 3), (2, 2), "valid", zero_pad=((1, 1), (1, 1)))
    if args.once:
        fwd()
        torch.cuda.synchronize()
        return []
    y = fwd()
    dy = torch.randn_like(y)
    t_f = _time(lambda: fwd(), args.iters, args.warmup, flush)
    t_fb = _time(lambda: torch.autograd.grad(fwd(), x, dy), args.iters, args.warmup, flush)
    _, bw, src = _peaks()
    fb = x.numel() * 2 + y.numel() * 3
    bb = y.numel() * 3 + x.numel() * 2
    return [{"kernel": "zero-pad+maxpool forward", "shape": list(x.shape), "ms": t_f, "gbs": fb / t_f / 1e6, "frac_of_peak": fb / t_f / 1e6 / bw, "peak": src},
            {"kernel": "zero-pad+maxpool forward+backward", "shape": list(x.shape), "ms": t_fb, "gbs": (fb + bb) / t_fb / 1e6,
             "frac_of_peak": (fb + bb) / t_fb / 1e6 / bw, "peak": src}]


def bench_norm(args, flush):
    from keras_b200.kernels import ops as kops

    rows, D = args.rows, args.channels
    x = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    g = torch.ones(D, device="cuda", requires_grad=True)
    b = torch.zeros(D, device="cuda", requires_grad=True)
    fwd = lambda: kops.FusedNorm.apply(x, g, b, 1e-5, False)
    if args.once:
        fwd().backward(torch.ones(rows, D, device="cuda", dtype=torch.bfloat16))
        torch.cuda.synchronize()
        return []
    dy = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
    t_f = _time(lambda: fwd(), args.iters, args.warmup, flush)
    t_fb = _time(lambda: torch.autograd.grad(fwd(), (x, g, b), dy), args.iters, args.warmup, flush)
    _, bw, src = _peaks()
    fb, bb = rows * D * 4, rows * D * 6
    return [{"kernel": "layer-norm forward", "shape": [rows, D], "ms": t_f, "gbs": fb / t_f / 1e6, "frac_of_peak": fb / t_f / 1e6 / bw, "peak": src},
            {"kernel": "layer-norm forward+backward", "shape": [rows, D], "ms": t_fb, "gbs": (fb + bb) / t_fb / 1e6,
             "frac_of_peak": (fb + bb) / t_fb / 1e6 / bw, "peak": src}]


def bench_xent(args, flush):
    from keras_b200.kernels import ops as kops

    rows, V = args.rows, args.channels
    ld = (V + 7) // 8 * 8
    logits = torch.randn(rows, ld, device="cuda", dtype=torch.bfloat16)[:, :V].requires_grad_(True)
    labels = torch.randint(0, V, (rows,), device="cuda")
    fwd = lambda: kops.FusedSoftmaxXent.apply(logits, labels)
    if args.once:
        fwd().sum().backward()
        torch.cuda.synchronize()
        return []
    g = torch.ones(rows, device="cuda")
    t_f = _time(lambda: fwd(), args.iters, args.warmup, flush)
    t_fb = _time(lambda: torch.autograd.grad(fwd(), logits, g), args.iters, args.warmup, flush)
    _, bw, src = _peaks()
    fb, bb = rows * V * 2, rows * V * 4
    return [{"kernel": "softmax-xent forward", "shape": [rows, V], "ms": t_f, "gbs": fb / t_f / 1e6, "frac_of_peak": fb / t_f / 1e6 / bw, "peak": src},
            {"kernel": "softmax-xent forward+backward", "shape": [rows, V], "ms": t_fb, "gbs": (fb + bb) / t_fb / 1e6,
             "frac_of_peak": (fb + bb) / t_fb / 1e6 / bw, "peak": src}]


# ResNet-50 v1 convolution shapes at 224x224 (keras/src/applications/resnet.py:219-273): (H, Cin, Cout, k, stride, count per step)
RESNET50_CONVS = [
    (224, 3, 64, 7, 2, 1),
    (56, 64, 64, 1, 1, 1), (56, 64, 64, 3, 1, 3), (56, 64, 256, 1, 1, 4), (56, 256, 64, 1, 1, 2),
    (56, 256, 128, 1, 2, 1), (28, 128, 128, 3, 1, 4), (28, 128, 512, 1, 1, 4), (56, 256, 512, 1, 2, 1), (28, 512, 128, 1, 1, 3),
    (28, 512, 256, 1, 2, 1), (14, 256, 256, 3, 1, 6), (14, 256, 1024, 1, 1, 6), (28, 512, 1024, 1, 2, 1), (14, 1024, 256, 1, 1, 5),
    (14, 1024, 512, 1, 2, 1), (7, 512, 512, 3, 1, 3), (7, 512, 2048, 1, 1, 3), (14, 1024, 2048, 1, 2, 1), (7, 2048, 512, 1, 1, 2),
]


def bench_conv(args, flush):
    """Forward / input-gradient / weight-gradient time of each shape on the tcgen05 kernel and on the library (cuDNN)."""
    import torch.nn.functional as F

    from keras_b200.kernels import conv as kconv

    peak, _, src = _peaks()
    N = args.batch
    cases = RESNET50_CONVS if args.case < 0 else [RESNET50_CONVS[args.case]]
    totals = {"ours": 0.0, "library": 0.0}
    for (H, Cin, Cout, k, s, count) in cases:
        stem = Cin < 8
        x = torch.randn(N, H, H, Cin, device="cuda").to(torch.bfloat16)
        w = (torch.randn(k, k, Cin, Cout, device="cuda") / (k * k * Cin) ** 0.5).to(torch.bfloat16)
        padding = (3, 3) if stem else "same"
        xg = x.clone().requires_grad_(not stem)
        wg = w.clone().requires_grad_(True)
        y = kconv.conv(xg, wg, (s, s), padding, "channels_last", (1, 1))
        assert y is not None
        dy = torch.randn_like(y)
        xc = x.permute(0, 3, 1, 2).requires_grad_(not stem)  # channels-last memory format view for the library
        wc = w.permute(3, 2, 0, 1).contiguous(memory_format=torch.channels_last).requires_grad_(True)
        pad = 3 if stem else (k // 2 if s == 1 else 0)
        yl = F.conv2d(xc, wc, stride=s, padding=pad)
        dyl = dy.permute(0, 3, 1, 2)
        if args.once:
            kconv.conv(x, w, (s, s), padding, "channels_last", (1, 1))
            y.backward(dy)
            torch.cuda.synchronize()
            return

        def ours_fwd():
            kconv.conv(x, w, (s, s), padding, "channels_last", (1, 1))

        def ours_bwd():
            y.backward(dy, retain_graph=True)

        def lib_fwd():
            F.conv2d(xc.detach(), wc.detach(), stride=s, padding=pad)

        def lib_bwd():
            yl.backward(dyl, retain_graph=True)

        t_of, t_ob = _time(ours_fwd, args.iters, args.warmup, flush), _time(ours_bwd, args.iters, args.warmup, flush)
        t_lf, t_lb = _time(lib_fwd, args.iters, args.warmup, flush), _time(lib_bwd, args.iters, args.warmup, flush)
        Ho = y.shape[1]
        flops = 2.0 * N * Ho * Ho * Cout * k * k * Cin
        nb = 1 if stem else 2
        totals["ours"] += count * (t_of + t_ob)
        totals["library"] += count * (t_lf + t_lb)
        yield {"kernel": "conv_tcgen05", "shape": f"{N}x{H}x{H}x{Cin}->{Cout} k{k} s{s}", "count": count, "fwd_ms": round(t_of, 4), "bwd_ms": round(t_ob, 4),
               "library_fwd_ms": round(t_lf, 4), "library_bwd_ms": round(t_lb, 4), "fwd_tflops": round(flops / t_of / 1e9, 1),
               "bwd_tflops": round(nb * flops / t_ob / 1e9, 1), "fwd_frac_of_%s_peak" % src: round(flops / t_of / 1e9 / peak, 3)}
    yield {"kernel": "conv_tcgen05", "sum_over_step_ms": {k_: round(v, 3) for k_, v in totals.items()}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_fp8", "attention", "optim", "bn", "pool", "norm", "xent", "conv"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--rows", type=int, default=802816)
    ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--tensors", type=int, default=32)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--case", type=int, default=-1)
    ap.add_argument("--once", action="store_true")
    args = ap.parse_args()
    flush = torch.zeros(96 * 1024 * 1024, device="cuda")  # 384 MB > 126 MB L2
    for row in {"gemm": bench_gemm, "gemm_fp8": bench_gemm_fp8, "attention": bench_attention, "optim": bench_optim, "bn": bench_bn, "pool": bench_pool, "norm": bench_norm, "xent": bench_xent, "conv": bench_conv}[args.what](args, flush):
        print(json.dumps(row))


if __name__ == "__main__":
    main()
