"""Front-end of the fp8 tensor-core GEMM (``csrc/gemm_sm100.cu``: ``kb200_gemm_fp8``; ``csrc/fp8_quant.cu``).

The float8 dtype policy of the reference quantises and de-quantises both operands to e4m3 around an ordinary matmul and the
output gradient to e5m2 in the backward pass, with delayed (history based) per-tensor scales
(keras/src/layers/core/dense.py:618-720, keras/src/quantizers/quantizers.py:560-627).  Here the quantised operands stay in
one-byte storage and the three products of the layer run on ``tcgen05.mma.kind::f8f6f4``:

    forward   y  = (s_x s_w) · q(x) q(w)ᵀ          e4m3 x e4m3
    dgrad     dx = (s_g s_w) · q(g) q(w)           e5m2 x e4m3
    wgrad     dw = (s_x s_g) · q(x)ᵀ q(g)          e4m3 x e5m2

Every operand is K-major for its product, so the quantisation kernel writes a tensor row-major and transposed from one read
and also returns max |x| for the amax history.  Scale and history updates follow the reference: they come back as the
"gradients" of the bookkeeping variables.
"""

import torch

from keras_b200.kernels import gemm as kgemm
from keras_b200.kernels import ops as kops

E4M3_MAX, E5M2_MAX = 448.0, 57344.0


def _pad16(n):
    return (n + 15) // 16 * 16


def quantize(x, scale, e5m2, row_major=True, transposed=False):
    """``x``: [R, C] bf16/fp32 (unit column stride).  Returns ``(q [R, pad16(C)] or None, qt [C, pad16(R)] or None, amax)``."""
    lib = kops._lib()
    R, C = x.shape
    dev = x.device
    q = torch.empty((R, _pad16(C)), dtype=torch.uint8, device=dev) if row_major else None
    qt = torch.empty((C, _pad16(R)), dtype=torch.uint8, device=dev) if transposed else None
    amax = torch.zeros(1, dtype=torch.int32, device=dev)
    s = scale.reshape(1).to(torch.float32)
    code = lib.kb200_fp8_quantize(kops._p(x), kops._ll(x.stride(0)), kops._i(R), kops._i(C), kops._p(s), kops._i(1 if e5m2 else 0), kops._p(q),
                                  kops._ll(q.stride(0) if q is not None else 0), kops._p(qt), kops._ll(qt.stride(0) if qt is not None else 0),
                                  kops._p(amax), kops._i(kops._dt(x)), kops._stream())
    kops._check(code, "fp8_quantize")
    return q, qt, amax.view(torch.float32)


def gemm(qa, qb, alpha, M, N, K, a_e5m2=False, b_e5m2=False, bias=None, act=0, out_dtype=torch.bfloat16):
    """``alpha * qa[M, K] @ qb[N, K]ᵀ`` on one-byte operands (both K-major, pitches multiples of 16 bytes)."""
    lib = kops._lib()
    out = torch.empty((M, N), dtype=out_dtype, device=qa.device)
    err = kgemm._err_flag(qa.device)
    code = lib.kb200_gemm_fp8(kops._p(qa), kops._p(qb), kops._p(out), kops._p(bias), kops._p(alpha), kops._i(M), kops._i(N), kops._i(K),
                              kops._ll(qa.stride(0)), kops._ll(qb.stride(0)), kops._ll(out.stride(0)), kops._i(1 if a_e5m2 else 0),
                              kops._i(1 if b_e5m2 else 0), kops._i(act), kops._i(1 if out_dtype == torch.float32 else 0), kops._p(err), kops._stream())
    kops._check(code, "gemm_fp8")
    return out


def delayed_scaling(history, scale, amax, dtype_max):
    """New scale and amax history of one tensor (one kernel): ``(scale', history')`` with ``scale' = 1 / (dtype_max /
    max(history))`` (the old scale when that maximum is zero or not finite) and ``history'`` = ``history`` rolled by one
    towards the front with ``amax`` in slot 0 (keras/src/quantizers/quantizers.py:585-606)."""
    lib = kops._lib()
    if history.dtype != torch.float32 or not history.is_contiguous() or scale.dtype != torch.float32:
        new_hist = torch.roll(history, shifts=-1).clone()
        new_hist[0] = amax.reshape(()).to(history.dtype)
        top = torch.amax(history, dim=0)
        old_sf = torch.reciprocal(scale)
        sf = torch.where(torch.isfinite(top), torch.where(top > 0.0, dtype_max / top, old_sf), old_sf)
        return torch.reciprocal(sf), new_hist
    new_scale = torch.empty_like(scale)
    new_hist = torch.empty_like(history)
    code = lib.kb200_fp8_delayed_scaling(kops._p(history), kops._i(history.numel()), kops._p(scale), kops._p(amax), kops._f(dtype_max), kops._p(new_scale),
                                         kops._p(new_hist), kops._stream())
    kops._check(code, "fp8_delayed_scaling")
    return new_scale, new_hist


class Fp8LinearFn(torch.autograd.Function):
    """``x[M, K] @ w[K, N] (+ bias)`` under the float8 policy; returns bf16.  The bias goes into the GEMM's epilogue and its
    gradient is a column sum of the output gradient (added into persistent storage when there is some)."""

    @staticmethod
    def forward(ctx, x, w, bias, x_scale, x_hist, w_scale, w_hist, g_scale, g_hist, training, bias_target=None):
        M, K = x.shape
        N = w.shape[1]
        # the weight-gradient product reads q(x) transposed, the input-gradient product q(w) row-major
        qx, qxt, x_amax = quantize(x, x_scale, False, row_major=True, transposed=bool(ctx.needs_input_grad[1]))
        qw, qwt, w_amax = quantize(w, w_scale, False, row_major=bool(ctx.needs_input_grad[0]), transposed=True)
        alpha = (x_scale.reshape(1) * w_scale.reshape(1)).float()
        y = gemm(qx, qwt, alpha, M, N, K, bias=bias.float().contiguous() if bias is not None else None)
        if training:
            ctx.new = delayed_scaling(x_hist, x_scale, x_amax, E4M3_MAX) + delayed_scaling(w_hist, w_scale, w_amax, E4M3_MAX)
        else:
            ctx.new = (None, None, None, None)
        ctx.save_for_backward(qxt, qw, x_scale, w_scale, g_scale, g_hist)
        ctx.shape = (M, K, N)
        ctx.w_dtype = w.dtype
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.bias_target = bias_target
        return y

    @staticmethod
    def backward(ctx, g):
        from keras_b200.kernels import shadow

        qxt, qw, x_scale, w_scale, g_scale, g_hist = ctx.saved_tensors
        M, K, N = ctx.shape
        if g.stride(-1) != 1:
            g = g.contiguous()
        qg, qgt, g_amax = quantize(g, g_scale, True, row_major=True, transposed=True)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(qg, qw, (g_scale.reshape(1) * w_scale.reshape(1)).float(), M, K, N, a_e5m2=True)
        if ctx.needs_input_grad[1]:
            dw = gemm(qxt, qgt, (x_scale.reshape(1) * g_scale.reshape(1)).float(), K, N, M, b_e5m2=True).to(ctx.w_dtype)
        if ctx.bias_dtype is not None and ctx.needs_input_grad[2]:
            slot = shadow.grad_slot(ctx.bias_target, (N,))
            if slot is not None:
                kops.column_sum(g, accumulate_into=slot.view(N))
            else:
                db = kops.column_sum(g).to(ctx.bias_dtype)
        new_g_scale, new_g_hist = delayed_scaling(g_hist, g_scale, g_amax, E5M2_MAX)
        nx_s, nx_h, nw_s, nw_h = ctx.new
        return dx, dw, db, nx_s, nx_h, nw_s, nw_h, new_g_scale, new_g_hist, None, None


def linear(layer, inputs, kernel, training, bias=None):
    """``inputs @ kernel (+ bias)`` for a float8 layer, or ``None`` when the shapes do not fit the kernel's contract.  ``bias``:
    a ``Variable`` (or tensor) with ``N`` elements; it is added by the GEMM's epilogue.

    An output width that is not a multiple of 16 (a 50257-word vocabulary) runs on a zero-padded kernel; the caller sees
    the first ``N`` columns of the padded result as a view."""
    if not isinstance(inputs, torch.Tensor) or not inputs.is_cuda or inputs.dtype != torch.bfloat16 or kernel.ndim != 2 or inputs.ndim < 2:
        return None
    K, N = kernel.shape
    lead = inputs.shape[:-1]
    x2 = inputs.reshape(-1, K)
    M = x2.shape[0]
    if M % 16 or K % 16 or 2 * M * N * K < (1 << 24) or x2.stride(1) != 1 or kernel.stride(1) != 1:
        return None
    if N % 16 and N < 256:
        return None
    if kernel.dtype not in (torch.bfloat16, torch.float32):
        return None
    from keras_b200.core.variables import Variable
    from keras_b200.kernels.gemm import _grad_target

    b = bias.value if isinstance(bias, Variable) else bias
    if b is not None and b.numel() != N:
        return None
    bias_target = _grad_target(bias, b) if isinstance(bias, Variable) else None
    Np = _pad16(N)
    if Np != N:
        kernel = torch.nn.functional.pad(kernel, (0, Np - N))
        if b is not None:
            b = torch.nn.functional.pad(b.reshape(-1), (0, Np - N))
            bias_target = None
    out = Fp8LinearFn.apply(x2, kernel, b.reshape(-1) if b is not None else None, layer.inputs_scale._value, layer.inputs_amax_history._value,
                            layer.kernel_scale._value, layer.kernel_amax_history._value, layer.outputs_grad_scale._value,
                            layer.outputs_grad_amax_history._value, bool(training), bias_target)
    if Np != N:
        out = out[:, :N]
    return out.reshape(tuple(lead) + (N,))
