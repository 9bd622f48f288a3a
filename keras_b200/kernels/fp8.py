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


def _new_scale(history, scale, dtype_max):
    amax = torch.amax(history, dim=0)
    old_sf = torch.reciprocal(scale)
    sf = dtype_max / amax
    sf = torch.where(amax > 0.0, sf, old_sf)
    sf = torch.where(torch.isfinite(amax), sf, old_sf)
    return torch.reciprocal(sf)


def _new_history(history, amax):
    new = torch.roll(history, shifts=-1).clone()
    new[0] = amax.reshape(()).to(history.dtype)
    return new


class Fp8LinearFn(torch.autograd.Function):
    """``x[M, K] @ w[K, N]`` under the float8 policy; returns bf16."""

    @staticmethod
    def forward(ctx, x, w, x_scale, x_hist, w_scale, w_hist, g_scale, g_hist, training):
        M, K = x.shape
        N = w.shape[1]
        # the weight-gradient product reads q(x) transposed, the input-gradient product q(w) row-major
        qx, qxt, x_amax = quantize(x, x_scale, False, row_major=True, transposed=bool(ctx.needs_input_grad[1]))
        qw, qwt, w_amax = quantize(w, w_scale, False, row_major=bool(ctx.needs_input_grad[0]), transposed=True)
        alpha = (x_scale.reshape(1) * w_scale.reshape(1)).float()
        y = gemm(qx, qwt, alpha, M, N, K)
        if training:
            ctx.new = (_new_scale(x_hist, x_scale, E4M3_MAX), _new_history(x_hist, x_amax), _new_scale(w_hist, w_scale, E4M3_MAX),
                       _new_history(w_hist, w_amax))
        else:
            ctx.new = (None, None, None, None)
        ctx.save_for_backward(qxt, qw, x_scale, w_scale, g_scale, g_hist)
        ctx.shape = (M, K, N)
        ctx.w_dtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, g):
        qxt, qw, x_scale, w_scale, g_scale, g_hist = ctx.saved_tensors
        M, K, N = ctx.shape
        if g.stride(-1) != 1:
            g = g.contiguous()
        qg, qgt, g_amax = quantize(g, g_scale, True, row_major=True, transposed=True)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(qg, qw, (g_scale.reshape(1) * w_scale.reshape(1)).float(), M, K, N, a_e5m2=True)
        if ctx.needs_input_grad[1]:
            dw = gemm(qxt, qgt, (x_scale.reshape(1) * g_scale.reshape(1)).float(), K, N, M, b_e5m2=True).to(ctx.w_dtype)
        new_g_scale = _new_scale(g_hist, g_scale, E5M2_MAX)
        new_g_hist = _new_history(g_hist, g_amax)
        nx_s, nx_h, nw_s, nw_h = ctx.new
        return dx, dw, nx_s, nx_h, nw_s, nw_h, new_g_scale, new_g_hist, None


def linear(layer, inputs, kernel, training):
    """``inputs @ kernel`` for a float8 layer, or ``None`` when the shapes do not fit the kernel's contract."""
    if not isinstance(inputs, torch.Tensor) or not inputs.is_cuda or inputs.dtype != torch.bfloat16 or kernel.ndim != 2 or inputs.ndim < 2:
        return None
    K, N = kernel.shape
    lead = inputs.shape[:-1]
    x2 = inputs.reshape(-1, K)
    M = x2.shape[0]
    if M % 16 or K % 16 or N % 16 or 2 * M * N * K < (1 << 24) or x2.stride(1) != 1 or kernel.stride(1) != 1:
        return None
    if kernel.dtype not in (torch.bfloat16, torch.float32):
        return None
    out = Fp8LinearFn.apply(x2, kernel, layer.inputs_scale._value, layer.inputs_amax_history._value, layer.kernel_scale._value,
                            layer.kernel_amax_history._value, layer.outputs_grad_scale._value, layer.outputs_grad_amax_history._value, bool(training))
    return out.reshape(tuple(lead) + (N,))
