"""Front-end of the tcgen05 bf16 GEMM (``csrc/gemm_sm100.cu``): autograd function and dispatch rules.

``matmul`` / ``dense`` return ``None`` when an operand does not meet the kernel's contract (bf16 on
CUDA, 16-byte aligned, row pitches multiples of 8 elements); callers then use ``torch.matmul``.
The three products of a dense layer map to operand-major flags of the same kernel:

    forward   C  = X  · W        A K-major,  B MN-major
    dgrad     dX = dY · Wᵀ       A K-major,  B K-major
    wgrad     dW = Xᵀ · dY       A MN-major, B MN-major
"""

import ctypes
import os

import torch

from keras_b200.kernels import ops as kops

_ACT = {None: 0, "linear": 0, "relu": 1, "gelu_tanh": 2, "silu": 3, "swish": 3, "gelu_erf": 4}
_ERR = {}
_MIN_WORK = int(os.environ.get("KERAS_B200_GEMM_MIN_FLOPS", str(1 << 22)))


def _err_flag(device):
    key = (device.type, device.index)
    t = _ERR.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _ERR[key] = t
    return t


def check_errors():
    """Raise if any GEMM launch gave up on a bounded wait (reads the device flag: synchronises)."""
    for t in _ERR.values():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"tcgen05 GEMM reported a pipeline time-out (code {code}).")


def _ok_2d(t):
    return t.is_cuda and t.dtype == torch.bfloat16 and t.ndim == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.stride(0) >= t.shape[1]


def gemm(a, b, a_mn, b_mn, M, N, K, bias=None, act=0, out_dtype=torch.bfloat16):
    """Raw launch. ``a``/``b`` are 2-D bf16 tensors in the storage layout named by the major flags."""
    lib = kops._lib()
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    err = _err_flag(a.device)
    code = lib.kb200_gemm_bf16(kops._p(a), kops._p(b), kops._p(out), kops._p(bias), kops._i(M), kops._i(N), kops._i(K), kops._ll(a.stride(0)),
                               kops._ll(b.stride(0)), kops._ll(out.stride(0)), kops._i(a_mn), kops._i(b_mn), kops._i(act),
                               kops._i(1 if out_dtype == torch.float32 else 0), kops._p(err), kops._stream())
    kops._check(code, "gemm_bf16")
    return out


class GemmFn(torch.autograd.Function):
    """out[M,N] = x[M,K] @ w[K,N] (+ bias), all three products on the tcgen05 kernel."""

    @staticmethod
    def forward(ctx, x, w, bias):
        M, K = x.shape
        N = w.shape[1]
        b32 = bias.float().contiguous() if bias is not None else None
        out = gemm(x, w, 0, 1, M, N, K, bias=b32)
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        M, K = x.shape
        N = w.shape[1]
        if not _ok_2d(dy):
            dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, 0, 0, M, K, N)
        if ctx.needs_input_grad[1]:
            dw = gemm(x, dy, 1, 1, K, N, M)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(ctx.bias_dtype)
        return dx, dw, db


def _qualifies(x2, w):
    if not (_ok_2d(x2) and _ok_2d(w)):
        return False
    M, K = x2.shape
    N = w.shape[1]
    if K % 8 or N % 8 or M % 8:
        return False
    return 2 * M * N * K >= _MIN_WORK


def matmul(a, b):
    if b.ndim != 2 or a.ndim < 2 or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        return None
    lead = a.shape[:-1]
    a2 = a.reshape(-1, a.shape[-1])
    if not _qualifies(a2, b):
        return None
    out = GemmFn.apply(a2, b, None)
    return out.reshape(tuple(lead) + (b.shape[1],))


def dense(x, kernel, bias, activation_name):
    """Returns ``(output, activation_applied)`` or ``None``."""
    from keras_b200.core.variables import Variable

    w = kernel.value if isinstance(kernel, Variable) else kernel
    if not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.ndim != 2 or x.ndim < 2:
        return None
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not _qualifies(x2, w):
        return None
    b = bias.value if isinstance(bias, Variable) else bias
    needs_grad = torch.is_grad_enabled() and (x2.requires_grad or w.requires_grad or (b is not None and b.requires_grad))
    if not needs_grad:
        name = {"gelu": "gelu_erf"}.get(activation_name, activation_name)
        act = _ACT.get(name)
        fused_act = act is not None
        out = gemm(x2, w, 0, 1, x2.shape[0], w.shape[1], x2.shape[1], bias=b.float().contiguous() if b is not None else None, act=act or 0)
        return out.reshape(tuple(lead) + (w.shape[1],)), fused_act
    out = GemmFn.apply(x2, w, b)
    return out.reshape(tuple(lead) + (w.shape[1],)), activation_name in (None, "linear")
