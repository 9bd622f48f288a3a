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
from keras_b200.kernels import shadow

_ACT = {None: 0, "linear": 0, "relu": 1, "gelu_tanh": 2, "silu": 3, "swish": 3, "gelu_erf": 4}
_ERR = {}
_MIN_WORK = int(os.environ.get("KERAS_B200_GEMM_MIN_FLOPS", str(1 << 22)))
# measured on GPT-2 (launch-bound step): 2 % slower than the bf16 gradient + one add, so off unless asked for
_WGRAD_IN_PLACE = os.environ.get("KERAS_B200_WGRAD_IN_PLACE", "1") == "1"


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


def _ok_2d(t, any_width=False):
    if any_width and t.is_cuda and t.dtype == torch.bfloat16 and t.ndim == 2 and t.is_contiguous() and t.data_ptr() % 16 == 0:
        return True  # a weight whose width is padded to a multiple of 8 before the launch
    return t.is_cuda and t.dtype == torch.bfloat16 and t.ndim == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.stride(0) >= t.shape[1]


_SM_COUNT = {}


def _sm_count(device):
    n = _SM_COUNT.get(device.index)
    if n is None:
        n = _SM_COUNT[device.index] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def split_k_for(M, N, K, device):
    """K slices for a product whose output has too few 128x256 tiles to fill the GPU (weight gradients: small M x N, K = tokens)."""
    tiles = -(-M // 128) * -(-N // 256)
    sms = _sm_count(device)
    if tiles * 2 > sms or K < 2048:
        return 1
    return max(1, min(sms // tiles, K // 512))


def gemm(a, b, a_mn, b_mn, M, N, K, bias=None, act=0, out_dtype=torch.bfloat16, split_k=1, accumulate_into=None):
    """Raw launch. ``a``/``b`` are 2-D bf16 tensors in the storage layout named by the major flags.

    ``split_k > 1`` accumulates K slices into a zeroed fp32 buffer (TMA reduce stores) and casts to ``out_dtype``.
    ``accumulate_into``: fp32 [M, N] tensor that the product is added to in place (returned)."""
    lib = kops._lib()
    err = _err_flag(a.device)
    if accumulate_into is not None:
        acc = accumulate_into
        code = lib.kb200_gemm_bf16_splitk(kops._p(a), kops._p(b), kops._p(acc), None, kops._i(M), kops._i(N), kops._i(K), kops._ll(a.stride(0)),
                                          kops._ll(b.stride(0)), kops._ll(acc.stride(0)), kops._i(a_mn), kops._i(b_mn), kops._i(0), kops._i(1),
                                          kops._i(-max(1, split_k)), kops._p(err), kops._stream())
        kops._check(code, "gemm_bf16")
        return acc
    if split_k > 1 and bias is None and act == 0:
        acc = torch.zeros((M, N), dtype=torch.float32, device=a.device)
        code = lib.kb200_gemm_bf16_splitk(kops._p(a), kops._p(b), kops._p(acc), None, kops._i(M), kops._i(N), kops._i(K), kops._ll(a.stride(0)),
                                          kops._ll(b.stride(0)), kops._ll(acc.stride(0)), kops._i(a_mn), kops._i(b_mn), kops._i(0), kops._i(1),
                                          kops._i(split_k), kops._p(err), kops._stream())
        kops._check(code, "gemm_bf16")
        return acc if out_dtype == torch.float32 else acc.to(out_dtype)
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    code = lib.kb200_gemm_bf16(kops._p(a), kops._p(b), kops._p(out), kops._p(bias), kops._i(M), kops._i(N), kops._i(K), kops._ll(a.stride(0)),
                               kops._ll(b.stride(0)), kops._ll(out.stride(0)), kops._i(a_mn), kops._i(b_mn), kops._i(act),
                               kops._i(1 if out_dtype == torch.float32 else 0), kops._p(err), kops._stream())
    kops._check(code, "gemm_bf16")
    return out


class GemmFn(torch.autograd.Function):
    """out[M,N] = x[M,K] @ w[K,N] (+ bias), all three products on the tcgen05 kernel.

    A width ``N`` that is not a multiple of 8 (a 50257-word vocabulary) runs on a zero-padded copy of the weight:
    the padded output keeps its 16-byte row pitch and the caller sees its first ``N`` columns as a view."""

    @staticmethod
    def forward(ctx, x, w, bias, grad_target=None, bias_target=None):
        """``grad_target``: the fp32 parameter behind ``w`` (its bf16 shadow) when its ``.grad`` is persistent fp32 storage: the
        weight gradient is then accumulated there by the GEMM itself and no bf16 gradient tensor is produced."""
        M, K = x.shape
        N = w.shape[1]
        ctx.grad_target = grad_target
        ctx.bias_target = bias_target
        Np = (N + 7) // 8 * 8
        b32 = bias.float().contiguous() if bias is not None else None
        if Np != N:
            w = torch.nn.functional.pad(w, (0, Np - N))
            if b32 is not None:
                b32 = torch.nn.functional.pad(b32, (0, Np - N))
        out = gemm(x, w, 0, 1, M, Np, K, bias=b32)
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.n = N
        return out if Np == N else out[:, :N]

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        M, K = x.shape
        N, Np = ctx.n, w.shape[1]
        if Np != N:
            if dy.dtype == torch.bfloat16 and dy.stride(1) == 1 and dy.stride(0) == Np and dy.data_ptr() % 16 == 0:
                # the gradient is itself the leading columns of a padded buffer (produced for a padded logits view)
                dyp = dy.as_strided((M, Np), (Np, 1))
                dyp[:, N:].zero_()
            else:
                dyp = torch.empty((M, Np), dtype=torch.bfloat16, device=dy.device)
                dyp[:, :N].copy_(dy)
                dyp[:, N:].zero_()
            dy = dyp
        elif not _ok_2d(dy):
            dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, 0, 0, M, K, Np)
        if ctx.needs_input_grad[1]:
            split = split_k_for(K, Np, M, x.device)
            g = shadow.grad_slot(ctx.grad_target, (K, N)) if Np == N and N % 4 == 0 else None
            if g is not None:
                gemm(x, dy, 1, 1, K, N, M, split_k=split, accumulate_into=g.view(K, N))  # dw stays None: already accumulated
            else:
                dw = gemm(x, dy, 1, 1, K, Np, M, split_k=split)
                if Np != N:
                    dw = dw[:, :N]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            g = shadow.grad_slot(ctx.bias_target, (N,)) if Np == N else None
            if g is not None:
                kops.column_sum(dy, accumulate_into=g.view(N))  # db stays None: already accumulated
            else:
                db = kops.column_sum(dy)[:N].to(ctx.bias_dtype)
        return (dx, dw, db, None, None)[: len(ctx.needs_input_grad)]


def _qualifies(x2, w):
    if not (_ok_2d(x2) and _ok_2d(w, any_width=True)):
        return False
    M, K = x2.shape
    N = w.shape[1]
    if K % 8 or M % 8 or (N % 8 and N < 256):
        return False
    return 2 * M * N * K >= _MIN_WORK


def matmul(a, b):
    if b.ndim != 2 or a.ndim < 2 or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        return None
    lead = a.shape[:-1]
    a2 = a.reshape(-1, a.shape[-1])
    if not _qualifies(a2, b):
        return None
    out = GemmFn.apply(a2, b, None, None, None)
    return out.reshape(tuple(lead) + (b.shape[1],))


def _grad_target(variable, w):
    """The fp32 parameter to accumulate the weight gradient into: only when ``w`` is the variable's bf16 shadow read."""
    p = getattr(variable, "_value", None)
    if not _WGRAD_IN_PLACE or variable is None or p is None or getattr(variable, "_shadow", None) is None or not p.requires_grad or p.dtype != torch.float32 or w.dtype != torch.bfloat16:
        return None
    if getattr(variable, "_shard_slices", None) is not None or p.numel() != w.numel():
        return None
    return p


def dense(x, kernel, bias, activation_name, kernel_shape=None):
    """Returns ``(output, activation_applied)`` or ``None``.  ``kernel`` may be a ``Variable`` (reshaped to the 2-D
    ``kernel_shape`` when given) or a tensor."""
    from keras_b200.core.variables import Variable

    w = kernel.value if isinstance(kernel, Variable) else kernel
    if kernel_shape is not None:
        w = w.reshape(kernel_shape)
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
        N = w.shape[1]
        b32 = b.float().contiguous() if b is not None else None
        if N % 8:
            w = torch.nn.functional.pad(w, (0, 8 - N % 8))
            b32 = torch.nn.functional.pad(b32, (0, 8 - N % 8)) if b32 is not None else None
        out = gemm(x2, w, 0, 1, x2.shape[0], w.shape[1], x2.shape[1], bias=b32, act=act or 0)
        if N % 8:
            out = out[:, :N]
        return out.reshape(tuple(lead) + (N,)), fused_act
    target = _grad_target(kernel, w) if isinstance(kernel, Variable) else None
    bias_target = _grad_target(bias, b) if isinstance(bias, Variable) else None
    out = GemmFn.apply(x2, w, b, target, bias_target)
    return out.reshape(tuple(lead) + (w.shape[1],)), activation_name in (None, "linear")
