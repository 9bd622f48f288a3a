"""Front-end of the tcgen05 flash-attention forward kernel (``csrc/attention.cu``).

``flash_attention`` takes query/key/value in the ``[batch, time, heads, head_dim]`` layout of the attention layers.  The
forward pass runs on this package's kernel; the backward pass recomputes the attention through the library's fused
attention under autograd (this package has no attention backward kernel yet), which costs one extra library forward.
For that reason the kernel is used for inference by default and for training only with ``KERAS_B200_FLASH_ATTENTION=1``;
otherwise the attention layers keep calling the library path (keras/src/backend/torch/nn.py:1124-1175).
"""

import os

import torch

from keras_b200.kernels import ops as kops

_ERR = {}


def _err_flag(device):
    t = _ERR.get(device.index)
    if t is None:
        t = _ERR[device.index] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def check_errors():
    for t in _ERR.values():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"flash-attention kernel reported a pipeline time-out (code {code}).")


def _ok(t):
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.ndim == 4 and t.stride(3) == 1 and t.data_ptr() % 16 == 0
            and all(s % 8 == 0 for s in t.stride()[:3]))


def forward(q, k, v, scale, is_causal):
    """Raw kernel launch: returns ``(out [B, Tq, H, D] bf16, lse [B, H, Tq] fp32)``."""
    lib = kops._lib()
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    out = torch.empty((B, Tq, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
    args = [kops._p(q), kops._p(k), kops._p(v), kops._p(out), kops._p(lse), kops._i(B), kops._i(Tq), kops._i(Tk), kops._i(H), kops._i(Hkv), kops._i(D)]
    for t in (q, k, v, out):
        args += [kops._ll(t.stride(1)), kops._ll(t.stride(2)), kops._ll(t.stride(0))]
    args += [kops._f(float(scale)), kops._i(1 if is_causal else 0), kops._p(_err_flag(q.device)), kops._stream()]
    kops._check(lib.kb200_flash_attention_fwd(*args), "flash_attention_fwd")
    return out, lse


class FlashAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, is_causal):
        out, _ = forward(q, k, v, scale, is_causal)
        ctx.save_for_backward(q, k, v)
        ctx.scale, ctx.is_causal = scale, is_causal
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v = ctx.saved_tensors
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
            ref = torch.nn.functional.scaled_dot_product_attention(qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=ctx.is_causal,
                                                                   scale=ctx.scale, enable_gqa=qq.shape[2] != kk.shape[2])
            dq, dk, dv = torch.autograd.grad(ref, (qq, kk, vv), grad_out.transpose(1, 2))
        return dq, dk, dv, None, None


def flash_attention(q, k, v, mask, scale, is_causal):
    """Attention on this package's kernel, or ``None`` when the call does not fit it (mask tensors, other head sizes,
    unaligned layouts) or the kernel is not selected for training."""
    if mask is not None or not (_ok(q) and _ok(k) and _ok(v)):
        return None
    D = q.shape[-1]
    if D not in (64, 128) or k.shape[-1] != D or v.shape[-1] != D or q.shape[2] % k.shape[2] or k.shape[1] != v.shape[1]:
        return None
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    mode = os.environ.get("KERAS_B200_FLASH_ATTENTION", "inference")
    if mode == "0" or (needs_grad and mode != "1"):
        return None
    if scale is None:
        scale = D ** -0.5
    if needs_grad:
        return FlashAttentionFn.apply(q, k, v, float(scale), bool(is_causal))
    return forward(q, k, v, float(scale), bool(is_causal))[0]
