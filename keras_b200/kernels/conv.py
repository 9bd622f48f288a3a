"""Front-end of the tcgen05 implicit-GEMM convolution (``csrc/conv_sm100.cu``).

``conv`` returns ``None`` when a call does not meet the kernel's contract (2-D, channels-last, bf16 on
CUDA, one group, filter count a multiple of 8, and either a 1x1 filter with any stride or a larger filter with
stride 1); the caller then uses the library convolution.  Inputs with few channels (an RGB stem) go through a
patch matrix (``kb200_im2col_rows``) followed by the same kernel.

The three products of a convolution layer (keras/src/backend/torch/nn.py:623-717 and its autograd companions):

    forward          y  = conv(x, w)          igemm, kernel rows contracted
    input gradient   dx = conv(dy, w^T, mirrored taps)   igemm, kernel columns contracted
    weight gradient  dw = x^T (*) dy          wgrad, pixels contracted, fp32 reduce-add of pixel slices

``want_stats`` makes the forward kernel's epilogue leave per-channel partial sums of y and y^2, which the following
BatchNormalization turns into its batch statistics without reading y again.
"""

import ctypes
import os

import torch

from keras_b200.kernels import grad_merge
from keras_b200.kernels import ops as kops
from keras_b200.kernels import shadow
from keras_b200.kernels.gemm import _err_flag

_MIN_WORK = int(os.environ.get("KERAS_B200_CONV_MIN_FLOPS", str(1 << 24)))
_ENABLED = os.environ.get("KERAS_B200_CONV", "1") != "0"
_MAX_PATCH = 1024  # widest patch-matrix row (elements) for the few-channel path


class ConvStats:
    """Partial sums left by the convolution epilogue: ``partials`` [grid, 2, ld] fp32 and the launch plan."""

    __slots__ = ("partials", "grid", "n_tiles", "bn", "ld", "count")

    def __init__(self, partials, grid, n_tiles, bn, ld, count):
        self.partials, self.grid, self.n_tiles, self.bn, self.ld, self.count = partials, grid, n_tiles, bn, ld, count


def _i(v):
    return ctypes.c_int(int(v))


def _ll(v):
    return ctypes.c_longlong(int(v))


def _igemm(a, a_dims, a_strides, w, out, out_dims, out_strides, taps, b_kmajor, rows_per_tap, w_cols, stats=None, stats_ld=0, plan=None,
           accumulate=False):
    """a_dims = (N, H, W, Ca); out_dims = (Ho, Wo, Cn); strides are (sw, sh, sn) in elements; taps = (R, S, dh0, dh_step, dw0, dw_step)."""
    lib = kops._lib()
    N, H, W, Ca = a_dims
    Ho, Wo, Cn = out_dims
    R, S, dh0, dhs, dw0, dws = taps
    err = _err_flag(a.device)
    code = lib.kb200_conv_igemm(kops._p(a), kops._p(w), kops._p(out), None, kops._p(stats) if stats is not None else kops._vp(0), _i(stats_ld),
                                plan if plan is not None else kops._vp(0), _i(N), _i(H), _i(W), _i(Ca), _ll(a_strides[0]), _ll(a_strides[1]),
                                _ll(a_strides[2]), _i(Ho), _i(Wo), _i(Cn), _ll(out_strides[0]), _ll(out_strides[1]), _ll(out_strides[2]), _i(R), _i(S),
                                _i(dh0), _i(dhs), _i(dw0), _i(dws), _i(b_kmajor), _i(rows_per_tap), _i(w_cols), _i(0), _i(1 if accumulate else 0),
                                kops._p(err), kops._stream())
    kops._check(code, "conv_igemm")


def _wgrad(x, x_dims, x_strides, dy, dy_dims, dy_strides, dw, taps):
    lib = kops._lib()
    N, H, W, Cin = x_dims
    Ho, Wo, Cout = dy_dims
    R, S, dh0, dhs, dw0, dws = taps
    err = _err_flag(x.device)
    code = lib.kb200_conv_wgrad(kops._p(x), kops._p(dy), kops._p(dw), _i(N), _i(H), _i(W), _i(Cin), _ll(x_strides[0]), _ll(x_strides[1]), _ll(x_strides[2]),
                                _i(Ho), _i(Wo), _i(Cout), _ll(dy_strides[0]), _ll(dy_strides[1]), _ll(dy_strides[2]), _i(R), _i(S), _i(dh0), _i(dhs),
                                _i(dw0), _i(dws), kops._p(err), kops._stream())
    kops._check(code, "conv_wgrad")


def _nhwc_strides(H, W, C):
    return (C, W * C, H * W * C)


class _Geom:
    """Static description of one convolution call (hashable pieces only)."""

    __slots__ = ("N", "H", "W", "Cin", "Cout", "R", "S", "sh", "sw", "dh", "dw", "pt", "pl", "Ho", "Wo", "patch", "seg")


class ConvFn(torch.autograd.Function):
    """y = conv2d(x, w) for channels-last bf16 tensors on the implicit-GEMM kernel; all three products run on it."""

    @staticmethod
    def forward(ctx, x, w, g, grad_target, partials, plan, merge=None):
        N, H, W, Cin, Cout, Ho, Wo = g.N, g.H, g.W, g.Cin, g.Cout, g.Ho, g.Wo
        y = torch.empty((N, Ho, Wo, Cout), dtype=torch.bfloat16, device=x.device)
        ld = partials.shape[-1] if partials is not None else 0
        saved_a = x
        if g.patch:
            # few input channels: rows of patches, then a 1x1 convolution over R*seg "channels"
            K = g.R * g.seg
            cols = torch.empty((N * Ho * Wo, K), dtype=torch.bfloat16, device=x.device)
            lib = kops._lib()
            code = lib.kb200_im2col_rows(kops._p(x), kops._p(cols), _i(N), _i(H), _i(W), _i(Cin), _i(Ho), _i(Wo), _i(g.R), _i(g.S), _i(g.sh), _i(g.sw),
                                         _i(g.pt), _i(g.pl), _i(g.seg), _i(kops._dt(x)), kops._stream())
            kops._check(code, "im2col_rows")
            wp = torch.nn.functional.pad(w.reshape(g.R, g.S * Cin, Cout), (0, 0, 0, g.seg - g.S * Cin)).reshape(K, Cout)
            M = N * Ho * Wo
            _igemm(cols, (1, 1, M, K), (K, M * K, M * K), wp, y, (1, M, Cout), (Cout, M * Cout, M * Cout), (1, 1, 0, 0, 0, 0), 0, K, Cout, partials, ld,
                   plan)
            saved_a = cols
        elif g.R == 1 and g.S == 1:
            if g.sh == 1 and g.sw == 1:
                M = N * H * W
                _igemm(x, (1, 1, M, Cin), (Cin, M * Cin, M * Cin), w, y, (1, M, Cout), (Cout, M * Cout, M * Cout), (1, 1, 0, 0, 0, 0), 0, Cin, Cout,
                       partials, ld, plan)
            else:
                _igemm(x, (N, Ho, Wo, Cin), (g.sw * Cin, g.sh * W * Cin, H * W * Cin), w, y, (Ho, Wo, Cout), _nhwc_strides(Ho, Wo, Cout),
                       (1, 1, 0, 0, 0, 0), 0, Cin, Cout, partials, ld, plan)
        else:
            _igemm(x, (N, H, W, Cin), _nhwc_strides(H, W, Cin), w, y, (Ho, Wo, Cout), _nhwc_strides(Ho, Wo, Cout),
                   (g.R, g.S, -g.pt, g.dh, -g.pl, g.dw), 0, Cin, Cout, partials, ld, plan)
        ctx.save_for_backward(saved_a, w)
        ctx.g = g
        ctx.grad_target = grad_target
        ctx.merge = merge  # grad_merge.MergeSlot of the input activation, or None
        ctx.w_dtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        a, w = ctx.saved_tensors
        g = ctx.g
        N, H, W, Cin, Cout, Ho, Wo = g.N, g.H, g.W, g.Cin, g.Cout, g.Ho, g.Wo
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        dy = dy.contiguous()
        dx = dw = None
        one = g.R == 1 and g.S == 1
        if ctx.needs_input_grad[0]:
            # another consumer of the same activation may already have left its gradient: then this one is added into it
            merged = None if g.patch else grad_merge.target(ctx.merge, (N, H, W, Cin), torch.bfloat16)
            add = merged is not None
            if one and g.sh == 1 and g.sw == 1:
                M = N * H * W
                dx = merged if add else torch.empty((N, H, W, Cin), dtype=torch.bfloat16, device=dy.device)
                _igemm(dy, (1, 1, M, Cout), (Cout, M * Cout, M * Cout), w, dx, (1, M, Cin), (Cin, M * Cin, M * Cin), (1, 1, 0, 0, 0, 0), 1, Cin, Cout,
                       accumulate=add)
            elif one:
                dx = merged if add else torch.zeros((N, H, W, Cin), dtype=torch.bfloat16, device=dy.device)
                _igemm(dy, (N, Ho, Wo, Cout), _nhwc_strides(Ho, Wo, Cout), w, dx, (Ho, Wo, Cin), (g.sw * Cin, g.sh * W * Cin, H * W * Cin),
                       (1, 1, 0, 0, 0, 0), 1, Cin, Cout, accumulate=add)
            else:
                dx = merged if add else torch.empty((N, H, W, Cin), dtype=torch.bfloat16, device=dy.device)
                _igemm(dy, (N, Ho, Wo, Cout), _nhwc_strides(Ho, Wo, Cout), w, dx, (H, W, Cin), _nhwc_strides(H, W, Cin),
                       (g.R, g.S, g.pt, -g.dh, g.pl, -g.dw), 1, Cin, Cout, accumulate=add)
            if add:
                dx = None  # already inside the other consumer's gradient tensor
            else:
                grad_merge.offer(ctx.merge, dx)
        if ctx.needs_input_grad[1]:
            acc = None if g.patch else shadow.grad_slot(ctx.grad_target, w.shape)
            in_place = acc is not None
            if g.patch:
                K = g.R * g.seg
                M = N * Ho * Wo
                buf = torch.zeros((K, Cout), dtype=torch.float32, device=dy.device)
                _wgrad(a, (1, 1, M, K), (K, M * K, M * K), dy, (1, M, Cout), (Cout, M * Cout, M * Cout), buf, (1, 1, 0, 0, 0, 0))
                dw = buf.reshape(g.R, g.seg, Cout)[:, : g.S * Cin].reshape(g.R, g.S, Cin, Cout).to(ctx.w_dtype)
            else:
                buf = acc if in_place else torch.zeros((g.R * g.S * Cin, Cout), dtype=torch.float32, device=dy.device)
                if one and g.sh == 1 and g.sw == 1:
                    M = N * H * W
                    _wgrad(a, (1, 1, M, Cin), (Cin, M * Cin, M * Cin), dy, (1, M, Cout), (Cout, M * Cout, M * Cout), buf, (1, 1, 0, 0, 0, 0))
                elif one:
                    _wgrad(a, (N, Ho, Wo, Cin), (g.sw * Cin, g.sh * W * Cin, H * W * Cin), dy, (Ho, Wo, Cout), _nhwc_strides(Ho, Wo, Cout), buf,
                           (1, 1, 0, 0, 0, 0))
                else:
                    _wgrad(a, (N, H, W, Cin), _nhwc_strides(H, W, Cin), dy, (Ho, Wo, Cout), _nhwc_strides(Ho, Wo, Cout), buf,
                           (g.R, g.S, -g.pt, g.dh, -g.pl, g.dw))
                if not in_place:
                    dw = buf.reshape(g.R, g.S, Cin, Cout).to(ctx.w_dtype)
        return dx, dw, None, None, None, None, None


def _geometry(x, kernel, strides, padding, dilation):
    if x.ndim != 4 or kernel.ndim != 4:
        return None
    N, H, W, Cin = x.shape
    R, S, kin, Cout = kernel.shape
    if kin != Cin or Cout % 8 or N == 0 or H == 0 or W == 0:
        return None
    sh, sw = strides
    dh, dw = dilation
    if isinstance(padding, str):
        mode = padding.lower()
        if mode == "same":
            Ho, Wo = -(-H // sh), -(-W // sw)
            pt = max((Ho - 1) * sh + (R - 1) * dh + 1 - H, 0) // 2
            pl = max((Wo - 1) * sw + (S - 1) * dw + 1 - W, 0) // 2
        elif mode == "valid":
            pt = pl = 0
            Ho = (H - (R - 1) * dh - 1) // sh + 1
            Wo = (W - (S - 1) * dw - 1) // sw + 1
        else:
            return None
    else:
        pt, pl = (int(p) for p in padding)
        Ho = (H + 2 * pt - (R - 1) * dh - 1) // sh + 1
        Wo = (W + 2 * pl - (S - 1) * dw - 1) // sw + 1
    if Ho <= 0 or Wo <= 0:
        return None
    g = _Geom()
    g.N, g.H, g.W, g.Cin, g.Cout, g.R, g.S = N, H, W, Cin, Cout, R, S
    g.sh, g.sw, g.dh, g.dw, g.pt, g.pl, g.Ho, g.Wo = sh, sw, dh, dw, pt, pl, Ho, Wo
    g.patch, g.seg = False, 0
    if Cin % 8 == 0:
        if R == 1 and S == 1:
            if pt or pl:
                return None
            return g
        if sh == 1 and sw == 1:
            return g
        return None
    # few input channels: patch matrix
    seg = -(-(S * Cin) // 8) * 8
    if dh != 1 or dw != 1 or R * seg > _MAX_PATCH:
        return None
    g.patch, g.seg = True, seg
    return g


def _target_param(variable, w):
    """The fp32 parameter whose persistent ``.grad`` the weight gradient can be added into: only when ``w`` is the
    variable's bf16 shadow (then no gradient tensor has to flow back through the read)."""
    p = getattr(variable, "_value", None)
    if p is None or getattr(variable, "_shadow", None) is None or not p.requires_grad or p.dtype != torch.float32 or w.dtype != torch.bfloat16:
        return None
    if getattr(variable, "_shard_slices", None) is not None or p.numel() != w.numel() or w.grad_fn is None:
        return None
    return p


def conv(x, kernel, strides, padding, data_format, dilation, grad_target=None, want_stats=False):
    """``conv2d`` on the sm_100a kernel or ``None``.  With ``want_stats`` the result is ``(y, ConvStats)``.

    ``grad_target``: the ``Variable`` that ``kernel`` was read from; when its gradient lives in persistent fp32 storage
    the weight-gradient kernel adds into it directly."""
    if not _ENABLED or data_format != "channels_last" or not isinstance(x, torch.Tensor) or not isinstance(kernel, torch.Tensor):
        return None
    if kernel.dtype != torch.bfloat16 or not x.is_cuda:
        return None
    g = _geometry(x, kernel, tuple(strides), padding, tuple(dilation))
    if g is None:
        return None
    if g.patch:
        if x.dtype not in (torch.bfloat16, torch.float32) or (torch.is_grad_enabled() and x.requires_grad):
            return None
    elif x.dtype != torch.bfloat16:
        return None
    if 2 * g.N * g.Ho * g.Wo * g.Cout * g.R * g.S * g.Cin < _MIN_WORK:
        return None
    x = x.contiguous()
    w = kernel if kernel.is_contiguous() else kernel.contiguous()
    if x.data_ptr() % 16 or w.data_ptr() % 16:
        return None
    partials = plan = None
    stats = None
    if want_stats:
        lib = kops._lib()
        plan = (ctypes.c_int * 3)()
        if g.patch or (g.R == 1 and g.S == 1 and g.sh == 1 and g.sw == 1):
            dims, taps, depth = (1, 1, g.N * g.Ho * g.Wo), (1, 1, 0), (g.R * g.seg if g.patch else g.Cin)
        else:
            dims, taps, depth = (g.N, g.Ho, g.Wo), (g.R, g.S, g.dh), g.Cin
        lib.kb200_conv_igemm_plan(_i(dims[0]), _i(dims[1]), _i(dims[2]), _i(depth), _i(g.Cout), _i(taps[0]), _i(taps[1]), _i(taps[2]), plan)
        grid, n_tiles, bn = plan[0], plan[1], plan[2]
        ld = n_tiles * bn
        partials = torch.empty((grid, 2, ld), dtype=torch.float32, device=x.device)
        stats = ConvStats(partials, grid, n_tiles, bn, ld, g.N * g.Ho * g.Wo)
    target = _target_param(grad_target, w) if grad_target is not None and w is kernel else None
    y = ConvFn.apply(x, w, g, target, partials, plan, grad_merge.slot_of(x))
    return (y, stats) if want_stats else y
