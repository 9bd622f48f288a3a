"""Neural-network ops (``keras.ops.nn``): activations, conv/pool, normalisation, losses, attention.

Semantics follow keras/src/ops/nn.py and keras/src/backend/torch/nn.py:21-1721.  Hot ops
(layer/RMS normalisation, softmax-cross-entropy, attention, conv) route through
``keras_b200.kernels.dispatch`` to the sm_100a kernels when the input lives on a B200.
"""

import math

import numpy as np
import torch
import torch.nn.functional as F

from keras_b200.core import config
from keras_b200.core.dtypes import result_type, standardize_dtype, to_torch_dtype
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.kernels import dispatch
from keras_b200.ops._dispatch import op
from keras_b200.ops.numpy import _floatize, _t

_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


# --- activations --------------------------------------------------------------------------

@op("nn")
def relu(x):
    return F.relu(_t(x))


@op("nn")
def relu6(x):
    return F.relu6(_t(x))


@op("nn")
def sigmoid(x):
    return torch.sigmoid(_floatize(x))


@op("nn")
def sparse_sigmoid(x):
    x = _floatize(x)
    return torch.where(x <= -1, torch.zeros_like(x), torch.where(x >= 1, torch.ones_like(x), 0.5 * (x + 1)))


@op("nn")
def tanh(x):
    return torch.tanh(_floatize(x))


@op("nn")
def tanh_shrink(x):
    x = _floatize(x)
    return x - torch.tanh(x)


@op("nn")
def softplus(x):
    return F.softplus(_floatize(x))


@op("nn")
def softsign(x):
    return F.softsign(_floatize(x))


@op("nn")
def soft_shrink(x, threshold=0.5):
    return F.softshrink(_floatize(x), lambd=threshold)


@op("nn")
def sparse_plus(x):
    x = _floatize(x)
    return torch.where(x <= -1, torch.zeros_like(x), torch.where(x < 1, 0.25 * (x + 1) ** 2, x))


@op("nn", also=("keras.ops.swish", "keras.ops.nn.swish"))
def silu(x):
    return F.silu(_floatize(x))


swish = silu


@op("nn")
def squareplus(x, b=4):
    x = _floatize(x)
    if not isinstance(b, (int, float)):
        b = _t(b).to(x.dtype)
    return (x + torch.sqrt(x * x + b)) / 2


@op("nn")
def log_sigmoid(x):
    return F.logsigmoid(_floatize(x))


@op("nn")
def leaky_relu(x, negative_slope=0.2):
    return F.leaky_relu(_floatize(x), negative_slope=negative_slope)


@op("nn")
def hard_sigmoid(x):
    return F.hardsigmoid(_floatize(x))


@op("nn", also=("keras.ops.hard_swish", "keras.ops.nn.hard_swish"))
def hard_silu(x):
    return F.hardswish(_floatize(x))


hard_swish = hard_silu


@op("nn")
def elu(x, alpha=1.0):
    return F.elu(_floatize(x), alpha)


@op("nn")
def selu(x):
    return F.selu(_floatize(x))


@op("nn")
def gelu(x, approximate=True):
    return F.gelu(_floatize(x), approximate="tanh" if approximate else "none")


@op("nn")
def celu(x, alpha=1.0):
    return F.celu(_floatize(x), alpha=alpha)


@op("nn")
def glu(x, axis=-1):
    return F.glu(_floatize(x), dim=axis)


@op("nn")
def hard_tanh(x):
    x = _t(x)
    if not x.dtype.is_floating_point:
        return torch.clamp(x, min=-1, max=1)  # integer inputs keep their dtype
    return F.hardtanh(x, min_val=-1.0, max_val=1.0)


@op("nn")
def hard_shrink(x, threshold=0.5):
    return F.hardshrink(_floatize(x), lambd=threshold)


@op("nn")
def threshold(x, threshold, default_value):
    return F.threshold(_floatize(x), threshold=threshold, value=default_value)


def _fused_softmax(x, axis, log):
    """The row kernel on CUDA tensors (fp32 arithmetic on bf16 / fp32 storage, no up-cast copy), or ``None``."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16) or x.ndim == 0:
        return None
    from keras_b200.kernels import dispatch

    if axis is None:
        out = dispatch.softmax(x.reshape(-1), log=log)
        return None if out is None else out.reshape(x.shape)
    axes = sorted({a % x.ndim for a in (axis if isinstance(axis, (list, tuple)) else (axis,))})
    keep = [i for i in range(x.ndim) if i not in axes]
    perm = keep + axes
    if perm == list(range(x.ndim)):
        rows = x.reshape(tuple(x.shape[: len(keep)]) + (-1,))
        out = dispatch.softmax(rows, log=log)
        return None if out is None else out.reshape(x.shape)
    y = x.permute(perm)
    out = dispatch.softmax(y.reshape(tuple(y.shape[: len(keep)]) + (-1,)), log=log)
    if out is None:
        return None
    return out.reshape(y.shape).permute([perm.index(i) for i in range(x.ndim)])


def _reduce_axes_softmax(fn, x, axis):
    x = _floatize(x)
    fused = _fused_softmax(x, axis, fn is torch.log_softmax)
    if fused is not None:
        return fused
    ori = x.dtype
    if ori in (torch.float16, torch.bfloat16):
        x = x.to(torch.float32)
    if axis is None:
        out = fn(x.reshape(-1), dim=-1).reshape(x.shape)
    elif isinstance(axis, (list, tuple)):
        axes = [a % x.ndim for a in axis]
        keep = [i for i in range(x.ndim) if i not in axes]
        perm = keep + axes
        y = x.permute(perm)
        lead = y.shape[: len(keep)]
        z = fn(y.reshape(tuple(lead) + (-1,)), dim=-1).reshape(y.shape)
        inv = [perm.index(i) for i in range(x.ndim)]
        out = z.permute(inv)
    else:
        out = fn(x, dim=axis)
    return out.to(ori)


@op("nn")
def softmax(x, axis=-1):
    return _reduce_axes_softmax(torch.softmax, x, axis)


@op("nn")
def log_softmax(x, axis=-1):
    return _reduce_axes_softmax(torch.log_softmax, x, axis)


@op("nn")
def sparsemax(x, axis=-1):
    # The threshold follows keras/src/backend/torch/nn.py:199-218 term by term: it is built from the sum of the running
    # sums over the support (not from the running sum at the support's size), and checkpoints trained against that
    # activation expect exactly this function.
    x = _floatize(x)
    z, _ = torch.sort(x, dim=axis, descending=True)
    running = torch.cumsum(z, dim=axis)
    shape = [1] * x.ndim
    shape[axis] = -1
    rank = torch.arange(1, x.shape[axis] + 1, device=x.device, dtype=x.dtype).reshape(shape)
    support = z - (running - 1) / rank > 0
    size = torch.sum(support, dim=axis, keepdim=True)
    tau = (torch.sum(torch.where(support, running, torch.zeros_like(running)), dim=axis, keepdim=True) - 1) / size
    return torch.clamp(x - tau, min=0)


# --- pooling / conv -----------------------------------------------------------------------

def _to_cf(x, data_format):
    """channels_last tensor → torch channels-first *view* (no copy)."""
    if data_format == "channels_last":
        n = x.ndim
        return x.permute(0, n - 1, *range(1, n - 1))
    return x


def _from_cf(x, data_format):
    if data_format == "channels_last":
        n = x.ndim
        return x.permute(0, *range(2, n), 1)
    return x


def _tuple(v, n):
    if isinstance(v, int):
        return (v,) * n
    return tuple(int(e) for e in v)


def _same_pad_amounts(in_size, k, s, d=1):
    out = -(-in_size // s)
    eff = (k - 1) * d + 1
    total = max((out - 1) * s + eff - in_size, 0)
    return total // 2, total - total // 2


def _pool(x, pool_size, strides, padding, data_format, kind):
    x = _t(x)
    data_format = config.standardize_data_format(data_format)
    nsp = x.ndim - 2
    pool_size = _tuple(pool_size, nsp)
    strides = pool_size if strides is None else _tuple(strides, nsp)
    padding = padding.lower()
    if kind == "max" and nsp == 2 and data_format == "channels_last" and x.is_cuda:
        from keras_b200.kernels import dispatch

        out = dispatch.max_pool2d(x, pool_size, strides, padding)
        if out is not None:
            return out
    if kind == "avg" and nsp == 2 and data_format == "channels_last" and x.is_cuda:
        from keras_b200.kernels import dispatch

        out = dispatch.avg_pool2d(x, pool_size, strides, padding)
        if out is not None:
            return out
    xc = _to_cf(x, data_format)
    fn_max = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nsp]
    fn_avg = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nsp]
    if padding == "same":
        pads = [_same_pad_amounts(xc.shape[2 + i], pool_size[i], strides[i]) for i in range(nsp)]
        if any(p != (0, 0) for p in pads):
            flat = []
            for lo, hi in reversed(pads):
                flat.extend([lo, hi])
            if kind == "max":
                fill = -math.inf if xc.dtype in _FLOATS else torch.iinfo(xc.dtype).min
                xc = F.pad(xc, flat, value=fill)
                out = fn_max(xc, pool_size, strides)
            else:
                # average over valid elements only
                ones = torch.ones((1, 1) + tuple(xc.shape[2:]), dtype=xc.dtype, device=xc.device)
                num = fn_avg(F.pad(xc, flat), pool_size, strides)
                den = fn_avg(F.pad(ones, flat), pool_size, strides)
                out = num / den
            return _from_cf(out, data_format)
    out = fn_max(xc, pool_size, strides) if kind == "max" else fn_avg(xc, pool_size, strides)
    return _from_cf(out, data_format)


@op("nn")
def max_pool(inputs, pool_size, strides=None, padding="valid", data_format=None):
    return _pool(inputs, pool_size, strides, padding, data_format, "max")


@op("nn")
def average_pool(inputs, pool_size, strides=None, padding="valid", data_format=None):
    return _pool(_floatize(inputs), pool_size, strides, padding, data_format, "avg")


def _adaptive(x, output_size, data_format, kind):
    x = _floatize(x)
    data_format = config.standardize_data_format(data_format)
    nsp = x.ndim - 2
    output_size = _tuple(output_size, nsp)
    fn = {("max", 1): F.adaptive_max_pool1d, ("max", 2): F.adaptive_max_pool2d, ("max", 3): F.adaptive_max_pool3d,
          ("avg", 1): F.adaptive_avg_pool1d, ("avg", 2): F.adaptive_avg_pool2d, ("avg", 3): F.adaptive_avg_pool3d}[(kind, nsp)]
    return _from_cf(fn(_to_cf(x, data_format), output_size), data_format)


@op("nn")
def adaptive_max_pool(inputs, output_size, data_format=None):
    return _adaptive(inputs, output_size, data_format, "max")


@op("nn")
def adaptive_average_pool(inputs, output_size, data_format=None):
    return _adaptive(inputs, output_size, data_format, "avg")


def _conv_kernel_to_torch(kernel):
    """Keras kernel (*spatial, in/groups, out) → torch (out, in/groups, *spatial) view."""
    n = kernel.ndim
    return kernel.permute(n - 1, n - 2, *range(n - 2))


def _explicit_same(xc, ksize, strides, dilation):
    nsp = len(ksize)
    pads = [_same_pad_amounts(xc.shape[2 + i], ksize[i], strides[i], dilation[i]) for i in range(nsp)]
    if all(lo == hi for lo, hi in pads):
        return xc, tuple(lo for lo, _ in pads)
    flat = []
    for lo, hi in reversed(pads):
        flat.extend([lo, hi])
    return F.pad(xc, flat), 0


@op("nn")
def conv(inputs, kernel, strides=1, padding="valid", data_format=None, dilation_rate=1):
    x, k = _t(inputs), _t(kernel)
    if x.dtype != k.dtype:
        d = to_torch_dtype(result_type(x.dtype, k.dtype))
        x, k = x.to(d), k.to(d)
    data_format = config.standardize_data_format(data_format)
    nsp = x.ndim - 2
    strides = _tuple(strides, nsp)
    dilation = _tuple(dilation_rate, nsp)
    fused = dispatch.conv(x, k, strides, padding, data_format, dilation)
    if fused is not None:
        return fused
    xc = _to_cf(x, data_format)
    in_ch = xc.shape[1]
    kin = k.shape[-2]
    if in_ch % kin != 0:
        raise ValueError(
            "The number of input channels must be evenly divisible by kernel's in_channels. "
            f"Received input channels {in_ch} and kernel in_channels {kin}."
        )
    groups = in_ch // kin
    kt = _conv_kernel_to_torch(k)
    pad = 0
    if not isinstance(padding, str):
        pad = _tuple(padding, nsp)  # explicit symmetric zero padding per spatial dimension
    elif padding.lower() == "same":
        xc, pad = _explicit_same(xc, tuple(k.shape[:nsp]), strides, dilation)
    elif padding.lower() == "causal":
        left = (k.shape[0] - 1) * dilation[0]
        xc = F.pad(xc, (left, 0))
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nsp]
    out = fn(xc, kt, stride=strides, padding=pad, dilation=dilation, groups=groups)
    return _from_cf(out, data_format)


@op("nn")
def depthwise_conv(inputs, kernel, strides=1, padding="valid", data_format=None, dilation_rate=1):
    k = _t(kernel)
    sp = tuple(k.shape[:-2])
    k2 = k.reshape(sp + (1, k.shape[-2] * k.shape[-1]))
    return conv(inputs, k2, strides, padding, data_format, dilation_rate)


@op("nn")
def separable_conv(inputs, depthwise_kernel, pointwise_kernel, strides=1, padding="valid", data_format=None, dilation_rate=1):
    dw = depthwise_conv(inputs, depthwise_kernel, strides, padding, data_format, dilation_rate)
    return conv(dw, pointwise_kernel, 1, "valid", data_format, 1)


@op("nn")
def conv_transpose(inputs, kernel, strides=1, padding="valid", output_padding=None, data_format=None, dilation_rate=1):
    x, k = _t(inputs), _t(kernel)
    if x.dtype != k.dtype:
        d = to_torch_dtype(result_type(x.dtype, k.dtype))
        x, k = x.to(d), k.to(d)
    data_format = config.standardize_data_format(data_format)
    nsp = x.ndim - 2
    strides = _tuple(strides, nsp)
    dilation = _tuple(dilation_rate, nsp)
    ksize = tuple(k.shape[:nsp])
    xc = _to_cf(x, data_format)
    # Keras transposed kernel: (*spatial, out, in) → torch (in, out, *spatial)
    kt = k.permute(k.ndim - 1, k.ndim - 2, *range(nsp))
    opad = None if output_padding is None else _tuple(output_padding, nsp)
    # The full transposed convolution (no padding) has (in - 1) * stride + eff samples per axis.  Keras semantics
    # (keras/src/backend/common/backend_utils.py:8-50, 215-268) select a window of it that is in general not centred:
    #   valid: everything, plus `output_padding` zeros on the right (default: up to (in - 1) * stride + max(eff, stride));
    #   same:  `total = stride + eff - 2` samples are dropped (with output_padding: eff + eff % 2 - 2 + output_padding are
    #          kept back), the larger half on the left but never more than eff - 1.
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nsp]
    out = fn(xc, kt, stride=strides, padding=0, output_padding=0, dilation=dilation)
    mode = padding.lower()
    if mode not in ("valid", "same"):
        raise ValueError(f"The `padding` argument must be one of 'valid', 'same'. Received: padding={padding}")
    grow = []  # zeros to append per axis (left, right), innermost axis first as F.pad wants them
    for i in range(nsp):
        eff = (ksize[i] - 1) * dilation[i] + 1
        s_i = strides[i]
        if mode == "valid":
            extra = (max(eff, s_i) - eff) if opad is None else opad[i]
            keep_left, keep_right = eff - 1, eff - 1 + extra
        else:
            kept = (s_i + eff - 2) if opad is None else (eff + eff % 2 - 2 + opad[i])
            keep_left = min(kept // 2 + kept % 2, eff - 1)
            keep_right = kept - keep_left
        drop_left, drop_right = (eff - 1) - keep_left, (eff - 1) - keep_right
        axis = 2 + i
        length = out.shape[axis]
        out = out.narrow(axis, max(drop_left, 0), length - max(drop_left, 0) - max(drop_right, 0))
        grow.append((max(-drop_left, 0), max(-drop_right, 0)))
    if any(l or r for l, r in grow):
        flat = []
        for l, r in reversed(grow):
            flat.extend([l, r])
        out = F.pad(out, flat)
    return _from_cf(out, data_format)


@op("nn")
def one_hot(x, num_classes, axis=-1, dtype=None, sparse=False):
    x = _t(x).long()
    dtype = dtype or config.floatx()
    valid = (x >= 0) & (x < num_classes)
    out = F.one_hot(torch.where(valid, x, torch.zeros_like(x)), num_classes)
    out = out * valid.unsqueeze(-1)
    out = out.to(to_torch_dtype(dtype))
    if axis != -1 and axis != out.ndim - 1:
        out = torch.movedim(out, -1, axis)
    return out


@op("nn")
def multi_hot(inputs, num_classes=None, axis=-1, dtype=None, sparse=False, **kwargs):
    if num_classes is None and "num_tokens" in kwargs:
        num_classes = kwargs.pop("num_tokens")
    if num_classes is None:
        raise ValueError("Argument `num_classes` must be specified.")
    x = _t(inputs)
    reduction_axis = 1 if x.ndim > 1 else 0
    oh = one_hot(x, num_classes, axis=axis, dtype=dtype)
    return torch.amax(oh, dim=reduction_axis)


def _loss_pair(target, output):
    target, output = _t(target), _floatize(output)
    return target, output


@op("nn")
def categorical_crossentropy(target, output, from_logits=False, axis=-1):
    target, output = _loss_pair(target, output)
    if target.shape != output.shape:
        raise ValueError(f"Arguments `target` and `output` must have the same shape. Received: target.shape={tuple(target.shape)}, output.shape={tuple(output.shape)}")
    if target.ndim < 1:
        raise ValueError(f"Arguments `target` and `output` must be at least rank 1. Received: target.shape={tuple(target.shape)}, output.shape={tuple(output.shape)}")
    target = target.to(output.dtype)
    if from_logits:
        logp = torch.log_softmax(output, dim=axis)
    else:
        output = output / torch.sum(output, dim=axis, keepdim=True)
        eps = config.epsilon()
        logp = torch.log(torch.clip(output, eps, 1.0 - eps))
    return -torch.sum(target * logp, dim=axis)


@op("nn")
def sparse_categorical_crossentropy(target, output, from_logits=False, axis=-1):
    target, output = _loss_pair(target, output)
    target = target.long()
    if target.ndim == output.ndim and target.shape[-1] == 1:
        target = target.squeeze(-1)
    if output.ndim < 1:
        raise ValueError(f"Argument `output` must be at least rank 1. Received: output.shape={tuple(output.shape)}")
    if tuple(target.shape) != tuple(output.shape[:axis % output.ndim]) + tuple(output.shape[axis % output.ndim + 1:]):
        raise ValueError(
            "Arguments `target` and `output` must have the same shape up until the last dimension: "
            f"target.shape={tuple(target.shape)}, output.shape={tuple(output.shape)}"
        )
    if axis % output.ndim != output.ndim - 1:
        output = torch.movedim(output, axis, -1)
    if from_logits:
        fused = dispatch.softmax_cross_entropy(output, target)
        if fused is not None:
            return fused
        flat = output.reshape(-1, output.shape[-1])
        loss = F.cross_entropy(flat.float() if flat.dtype in (torch.float16, torch.bfloat16) else flat, target.reshape(-1), reduction="none")
        return loss.reshape(target.shape).to(output.dtype)
    output = output / torch.sum(output, dim=-1, keepdim=True)
    eps = config.epsilon()
    logp = torch.log(torch.clip(output, eps, 1.0 - eps))
    return -torch.gather(logp, -1, target.unsqueeze(-1)).squeeze(-1)


@op("nn")
def binary_crossentropy(target, output, from_logits=False):
    target, output = _loss_pair(target, output)
    if target.shape != output.shape:
        raise ValueError(f"Arguments `target` and `output` must have the same shape. Received: target.shape={tuple(target.shape)}, output.shape={tuple(output.shape)}")
    target = target.to(output.dtype)
    if from_logits:
        return F.binary_cross_entropy_with_logits(output, target, reduction="none")
    eps = config.epsilon()
    output = torch.clip(output, eps, 1.0 - eps)
    return -(target * torch.log(output) + (1 - target) * torch.log(1 - output))


@op("nn")
def moments(x, axes, keepdims=False, synchronized=False):
    if synchronized:
        raise NotImplementedError("Argument synchronized=True is not supported by ops.moments; use BatchNormalization(synchronized=True).")
    x = _floatize(x)
    ori = x.dtype
    need_cast = ori in (torch.float16, torch.bfloat16)
    xc = x.to(torch.float32) if need_cast else x
    axes = tuple(axes) if isinstance(axes, (list, tuple)) else (axes,)
    mean = torch.mean(xc, dim=axes, keepdim=True)
    # E[x^2] - E[x]^2 (biased), as keras/src/backend/torch/nn.py:1035-1043
    var = torch.mean(xc * xc, dim=axes, keepdim=True) - mean * mean
    if not keepdims:
        mean = torch.squeeze(mean, axes)
        var = torch.squeeze(var, axes)
    if need_cast:
        lim = torch.finfo(ori).max
        mean = torch.clip(mean, -lim, lim).to(ori)
        var = torch.clip(var, -lim, lim).to(ori)
    return mean, var


@op("nn")
def batch_normalization(x, mean, variance, axis, offset=None, scale=None, epsilon=1e-3):
    x = _t(x)
    mean, variance = _t(mean), _t(variance)
    shape = [1] * x.ndim
    shape[axis] = mean.shape[0]
    inv = torch.rsqrt(variance.reshape(shape) + epsilon)
    if scale is not None:
        inv = inv * _t(scale).reshape(shape)
    res = -mean.reshape(shape) * inv
    if offset is not None:
        res = res + _t(offset).reshape(shape)
    return x * inv.to(x.dtype) + res.to(x.dtype)


@op("nn")
def normalize(x, axis=-1, order=2, epsilon=None):
    x = _floatize(x)
    if not isinstance(order, (int, float)) or order < 1:
        raise ValueError(f"Argument `order` must be an int >= 1. Received: order={order}")
    eps = epsilon if epsilon is not None else config.epsilon()
    if order == 2:
        sq = torch.sum(x * x, dim=axis, keepdim=True)
        return x * torch.rsqrt(torch.clamp(sq, min=eps * eps))
    norm = torch.linalg.vector_norm(x, ord=order, dim=axis, keepdim=True)
    return x / torch.clamp(norm, min=eps)


@op("nn")
def layer_normalization(x, gamma=None, beta=None, axis=-1, epsilon=None, **kwargs):
    rms_scaling = kwargs.pop("rms_scaling", False)
    if rms_scaling:
        return rms_normalization(x, scale=gamma, axis=axis, epsilon=epsilon)
    x = _floatize(x)
    eps = epsilon if epsilon is not None else config.epsilon()
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    axes = tuple(sorted(a % x.ndim for a in axes))
    contiguous_tail = axes == tuple(range(x.ndim - len(axes), x.ndim))
    g = _t(gamma) if gamma is not None else None
    b = _t(beta) if beta is not None else None
    if contiguous_tail:
        if len(axes) == 1:
            fused = dispatch.layer_norm(x, g, b, eps)
            if fused is not None:
                return fused
        shape = tuple(x.shape[a] for a in axes)
        ori = x.dtype
        xc = x.float() if ori in (torch.float16, torch.bfloat16) else x
        gg = g.reshape(shape).to(xc.dtype) if g is not None else None
        bb = b.reshape(shape).to(xc.dtype) if b is not None else None
        return F.layer_norm(xc, shape, gg, bb, eps).to(ori)
    ori = x.dtype
    xc = x.float() if ori in (torch.float16, torch.bfloat16) else x
    mean = torch.mean(xc, dim=axes, keepdim=True)
    var = torch.var(xc, dim=axes, keepdim=True, correction=0)
    out = (xc - mean) * torch.rsqrt(var + eps)
    bshape = [x.shape[i] if i in axes else 1 for i in range(x.ndim)]
    if g is not None:
        out = out * g.to(out.dtype).reshape(bshape)
    if b is not None:
        out = out + b.to(out.dtype).reshape(bshape)
    return out.to(ori)


@op("nn")
def rms_normalization(x, scale=None, axis=-1, epsilon=None):
    x = _floatize(x)
    eps = epsilon if epsilon is not None else config.epsilon()
    s = _t(scale) if scale is not None else None
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    axes = tuple(sorted(a % x.ndim for a in axes))
    if axes == (x.ndim - 1,):
        fused = dispatch.rms_norm(x, s, eps)
        if fused is not None:
            return fused
    ori = x.dtype
    xc = x.float() if ori in (torch.float16, torch.bfloat16) else x
    if axes == tuple(range(x.ndim - len(axes), x.ndim)):
        shape = tuple(x.shape[a] for a in axes)
        return F.rms_norm(xc, shape, s.reshape(shape).to(xc.dtype) if s is not None else None, eps).to(ori)
    ms = torch.mean(xc * xc, dim=axes, keepdim=True)
    out = xc * torch.rsqrt(ms + eps)
    if s is not None:
        out = out * s.to(out.dtype)
    return out.to(ori)


@op("nn")
def psnr(x1, x2, max_val):
    x1, x2 = _floatize(x1), _floatize(x2)
    if x1.shape != x2.shape:
        raise ValueError(f"Input shapes {tuple(x1.shape)} and {tuple(x2.shape)} must match for PSNR calculation.")
    mse = torch.mean((x1 - x2) ** 2)
    mv = torch.as_tensor(max_val, dtype=x1.dtype, device=x1.device)
    return 20 * torch.log10(mv) - 10 * torch.log10(mse)


@op("nn")
def polar(abs_, angle):
    a, ang = _floatize(abs_), _floatize(angle)
    return torch.polar(a, ang)


def _attention_mask_bias(mask, dtype):
    return torch.where(mask, torch.zeros((), dtype=dtype, device=mask.device), torch.full((), -0.7 * torch.finfo(dtype).max, dtype=dtype, device=mask.device))


@op("nn")
def dot_product_attention(query, key, value, bias=None, mask=None, scale=None, is_causal=False, flash_attention=None, attn_logits_soft_cap=None):
    """Inputs are ``[B, T, N, H]`` / ``[B, S, K, H]`` (K divides N: grouped-query)."""
    q, k, v = _t(query), _t(key), _t(value)
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError(f"`dot_product_attention` only supports 4D inputs. Received: query.shape={tuple(q.shape)}, key.shape={tuple(k.shape)}, value.shape={tuple(v.shape)}.")
    d = to_torch_dtype(result_type(q.dtype, k.dtype, v.dtype))
    q, k, v = q.to(d), k.to(d), v.to(d)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if bias is None and attn_logits_soft_cap is None and flash_attention is not False:
        fused = dispatch.flash_attention(q, k, v, mask, scale, is_causal)
        if fused is not None:
            return fused
    if flash_attention and (bias is not None or attn_logits_soft_cap is not None):
        raise ValueError("Flash attention does not support `bias` or `attn_logits_soft_cap`.")
    B, T, N, H = q.shape
    S, K = k.shape[1], k.shape[2]
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if attn_logits_soft_cap is not None:
        if K != N:
            kh = kh.repeat_interleave(N // K, dim=1)
            vh = vh.repeat_interleave(N // K, dim=1)
        logits = torch.matmul(qh, kh.transpose(-1, -2)) * scale
        logits = attn_logits_soft_cap * torch.tanh(logits / attn_logits_soft_cap)
        if bias is not None:
            logits = logits + _t(bias).to(logits.dtype)
        if is_causal:
            cm = torch.ones((T, S), dtype=torch.bool, device=q.device).tril()
            logits = logits + _attention_mask_bias(cm, logits.dtype)
        if mask is not None:
            logits = logits + _attention_mask_bias(_t(mask).to(torch.bool), logits.dtype)
        probs = torch.softmax(logits.float(), dim=-1).to(d)
        return torch.matmul(probs, vh).transpose(1, 2)
    attn_mask = None
    if mask is not None:
        attn_mask = _t(mask).to(torch.bool)
        if is_causal:
            attn_mask = attn_mask & torch.ones((T, S), dtype=torch.bool, device=q.device).tril()
            is_causal = False
    if bias is not None:
        b = _t(bias).to(d)
        attn_mask = b if attn_mask is None else b + _attention_mask_bias(attn_mask, d)
    elif attn_mask is not None:
        # a large finite negative instead of -inf: a row with every position masked attends uniformly instead of producing
        # zeros or NaN (keras/src/backend/torch/nn.py:1539)
        attn_mask = _attention_mask_bias(attn_mask, d)
    out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=attn_mask, is_causal=is_causal and attn_mask is None, scale=scale, enable_gqa=(K != N))
    return out.transpose(1, 2)


# --- folding / depth-space ----------------------------------------------------------------

@op("nn")
def unfold(x, kernel_size, dilation=1, padding=0, stride=1):
    return F.unfold(_t(x), kernel_size, dilation=dilation, padding=padding, stride=stride)


@op("nn")
def fold(x, output_size, kernel_size, dilation=1, padding=0, stride=1):
    return F.fold(_t(x), output_size, kernel_size, dilation=dilation, padding=padding, stride=stride)


@op("nn")
def depth_to_space(x, block_size, data_format=None):
    x = _t(x)
    data_format = config.standardize_data_format(data_format)
    if data_format == "channels_last":
        b, h, w, c = x.shape
        oc = c // (block_size ** 2)
        y = x.reshape(b, h, w, block_size, block_size, oc).permute(0, 1, 3, 2, 4, 5)
        return y.reshape(b, h * block_size, w * block_size, oc)
    b, c, h, w = x.shape
    oc = c // (block_size ** 2)
    y = x.reshape(b, block_size, block_size, oc, h, w).permute(0, 3, 4, 1, 5, 2)
    return y.reshape(b, oc, h * block_size, w * block_size)


@op("nn")
def space_to_depth(x, block_size, data_format=None):
    x = _t(x)
    data_format = config.standardize_data_format(data_format)
    if data_format == "channels_last":
        b, h, w, c = x.shape
        y = x.reshape(b, h // block_size, block_size, w // block_size, block_size, c).permute(0, 1, 3, 2, 4, 5)
        return y.reshape(b, h // block_size, w // block_size, c * block_size ** 2)
    b, c, h, w = x.shape
    y = x.reshape(b, c, h // block_size, block_size, w // block_size, block_size).permute(0, 3, 5, 1, 2, 4)
    return y.reshape(b, c * block_size ** 2, h // block_size, w // block_size)


# --- CTC ----------------------------------------------------------------------------------

@op("nn")
def ctc_loss(target, output, target_length, output_length, mask_index=0):
    target, output = _t(target), _floatize(output)
    target_length, output_length = _t(target_length), _t(output_length)
    logp = torch.log_softmax(output.float(), dim=-1).transpose(0, 1)
    loss = F.ctc_loss(logp, target.long(), output_length.long(), target_length.long(), blank=mask_index, reduction="none", zero_infinity=False)
    return loss.to(output.dtype)


def _ctc_greedy(inputs, sequence_lengths, merge_repeated, mask_index):
    B, T, C = inputs.shape
    if mask_index is None:
        mask_index = C - 1
    idx = torch.argmax(inputs, dim=-1).to(torch.int32)
    scores = torch.amax(inputs, dim=-1)
    seq_mask = torch.arange(T, device=inputs.device)[None, :] >= sequence_lengths[:, None]
    idx = torch.where(seq_mask, torch.full_like(idx, mask_index), idx)
    scores = torch.where(seq_mask, torch.zeros_like(scores), scores)
    if merge_repeated:
        rep = idx[:, 1:] == idx[:, :-1]
        rep = F.pad(rep, (1, 0))
        idx = torch.where(rep, torch.full_like(idx, mask_index), idx)
    invalid = idx == mask_index
    idx = torch.where(invalid, torch.full_like(idx, -1), idx)
    order = torch.argsort(invalid.to(torch.uint8), dim=-1, stable=True)
    idx = torch.take_along_dim(idx, order, dim=-1)
    return idx.unsqueeze(0), -torch.sum(scores, dim=1, keepdim=True)


def _ctc_beam(inputs, sequence_lengths, beam_width, top_paths, mask_index):
    # Host-side prefix beam search (decoding is not a training hot path).
    logp = torch.log_softmax(inputs.float(), dim=-1).cpu().numpy()
    lens = sequence_lengths.cpu().numpy()
    B, T, C = logp.shape
    if mask_index is None:
        mask_index = C - 1
    NEG = -np.inf
    all_paths = np.full((top_paths, B, T), -1, dtype=np.int32)
    all_scores = np.zeros((B, top_paths), dtype=np.float32)
    for b in range(B):
        beams = {(): (0.0, NEG)}  # prefix -> (log p_blank, log p_nonblank)
        for t in range(int(lens[b])):
            nxt = {}

            def upd(prefix, pb, pnb):
                opb, opnb = nxt.get(prefix, (NEG, NEG))
                nxt[prefix] = (np.logaddexp(opb, pb), np.logaddexp(opnb, pnb))

            for prefix, (pb, pnb) in beams.items():
                total = np.logaddexp(pb, pnb)
                for c in range(C):
                    p = logp[b, t, c]
                    if c == mask_index:
                        upd(prefix, total + p, NEG)
                    else:
                        new = prefix + (c,)
                        if prefix and prefix[-1] == c:
                            upd(new, NEG, pb + p)
                            upd(prefix, NEG, pnb + p)
                        else:
                            upd(new, NEG, total + p)
            beams = dict(sorted(nxt.items(), key=lambda kv: -np.logaddexp(*kv[1]))[:beam_width])
        ranked = sorted(beams.items(), key=lambda kv: -np.logaddexp(*kv[1]))[:top_paths]
        for i, (prefix, (pb, pnb)) in enumerate(ranked):
            all_paths[i, b, : len(prefix)] = prefix
            all_scores[b, i] = np.logaddexp(pb, pnb)
    return torch.as_tensor(all_paths, device=inputs.device), torch.as_tensor(all_scores, device=inputs.device)


@op("nn")
def ctc_decode(inputs, sequence_lengths, strategy="greedy", beam_width=100, top_paths=1, merge_repeated=True, mask_index=0):
    inputs = _floatize(inputs)
    sequence_lengths = _t(sequence_lengths).to(torch.int32)
    if strategy == "greedy":
        return _ctc_greedy(inputs, sequence_lengths, merge_repeated, mask_index)
    if strategy == "beam_search":
        return _ctc_beam(inputs, sequence_lengths, beam_width, top_paths, mask_index)
    raise ValueError(f"Invalid strategy {strategy}. Supported values are 'greedy' and 'beam_search'.")
