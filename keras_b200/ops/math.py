"""Math ops (``keras.ops`` math set): FFT, segment reductions, top-k, special functions.

Semantics follow keras/src/ops/math.py and keras/src/backend/torch/math.py.
"""

import math as _math

import torch

from keras_b200.core import config
from keras_b200.core.dtypes import result_type, to_torch_dtype
from keras_b200.ops._dispatch import op
from keras_b200.ops.numpy import _floatize, _t


def _segment(data, segment_ids, num_segments, reduce, sorted=False):
    data, ids = _t(data), _t(segment_ids).long()
    if num_segments is None:
        num_segments = int(ids.max().item()) + 1 if ids.numel() else 0
    valid = (ids >= 0) & (ids < num_segments)
    idx = torch.where(valid, ids, torch.zeros_like(ids))
    shape = (num_segments,) + tuple(data.shape[1:])
    view = idx.reshape((-1,) + (1,) * (data.ndim - 1)).expand_as(data)
    if reduce == "sum":
        src = torch.where(valid.reshape((-1,) + (1,) * (data.ndim - 1)), data, torch.zeros_like(data))
        return torch.zeros(shape, dtype=data.dtype, device=data.device).scatter_add_(0, view, src)
    if reduce == "prod":
        src = torch.where(valid.reshape((-1,) + (1,) * (data.ndim - 1)), data, torch.ones_like(data))
        return torch.ones(shape, dtype=data.dtype, device=data.device).scatter_reduce_(0, view, src, reduce="prod")
    if data.dtype.is_floating_point:
        init = -_math.inf if reduce == "amax" else _math.inf
    else:
        info = torch.iinfo(data.dtype)
        init = info.min if reduce == "amax" else info.max
    src = torch.where(valid.reshape((-1,) + (1,) * (data.ndim - 1)), data, torch.full_like(data, init))
    return torch.full(shape, init, dtype=data.dtype, device=data.device).scatter_reduce_(0, view, src, reduce=reduce)


@op()
def segment_sum(data, segment_ids, num_segments=None, sorted=False):
    return _segment(data, segment_ids, num_segments, "sum")


@op()
def segment_max(data, segment_ids, num_segments=None, sorted=False):
    return _segment(data, segment_ids, num_segments, "amax")


@op()
def segment_min(data, segment_ids, num_segments=None, sorted=False):
    return _segment(data, segment_ids, num_segments, "amin")


@op()
def segment_prod(data, segment_ids, num_segments=None, sorted=False):
    return _segment(data, segment_ids, num_segments, "prod")


@op()
def top_k(x, k, sorted=True):
    x = _t(x)
    if x.dtype == torch.bool:
        x = x.to(torch.uint8)
    values, indices = torch.sort(x, dim=-1, descending=True, stable=True)
    return values[..., :k], indices[..., :k]


@op()
def in_top_k(targets, predictions, k):
    targets = _t(targets).long()
    predictions = _t(predictions)
    target_scores = torch.take_along_dim(predictions, targets[:, None], dim=1)
    # ties count: position = number of strictly greater entries
    rank = torch.sum(predictions > target_scores, dim=1)
    return rank < k


@op()
def logsumexp(x, axis=None, keepdims=False):
    x = _floatize(x)
    if axis is None:
        r = torch.logsumexp(x.reshape(-1), dim=0)
        return r.reshape((1,) * x.ndim) if keepdims else r
    if axis == () or axis == []:
        return x
    return torch.logsumexp(x, dim=axis if isinstance(axis, int) else tuple(axis), keepdim=keepdims)


@op()
def extract_sequences(x, sequence_length, sequence_stride):
    x = _t(x)
    return x.unfold(-1, sequence_length, sequence_stride)


def _complex_in(x):
    if not isinstance(x, (tuple, list)) or len(x) != 2:
        raise ValueError(f"Input `x` should be a tuple of two tensors - real and imaginary. Received: x={x}")
    real, imag = _t(x[0]), _t(x[1])
    if real.shape != imag.shape:
        raise ValueError(f"Input `x` should be a tuple of two tensors - real and imaginary. Both the real and imaginary parts should have the same shape. Received: x[0].shape = {tuple(real.shape)}, x[1].shape = {tuple(imag.shape)}")
    if not real.dtype.is_floating_point or not imag.dtype.is_floating_point:
        raise ValueError(f"At least one tensor in input `x` is not of type float. Received: x={x}.")
    d = real.dtype
    if d in (torch.float16, torch.bfloat16):
        real, imag = real.float(), imag.float()
    return torch.complex(real, imag), d


@op()
def fft(x):
    c, d = _complex_in(x)
    r = torch.fft.fft(c)
    return r.real.to(d), r.imag.to(d)


@op()
def fft2(x):
    c, d = _complex_in(x)
    r = torch.fft.fft2(c)
    return r.real.to(d), r.imag.to(d)


@op()
def ifft2(x):
    c, d = _complex_in(x)
    r = torch.fft.ifft2(c)
    return r.real.to(d), r.imag.to(d)


@op()
def rfft(x, fft_length=None):
    x = _floatize(x)
    r = torch.fft.rfft(x.float() if x.dtype in (torch.float16, torch.bfloat16) else x, n=fft_length, dim=-1)
    return r.real.to(x.dtype), r.imag.to(x.dtype)


@op()
def irfft(x, fft_length=None):
    c, d = _complex_in(x)
    return torch.fft.irfft(c, n=fft_length, dim=-1).to(d)


def _get_window(window, length, dtype, device):
    if window is None:
        return None
    if isinstance(window, str):
        if window == "hann":
            return torch.hann_window(length, periodic=True, dtype=dtype, device=device)
        if window == "hamming":
            return torch.hamming_window(length, periodic=True, dtype=dtype, device=device)
        raise ValueError(f"If a string is passed to `window`, it must be one of `'hann'`, `'hamming'`. Received: window={window}")
    return _t(window).to(dtype)


@op()
def stft(x, sequence_length, sequence_stride, fft_length, window="hann", center=True):
    x = _floatize(x)
    if fft_length < sequence_length:
        raise ValueError(f"`fft_length` must equal or larger than `sequence_length`. Received: sequence_length={sequence_length}, fft_length={fft_length}")
    d = x.dtype
    xc = x.float() if d in (torch.float16, torch.bfloat16) else x
    win = _get_window(window, sequence_length, xc.dtype, x.device)
    if win is None:
        win = torch.ones(sequence_length, dtype=xc.dtype, device=x.device)
    lead = xc.shape[:-1]
    flat = xc.reshape(-1, xc.shape[-1])
    r = torch.stft(flat, n_fft=fft_length, hop_length=sequence_stride, win_length=sequence_length, window=win, center=center, return_complex=True, pad_mode="reflect")
    r = r.transpose(-1, -2).reshape(tuple(lead) + (r.shape[-1], r.shape[-2]))
    return r.real.to(d), r.imag.to(d)


@op()
def istft(x, sequence_length, sequence_stride, fft_length, length=None, window="hann", center=True):
    c, d = _complex_in(x)
    win = _get_window(window, sequence_length, c.real.dtype, c.device)
    if win is None:
        win = torch.ones(sequence_length, dtype=c.real.dtype, device=c.device)
    lead = c.shape[:-2]
    flat = c.reshape((-1,) + tuple(c.shape[-2:])).transpose(-1, -2)
    if center:
        r = torch.istft(flat, n_fft=fft_length, hop_length=sequence_stride, win_length=sequence_length, window=win, center=True, length=length)
    else:
        # overlap-add by hand: torch.istft needs center=True for NOLA checks at the edges
        frames = torch.fft.irfft(flat.transpose(-1, -2), n=fft_length)[..., :fft_length]
        wpad = torch.nn.functional.pad(win, ((fft_length - sequence_length) // 2, fft_length - sequence_length - (fft_length - sequence_length) // 2))
        frames = frames * wpad
        nfr = frames.shape[-2]
        out_len = fft_length + sequence_stride * (nfr - 1)
        fold = torch.nn.functional.fold(frames.transpose(-1, -2), (1, out_len), (1, fft_length), stride=(1, sequence_stride))[:, 0, 0]
        wsq = torch.nn.functional.fold((wpad ** 2)[None, :, None].expand(1, -1, nfr), (1, out_len), (1, fft_length), stride=(1, sequence_stride))[:, 0, 0]
        r = fold / torch.clamp(wsq, min=1e-11)
        if length is not None:
            r = r[..., :length] if r.shape[-1] >= length else torch.nn.functional.pad(r, (0, length - r.shape[-1]))
    return r.reshape(tuple(lead) + (r.shape[-1],)).to(d)


@op()
def rsqrt(x):
    return torch.rsqrt(_floatize(x))


@op()
def erf(x):
    return torch.erf(_floatize(x))


@op()
def erfc(x):
    return torch.erfc(_floatize(x))


@op()
def erfinv(x):
    return torch.erfinv(_floatize(x))


@op()
def gammainc(a, x):
    from keras_b200.ops.numpy import _pair_converted

    a, x = _pair_converted(a, x, floating=True)
    out = a.dtype
    if out in (torch.float16, torch.bfloat16):
        a, x = a.float(), x.float()
    return torch.special.gammainc(a, x).to(out)


@op()
def logdet(x):
    return torch.logdet(_floatize(x))


@op()
def cdist(x1, x2, p=2.0):
    x1, x2 = _floatize(x1), _floatize(x2)
    d = to_torch_dtype(result_type(x1.dtype, x2.dtype))
    return torch.cdist(x1.to(d), x2.to(d), p=p)


@op()
def view_as_complex(x):
    x = _floatize(x)
    if x.shape[-1] != 2:
        raise ValueError(f"Last dimension of input must be size 2 (real and imaginary). Received shape: {tuple(x.shape)}")
    return torch.view_as_complex(x.contiguous())


@op()
def view_as_real(x):
    x = _t(x)
    if not x.is_complex():
        return torch.stack([x, torch.zeros_like(x)], dim=-1)
    return torch.view_as_real(x)
