"""Image ops (``keras.ops.image``): pure tensor arithmetic on torch (no graphics API).

Semantics follow keras/src/ops/image.py and keras/src/backend/torch/image.py.
"""

import math

import numpy as np
import torch
import torch.nn.functional as F

from keras_b200.core import config
from keras_b200.core.dtypes import to_torch_dtype
from keras_b200.ops._dispatch import op
from keras_b200.ops.numpy import _floatize, _t


def _df(data_format):
    return config.standardize_data_format(data_format)


def _check_rank(x, name="images"):
    if x.ndim not in (3, 4):
        raise ValueError(f"Invalid {name} rank: expected rank 3 (single image) or rank 4 (batch of images). Received input with shape: {name}.shape={tuple(x.shape)}")


def _to_nchw(x, data_format):
    """→ (batched NCHW tensor, restore function)."""
    single = x.ndim == 3
    if single:
        x = x.unsqueeze(0)
    if data_format == "channels_last":
        x = x.permute(0, 3, 1, 2)

    def restore(y):
        if data_format == "channels_last":
            y = y.permute(0, 2, 3, 1)
        return y.squeeze(0) if single else y

    return x, restore


@op("image")
def rgb_to_grayscale(images, data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    ch = -1 if data_format == "channels_last" else -3
    if images.shape[ch] not in (1, 3):
        raise ValueError(f"Invalid channel size: expected 3 (RGB) or 1 (Grayscale). Received input with shape: images.shape={tuple(images.shape)}")
    if images.shape[ch] == 1:
        return images
    ori = images.dtype
    x = images.to(to_torch_dtype(config.floatx())) if not ori.is_floating_point else images
    w = torch.tensor([0.2989, 0.5870, 0.1140], dtype=x.dtype, device=x.device)
    if data_format == "channels_last":
        out = torch.tensordot(x, w, dims=([-1], [0])).unsqueeze(-1)
    else:
        out = torch.tensordot(x.movedim(-3, -1), w, dims=([-1], [0])).unsqueeze(-3)
    return out.to(ori)


@op("image")
def rgb_to_hsv(images, data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    if not images.dtype.is_floating_point:
        raise ValueError(f"Invalid images dtype: expected float dtype. Received: images.dtype={images.dtype}")
    ch = -1 if data_format == "channels_last" else -3
    r, g, b = torch.unbind(images, dim=ch)
    mx = torch.maximum(torch.maximum(r, g), b)
    mn = torch.minimum(torch.minimum(r, g), b)
    delta = mx - mn
    safe = torch.where(delta > 0, delta, torch.ones_like(delta))
    s = torch.where(mx > 0, delta / torch.where(mx > 0, mx, torch.ones_like(mx)), torch.zeros_like(mx))
    h = torch.where(mx == r, (g - b) / safe, torch.where(mx == g, 2.0 + (b - r) / safe, 4.0 + (r - g) / safe))
    h = torch.where(delta > 0, (h / 6.0) % 1.0, torch.zeros_like(h))
    return torch.stack([h, s, mx], dim=ch)


@op("image")
def hsv_to_rgb(images, data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    if not images.dtype.is_floating_point:
        raise ValueError(f"Invalid images dtype: expected float dtype. Received: images.dtype={images.dtype}")
    ch = -1 if data_format == "channels_last" else -3
    h, s, v = torch.unbind(images, dim=ch)
    dh = h * 6.0
    dr = torch.clip(torch.abs(dh - 3.0) - 1.0, 0.0, 1.0)
    dg = torch.clip(2.0 - torch.abs(dh - 2.0), 0.0, 1.0)
    db = torch.clip(2.0 - torch.abs(dh - 4.0), 0.0, 1.0)
    one_minus_s = 1.0 - s
    return torch.stack([(one_minus_s + s * dr) * v, (one_minus_s + s * dg) * v, (one_minus_s + s * db) * v], dim=ch)


_RESIZE_MODES = {"bilinear": "bilinear", "nearest": "nearest-exact", "bicubic": "bicubic", "lanczos3": None, "lanczos5": None}


def _lanczos_matrix(in_size, out_size, radius, antialias, dtype, device):
    scale = in_size / out_size
    support_scale = max(scale, 1.0) if antialias else 1.0
    centers = (torch.arange(out_size, dtype=torch.float64) + 0.5) * scale - 0.5
    src = torch.arange(in_size, dtype=torch.float64)
    d = (src[None, :] - centers[:, None]) / support_scale
    w = torch.where(torch.abs(d) < radius, torch.sinc(d) * torch.sinc(d / radius), torch.zeros_like(d))
    w = w / torch.clamp(w.sum(dim=1, keepdim=True), min=1e-12)
    return w.to(dtype=dtype, device=device)


@op("image")
def resize(images, size, interpolation="bilinear", antialias=False, crop_to_aspect_ratio=False, pad_to_aspect_ratio=False, fill_mode="constant", fill_value=0.0, data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    if interpolation not in _RESIZE_MODES:
        raise ValueError(f"Invalid value for argument `interpolation`. Expected of one {tuple(_RESIZE_MODES)}. Received: interpolation={interpolation}")
    if fill_mode != "constant":
        raise ValueError(f"Invalid value for argument `fill_mode`. Only `'constant'` is supported. Received: fill_mode={fill_mode}")
    if pad_to_aspect_ratio and crop_to_aspect_ratio:
        raise ValueError("Only one of `pad_to_aspect_ratio` & `crop_to_aspect_ratio` can be `True`.")
    if len(size) != 2:
        raise ValueError(f"Argument `size` must be a tuple of two elements (height, width). Received: size={size}")
    _check_rank(images)
    th, tw = int(size[0]), int(size[1])
    ori = images.dtype
    if images.is_cuda and data_format == "channels_last" and not (antialias or crop_to_aspect_ratio or pad_to_aspect_ratio):
        from keras_b200.kernels import dispatch

        batched = images if images.ndim == 4 else images.unsqueeze(0)
        out = dispatch.resize(batched, (th, tw), interpolation)
        if out is not None:
            return out if images.ndim == 4 else out[0]
    x, restore = _to_nchw(images, data_format)
    h, w = x.shape[-2:]
    if crop_to_aspect_ratio:
        ch = min(int(w * th / tw), h)
        cw = min(int(h * tw / th), w)
        top, left = int((h - ch) / 2), int((w - cw) / 2)
        x = x[..., top: top + ch, left: left + cw]
    elif pad_to_aspect_ratio:
        ph = max(int(w * th / tw), h)
        pw = max(int(h * tw / th), w)
        top, left = int((ph - h) / 2), int((pw - w) / 2)
        # the same margin on both sides, so an odd difference pads one line less than the target aspect asks for
        # (keras/src/backend/torch/image.py:268-321)
        x = F.pad(x, (left, left, top, top), value=fill_value)
    xf = x if x.dtype in (torch.float32, torch.float64) else x.float()
    if interpolation in ("lanczos3", "lanczos5"):
        radius = 3 if interpolation == "lanczos3" else 5
        mh = _lanczos_matrix(xf.shape[-2], th, radius, antialias, xf.dtype, xf.device)
        mw = _lanczos_matrix(xf.shape[-1], tw, radius, antialias, xf.dtype, xf.device)
        y = torch.einsum("oh,nchw,pw->ncop", mh, xf, mw)
    elif interpolation == "nearest":
        y = F.interpolate(xf, size=(th, tw), mode="nearest-exact")
    else:
        y = F.interpolate(xf, size=(th, tw), mode=interpolation, align_corners=False, antialias=antialias)
    if not ori.is_floating_point:
        if interpolation != "nearest":
            y = torch.round(y)
        if ori == torch.uint8:
            y = torch.clip(y, 0, 255)
    return restore(y.to(ori))


def _fill_mode_coords(coord, size, fill_mode):
    if fill_mode == "nearest":
        return torch.clip(coord, 0, size - 1), None
    if fill_mode == "wrap":
        return torch.remainder(coord, size), None
    if fill_mode == "mirror":
        if size == 1:
            return torch.zeros_like(coord), None
        period = 2 * (size - 1)
        c = torch.remainder(coord, period)
        return torch.where(c > size - 1, period - c, c), None
    if fill_mode == "reflect":
        period = 2 * size
        c = torch.remainder(coord, period)
        return torch.where(c > size - 1, period - 1 - c, c), None
    # constant
    valid = (coord >= 0) & (coord <= size - 1)
    return torch.clip(coord, 0, size - 1), valid


def _sample_2d(x, ys, xs, interpolation, fill_mode, fill_value):
    """x: (N,C,H,W); ys/xs: (N,Ho,Wo) float source coordinates."""
    N, C, H, W = x.shape
    if interpolation == "nearest":
        yi, xi = torch.round(ys), torch.round(xs)
        if fill_mode == "constant":
            valid = (yi >= 0) & (yi <= H - 1) & (xi >= 0) & (xi <= W - 1)
        else:
            valid = None
        yi, _ = _fill_mode_coords(yi, H, fill_mode if fill_mode != "constant" else "nearest")
        xi, _ = _fill_mode_coords(xi, W, fill_mode if fill_mode != "constant" else "nearest")
        lin = (yi.long() * W + xi.long()).reshape(N, 1, -1).expand(-1, C, -1)
        out = torch.gather(x.reshape(N, C, -1), 2, lin).reshape(N, C, *ys.shape[1:])
        if valid is not None:
            out = torch.where(valid.unsqueeze(1), out, torch.full_like(out, fill_value))
        return out
    y0, x0 = torch.floor(ys), torch.floor(xs)
    wy, wx = (ys - y0).unsqueeze(1), (xs - x0).unsqueeze(1)
    out = 0
    for dy, wyv in ((0, 1 - wy), (1, wy)):
        for dx, wxv in ((0, 1 - wx), (1, wx)):
            yy, xx = y0 + dy, x0 + dx
            if fill_mode == "constant":
                valid = (yy >= 0) & (yy <= H - 1) & (xx >= 0) & (xx <= W - 1)
                yc, xc = torch.clip(yy, 0, H - 1), torch.clip(xx, 0, W - 1)
            else:
                valid = None
                yc, _ = _fill_mode_coords(yy, H, fill_mode)
                xc, _ = _fill_mode_coords(xx, W, fill_mode)
            lin = (yc.long() * W + xc.long()).reshape(N, 1, -1).expand(-1, C, -1)
            v = torch.gather(x.reshape(N, C, -1), 2, lin).reshape(N, C, *ys.shape[1:])
            if valid is not None:
                v = torch.where(valid.unsqueeze(1), v, torch.full_like(v, fill_value))
            out = out + v * wyv * wxv
    return out


@op("image")
def affine_transform(images, transform, interpolation="bilinear", fill_mode="constant", fill_value=0, data_format=None):
    images, transform = _t(images), _t(transform)
    data_format = _df(data_format)
    if interpolation not in ("nearest", "bilinear"):
        raise ValueError(f"Invalid value for argument `interpolation`. Expected of one ('nearest', 'bilinear'). Received: interpolation={interpolation}")
    if fill_mode not in ("constant", "nearest", "wrap", "mirror", "reflect"):
        raise ValueError(f"Invalid value for argument `fill_mode`. Expected of one ('constant', 'nearest', 'wrap', 'mirror', 'reflect'). Received: fill_mode={fill_mode}")
    _check_rank(images)
    if transform.ndim not in (1, 2):
        raise ValueError(f"Invalid transform rank: expected rank 1 (single transform) or rank 2 (batch of transforms). Received input with shape: transform.shape={tuple(transform.shape)}")
    ori = images.dtype
    x, restore = _to_nchw(images, data_format)
    xf = x if x.dtype in (torch.float32, torch.float64) else x.float()
    N, C, H, W = xf.shape
    t = transform.to(xf.dtype)
    if t.ndim == 1:
        t = t.unsqueeze(0)
    t = t.expand(N, -1)
    gy, gx = torch.meshgrid(torch.arange(H, dtype=xf.dtype, device=xf.device), torch.arange(W, dtype=xf.dtype, device=xf.device), indexing="ij")
    a0, a1, a2, b0, b1, b2, c0, c1 = [t[:, i].reshape(N, 1, 1) for i in range(8)]
    k = c0 * gx + c1 * gy + 1.0
    xs = (a0 * gx + a1 * gy + a2) / k
    ys = (b0 * gx + b1 * gy + b2) / k
    y = _sample_2d(xf, ys, xs, interpolation, fill_mode, fill_value)
    if not ori.is_floating_point:
        y = torch.round(y)
    return restore(y.to(ori))


def _perspective_coeffs(start, end):
    """Solve the 8 homography coefficients mapping output (end) → input (start) points."""
    B = start.shape[0]
    rows = []
    for i in range(4):
        sx, sy = start[:, i, 0], start[:, i, 1]
        ex, ey = end[:, i, 0], end[:, i, 1]
        z, o = torch.zeros_like(sx), torch.ones_like(sx)
        rows.append(torch.stack([ex, ey, o, z, z, z, -sx * ex, -sx * ey], dim=-1))
        rows.append(torch.stack([z, z, z, ex, ey, o, -sy * ex, -sy * ey], dim=-1))
    A = torch.stack(rows, dim=1)
    rhs = torch.stack([start[:, i // 2, i % 2] for i in range(8)], dim=-1).unsqueeze(-1)
    return torch.linalg.solve(A.double(), rhs.double()).squeeze(-1).to(start.dtype)


@op("image")
def perspective_transform(images, start_points, end_points, interpolation="bilinear", fill_value=0, data_format=None):
    images = _t(images)
    sp, ep = _floatize(start_points), _floatize(end_points)
    data_format = _df(data_format)
    if interpolation not in ("nearest", "bilinear"):
        raise ValueError(f"Invalid value for argument `interpolation`. Expected of one ('nearest', 'bilinear'). Received: interpolation={interpolation}")
    _check_rank(images)
    if sp.shape[-2:] != (4, 2) or sp.ndim not in (2, 3):
        raise ValueError(f"Invalid start_points shape: expected (4,2) for a single image or (N,4,2) for a batch. Received shape: {tuple(sp.shape)}")
    if ep.shape[-2:] != (4, 2) or ep.ndim not in (2, 3):
        raise ValueError(f"Invalid end_points shape: expected (4,2) for a single image or (N,4,2) for a batch. Received shape: {tuple(ep.shape)}")
    if sp.ndim == 2:
        sp, ep = sp.unsqueeze(0), ep.unsqueeze(0)
    coeffs = _perspective_coeffs(sp.float(), ep.float())
    single = images.ndim == 3
    out = affine_transform(images, coeffs if not single else coeffs[0], interpolation=interpolation, fill_mode="constant", fill_value=fill_value, data_format=data_format)
    return out


@op("image")
def map_coordinates(inputs, coordinates, order, fill_mode="constant", fill_value=0.0):
    x = _t(inputs)
    coords = [_t(c) for c in coordinates] if isinstance(coordinates, (list, tuple)) else list(torch.unbind(_t(coordinates), 0))
    if len(coords) != x.ndim:
        raise ValueError(f"First dim of `coordinates` must be the same as the rank of `inputs`. Received inputs with shape: {tuple(x.shape)} and coordinate leading dim of {len(coords)}")
    if order not in (0, 1):
        raise ValueError(f"Invalid value for argument `order`. Expected one of [0, 1]. Received: order={order}")
    if fill_mode not in ("constant", "nearest", "wrap", "mirror", "reflect"):
        raise ValueError(f"Invalid value for argument `fill_mode`. Received: fill_mode={fill_mode}")
    ori = x.dtype
    xf = x if x.dtype.is_floating_point else x.float()
    cf = [c.to(xf.dtype) if c.dtype.is_floating_point else c.float() for c in coords]
    strides = [int(np.prod(x.shape[i + 1:])) for i in range(x.ndim)]
    flat = xf.reshape(-1)

    def fetch(idx_list):
        valid = None
        lin = 0
        for d, idx in enumerate(idx_list):
            size = x.shape[d]
            if fill_mode == "constant":
                v = (idx >= 0) & (idx <= size - 1)
                valid = v if valid is None else (valid & v)
                idx = torch.clip(idx, 0, size - 1)
            else:
                idx, _ = _fill_mode_coords(idx, size, fill_mode)
            lin = lin + idx.long() * strides[d]
        vals = flat[lin]
        if valid is not None:
            vals = torch.where(valid, vals, torch.full_like(vals, fill_value))
        return vals

    if order == 0:
        out = fetch([torch.round(c) for c in cf])
    else:
        lows = [torch.floor(c) for c in cf]
        out = 0
        for corner in range(2 ** x.ndim):
            idxs, wgt = [], 1.0
            for d in range(x.ndim):
                up = (corner >> d) & 1
                idxs.append(lows[d] + up)
                frac = cf[d] - lows[d]
                wgt = wgt * (frac if up else (1 - frac))
            out = out + fetch(idxs) * wgt
    if not ori.is_floating_point:
        out = torch.round(out)
    return out.to(ori)


@op("image")
def pad_images(images, top_padding=None, left_padding=None, bottom_padding=None, right_padding=None, target_height=None, target_width=None, data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    hax, wax = (-3, -2) if data_format == "channels_last" else (-2, -1)
    h, w = images.shape[hax], images.shape[wax]
    if sum(v is None for v in (top_padding, bottom_padding, target_height)) != 1:
        raise ValueError(f"Must specify exactly two of top_padding, bottom_padding, target_height. Received: top_padding={top_padding}, bottom_padding={bottom_padding}, target_height={target_height}")
    if sum(v is None for v in (left_padding, right_padding, target_width)) != 1:
        raise ValueError(f"Must specify exactly two of left_padding, right_padding, target_width. Received: left_padding={left_padding}, right_padding={right_padding}, target_width={target_width}")
    if top_padding is None:
        top_padding = target_height - bottom_padding - h
    if bottom_padding is None:
        bottom_padding = target_height - h - top_padding
    if left_padding is None:
        left_padding = target_width - right_padding - w
    if right_padding is None:
        right_padding = target_width - w - left_padding
    for name, v in (("top_padding", top_padding), ("left_padding", left_padding), ("bottom_padding", bottom_padding), ("right_padding", right_padding)):
        if v < 0:
            raise ValueError(f"padding must be >= 0. Received: {name}={v}")
    if data_format == "channels_last":
        padding = (0, 0, left_padding, right_padding, top_padding, bottom_padding)
    else:
        padding = (left_padding, right_padding, top_padding, bottom_padding)
    return F.pad(images, padding)


@op("image")
def crop_images(images, top_cropping=None, left_cropping=None, bottom_cropping=None, right_cropping=None, target_height=None, target_width=None, data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    hax, wax = (-3, -2) if data_format == "channels_last" else (-2, -1)
    h, w = images.shape[hax], images.shape[wax]
    if sum(v is None for v in (top_cropping, bottom_cropping, target_height)) != 1:
        raise ValueError(f"Must specify exactly two of top_cropping, bottom_cropping, target_height. Received: top_cropping={top_cropping}, bottom_cropping={bottom_cropping}, target_height={target_height}")
    if sum(v is None for v in (left_cropping, right_cropping, target_width)) != 1:
        raise ValueError(f"Must specify exactly two of left_cropping, right_cropping, target_width. Received: left_cropping={left_cropping}, right_cropping={right_cropping}, target_width={target_width}")
    if top_cropping is None:
        top_cropping = h - target_height - bottom_cropping
    if target_height is None:
        target_height = h - bottom_cropping - top_cropping
    if left_cropping is None:
        left_cropping = w - target_width - right_cropping
    if target_width is None:
        target_width = w - right_cropping - left_cropping
    if top_cropping < 0 or left_cropping < 0 or target_height < 0 or target_width < 0:
        raise ValueError("cropping amounts and target sizes must be >= 0.")
    out = images.narrow(hax % images.ndim, top_cropping, target_height)
    return out.narrow(wax % images.ndim, left_cropping, target_width)


def _patches(x, size, strides, dilation_rate, padding, data_format, nsp):
    x = _t(x)
    data_format = _df(data_format)
    size = (size,) * nsp if isinstance(size, int) else tuple(size)
    strides = size if strides is None else ((strides,) * nsp if isinstance(strides, int) else tuple(strides))
    dil = (dilation_rate,) * nsp if isinstance(dilation_rate, int) else tuple(dilation_rate)
    single = x.ndim == nsp + 1
    if single:
        x = x.unsqueeze(0)
    cin = x.shape[-1] if data_format == "channels_last" else x.shape[1]
    n = int(np.prod(size)) * cin
    from keras_b200.ops.nn import conv

    ori = x.dtype
    xf = x if x.dtype.is_floating_point else x.float()
    kernel = torch.eye(n, dtype=xf.dtype, device=x.device).reshape(size + (cin, n))
    out = conv(xf, kernel, strides=strides, padding=padding, data_format=data_format, dilation_rate=dil).to(ori)
    return out.squeeze(0) if single else out


@op("image")
def extract_patches(images, size, strides=None, dilation_rate=1, padding="valid", data_format=None):
    return _patches(images, size, strides, dilation_rate, padding, data_format, 2)


@op("image")
def extract_patches_3d(volumes, size, strides=None, dilation_rate=1, padding="valid", data_format=None):
    return _patches(volumes, size, strides, dilation_rate, padding, data_format, 3)


@op("image")
def reconstruct_patches(patches, size, strides=None, data_format=None):
    """Inverse of ``extract_patches`` for non-dilated patches (overlaps are averaged)."""
    p = _t(patches)
    data_format = _df(data_format)
    single = p.ndim == 3
    if single:
        p = p.unsqueeze(0)
    if data_format == "channels_first":
        p = p.permute(0, 2, 3, 1)
    size = (size, size) if isinstance(size, int) else tuple(size)
    B, gh, gw, n = p.shape
    ph, pw = size
    c = n // (ph * pw)
    strides = size if strides is None else ((strides, strides) if isinstance(strides, int) else tuple(strides))
    H, W = (gh - 1) * strides[0] + ph, (gw - 1) * strides[1] + pw
    cols = p.reshape(B, gh * gw, ph, pw, c).permute(0, 4, 2, 3, 1).reshape(B, c * ph * pw, gh * gw)
    colsf = cols.float()
    out = F.fold(colsf, (H, W), (ph, pw), stride=strides)
    cnt = F.fold(torch.ones_like(colsf), (H, W), (ph, pw), stride=strides)
    out = (out / cnt).to(p.dtype)
    if data_format == "channels_last":
        out = out.permute(0, 2, 3, 1)
    return out.squeeze(0) if single else out


def _gauss_kernel1d(size, sigma, dtype, device):
    ax = torch.arange(size, dtype=dtype, device=device) - (size - 1) / 2.0
    k = torch.exp(-(ax ** 2) / (2.0 * sigma ** 2))
    return k / k.sum()


@op("image")
def gaussian_blur(images, kernel_size=(3, 3), sigma=(1.0, 1.0), data_format=None):
    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    ori = images.dtype
    x, restore = _to_nchw(images, data_format)
    xf = x if x.dtype in (torch.float32, torch.float64) else x.float()
    C = xf.shape[1]
    ks = (kernel_size, kernel_size) if isinstance(kernel_size, int) else tuple(kernel_size)
    sg = (sigma, sigma) if isinstance(sigma, (int, float)) else tuple(float(s) for s in (sigma.tolist() if isinstance(sigma, torch.Tensor) else sigma))
    # entry 0 of `kernel_size` / `sigma` runs along the width, entry 1 along the height
    # (keras/src/backend/torch/image.py:859-862 builds outer(g(size[1], sigma[1]), g(size[0], sigma[0])))
    ky = _gauss_kernel1d(ks[1], sg[1], xf.dtype, xf.device)
    kx = _gauss_kernel1d(ks[0], sg[0], xf.dtype, xf.device)
    k2 = torch.outer(ky, kx).expand(C, 1, -1, -1)
    pads = ((ks[0] - 1) // 2, ks[0] - 1 - (ks[0] - 1) // 2, (ks[1] - 1) // 2, ks[1] - 1 - (ks[1] - 1) // 2)
    y = F.conv2d(F.pad(xf, pads), k2, groups=C)
    return restore(y.to(ori))


@op("image")
def elastic_transform(images, alpha=20.0, sigma=5.0, interpolation="bilinear", fill_mode="reflect", fill_value=0.0, seed=None, data_format=None):
    from keras_b200.random import random as _random

    images = _t(images)
    data_format = _df(data_format)
    _check_rank(images)
    ori = images.dtype
    x, restore = _to_nchw(images, data_format)
    xf = x if x.dtype in (torch.float32, torch.float64) else x.float()
    N, C, H, W = xf.shape
    from keras_b200.random.seed_generator import draw_seed

    dx = _random.normal((N, H, W), mean=0.0, stddev=1.0, dtype="float32", seed=seed).to(xf.device)
    dy = _random.normal((N, H, W), mean=0.0, stddev=1.0, dtype="float32", seed=(seed if seed is None else _bump(seed))).to(xf.device)
    ksize = max(int(6 * sigma) | 1, 3)
    blur = lambda d: gaussian_blur(d.unsqueeze(-1), (ksize, ksize), (sigma, sigma), data_format="channels_last").squeeze(-1)
    dx, dy = blur(dx) * alpha, blur(dy) * alpha
    gy, gx = torch.meshgrid(torch.arange(H, dtype=xf.dtype, device=xf.device), torch.arange(W, dtype=xf.dtype, device=xf.device), indexing="ij")
    y = _sample_2d(xf, gy + dy.to(xf.dtype), gx + dx.to(xf.dtype), interpolation, fill_mode, fill_value)
    return restore(y.to(ori))


def _bump(seed):
    return seed + 1 if isinstance(seed, int) else seed


@op("image")
def scale_and_translate(images, output_shape, scale, translation, spatial_dims, method, antialias=True):
    images = _t(images)
    scale, translation = _floatize(scale), _floatize(translation)
    out = images if images.dtype.is_floating_point else images.float()
    radius = {"linear": 1.0, "bilinear": 1.0, "trilinear": 1.0, "cubic": 2.0, "bicubic": 2.0, "tricubic": 2.0, "lanczos3": 3.0, "lanczos5": 5.0}
    if method not in radius:
        raise ValueError(f"Invalid value for argument `method`. Received: method={method}")

    def kernel(d):
        if method in ("linear", "bilinear", "trilinear"):
            return torch.clamp(1 - torch.abs(d), min=0)
        if method in ("cubic", "bicubic", "tricubic"):
            a = torch.abs(d)
            return torch.where(a <= 1, (1.5 * a - 2.5) * a * a + 1, torch.where(a < 2, ((-0.5 * a + 2.5) * a - 4) * a + 2, torch.zeros_like(a)))
        r = radius[method]
        return torch.where(torch.abs(d) < r, torch.sinc(d) * torch.sinc(d / r), torch.zeros_like(d))

    for i, dim in enumerate(spatial_dims):
        in_size, out_size = out.shape[dim], int(output_shape[dim])
        s, t = scale[i].double(), translation[i].double()
        inv = 1.0 / s
        kscale = torch.clamp(inv, min=1.0) if antialias else torch.ones_like(inv)
        sample = (torch.arange(out_size, dtype=torch.float64, device=out.device) + 0.5) * inv - t * inv - 0.5
        src = torch.arange(in_size, dtype=torch.float64, device=out.device)
        w = kernel((src[None, :] - sample[:, None]) / kscale)
        tot = w.sum(dim=1, keepdim=True)
        w = torch.where(torch.abs(tot) > 1000 * torch.finfo(torch.float32).eps, w / torch.where(tot != 0, tot, torch.ones_like(tot)), torch.zeros_like(w))
        inside = (sample >= -0.5) & (sample <= in_size - 0.5)
        w = torch.where(inside[:, None], w, torch.zeros_like(w)).to(out.dtype)
        out = torch.movedim(torch.tensordot(out, w, dims=([dim], [1])), -1, dim)
    return out.to(images.dtype) if images.dtype.is_floating_point else out


@op("image")
def sobel_edges(images, data_format=None):
    images = _floatize(images)
    data_format = _df(data_format)
    _check_rank(images)
    x, restore = _to_nchw(images, data_format)
    C = x.shape[1]
    kh = torch.tensor([[-1, -2, -1], [0, 0, 0], [1, 2, 1]], dtype=x.dtype, device=x.device)
    kw = kh.t()
    # zero padding at the border, as keras/src/backend/torch/image.py:1196-1236
    gy = F.conv2d(x, kh.expand(C, 1, 3, 3), padding=1, groups=C)
    gx = F.conv2d(x, kw.expand(C, 1, 3, 3), padding=1, groups=C)
    out = torch.stack([restore(gy), restore(gx)], dim=-1)
    return out


@op("image")
def ssim(img1, img2, max_val=1.0, filter_size=11, filter_sigma=1.5, k1=0.01, k2=0.03, data_format=None):
    a, b = _floatize(img1), _floatize(img2)
    data_format = _df(data_format)
    xa, _ = _to_nchw(a, data_format)
    xb, _ = _to_nchw(b, data_format)
    C = xa.shape[1]
    k = _gauss_kernel1d(filter_size, filter_sigma, xa.dtype, xa.device)
    k2d = torch.outer(k, k).expand(C, 1, -1, -1)
    f = lambda t: F.conv2d(t, k2d, groups=C)
    mu_a, mu_b = f(xa), f(xb)
    saa, sbb, sab = f(xa * xa) - mu_a ** 2, f(xb * xb) - mu_b ** 2, f(xa * xb) - mu_a * mu_b
    c1, c2 = (k1 * max_val) ** 2, (k2 * max_val) ** 2
    ssim_map = ((2 * mu_a * mu_b + c1) * (2 * sab + c2)) / ((mu_a ** 2 + mu_b ** 2 + c1) * (saa + sbb + c2))
    out = ssim_map.mean(dim=(1, 2, 3))
    return out[0] if a.ndim == 3 else out
