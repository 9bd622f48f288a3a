"""Weight-only post-training quantisation with calibration data: the numerical cores of GPTQ and AWQ.

Both methods turn a float kernel ``W[in, out]`` into unsigned integer codes with an affine grid per output row and per
group of input features, ``W[i, o] ~ scale[o, g(i)] * (code[o, i] - zero[o, g(i)])``:

* GPTQ (``gptq_solve``) quantises input features one at a time and pushes the rounding error of each onto the features
  not yet quantised, weighted by the inverse of the layer's input second-moment matrix ``H = 2/N * X^T X``
  (``HessianEstimate``); arXiv 2210.17323.
* AWQ (``awq_solve``) first rescales input features by ``s[i] = a[i]^r / w[i]^(1-r)`` (``a``: mean activation magnitude,
  ``w``: normalised weight magnitude, ``r`` picked on a grid by weighted reconstruction error), optionally clips each
  group's range on a grid against a sample of activations, then rounds to nearest; arXiv 2306.00978.

Everything here works on ``[out, in]`` matrices (the kernel transposed) in float32 torch tensors, in place where the
algorithm allows, on whatever device the kernel lives.  The numerics (grid search order, tie breaking, the Cholesky
formulation, rounding) follow keras/src/quantizers/gptq.py:28-260, awq.py:15-330 and quantizers.py:1410-1660, so codes
and scales agree with the reference's to rounding.
"""

import torch

MAX_CLIP_SAMPLE_ROWS = 512


# ----------------------------------------------------------------------------------------- affine grids
def affine_parameters(w, bits, symmetric=False, per_channel=True, group_size=-1):
    """Scale, zero point and top code of the unsigned ``bits``-wide grid that covers ``w[out, in]``.

    ``per_channel`` with ``group_size > 0``: one grid per row and group of ``group_size`` columns (``[out, n_groups]``);
    ``per_channel`` alone: one per row (``[out, 1]``); otherwise one for the whole matrix, repeated per row."""
    w = w.float()
    out_features, in_features = w.shape
    n_groups = -(-in_features // group_size) if (per_channel and group_size > 0) else 1
    if n_groups > 1:
        pad = n_groups * group_size - in_features
        grouped = torch.nn.functional.pad(w, (0, pad)) if pad else w
        grouped = grouped.reshape(out_features, n_groups, group_size)
        lo, hi = grouped.amin(dim=2), grouped.amax(dim=2)
    elif per_channel:
        lo, hi = w.amin(dim=1), w.amax(dim=1)
    else:
        lo, hi = w.amin().reshape(1), w.amax().reshape(1)
    if symmetric:
        bound = torch.maximum(lo.abs(), hi)
        lo = torch.where(lo < 0, -bound, lo)
        hi = bound
    flat = lo == hi
    lo = torch.where(flat, lo - 1, lo)
    hi = torch.where(flat, hi + 1, hi)
    maxq = float(2 ** bits - 1)
    scale = (hi - lo) / maxq
    scale = torch.where(scale <= 0, torch.full_like(scale, 1e-8), scale)
    zero = torch.full_like(scale, (maxq + 1) / 2) if symmetric else torch.round(-lo / scale)
    if n_groups == 1:
        scale, zero = scale.reshape(-1, 1), zero.reshape(-1, 1)
        if not per_channel:
            scale, zero = scale.expand(out_features, 1).contiguous(), zero.expand(out_features, 1).contiguous()
    return scale, zero.to(torch.uint8), maxq


def to_codes(w, scale, zero, maxq):
    safe = torch.where(scale == 0, torch.full_like(scale, 1e-8), scale)
    return torch.clamp(torch.round(w / safe + zero.to(scale.dtype)), 0, maxq)


def from_codes(codes, scale, zero):
    return scale * (codes - zero.to(scale.dtype))


def spread(parameter, g_idx):
    """``[out, n_groups]`` -> ``[out, in]``: every input feature gets the parameter of its group."""
    return parameter.index_select(1, g_idx.to(torch.int64))


def dequantize(codes, scale, zero, g_idx):
    """Codes ``[out, in]`` back to floats with per-group parameters."""
    return (codes.to(scale.dtype) - spread(zero, g_idx).to(scale.dtype)) * spread(scale, g_idx)


def round_to_nearest(w, bits, group_size):
    """Plain grouped rounding (no calibration): ``(codes, scale, zero, g_idx)``."""
    in_features = w.shape[1]
    scale, zero, maxq = affine_parameters(w, bits, per_channel=True, group_size=group_size)
    g_idx = torch.zeros(in_features, dtype=torch.int32, device=w.device) if group_size == -1 else (
        torch.arange(in_features, device=w.device) // group_size).to(torch.int32)
    return to_codes(w, spread(scale, g_idx), spread(zero, g_idx), maxq), scale, zero, g_idx


# ------------------------------------------------------------------------------------------------ GPTQ
class HessianEstimate:
    """Running estimate of ``2/N * X^T X`` over every calibration row seen so far."""

    def __init__(self, features, device=None):
        self.features = features
        self.matrix = torch.zeros((features, features), dtype=torch.float32, device=device)
        self.rows_seen = 0

    def add(self, x):
        if x is None:
            raise ValueError("Input tensor cannot be None.")
        if x.ndim < 2:
            raise ValueError(f"Input tensor must have rank >= 2 (got rank {x.ndim}).")
        if x.numel() == 0:
            raise ValueError("Input tensor cannot be empty.")
        x = x.reshape(-1, x.shape[-1]).float()
        if x.shape[1] != self.features:
            raise ValueError(f"Hessian dimensions ({self.features}) do not match input features ({x.shape[1]}).")
        if x.device != self.matrix.device:
            self.matrix = self.matrix.to(x.device)
        total = self.rows_seen + x.shape[0]
        gram = x.T @ x
        gram = (gram + gram.T) / 2.0
        if self.rows_seen:
            self.matrix.mul_(self.rows_seen / total)
        self.matrix.add_(gram, alpha=2.0 / total)
        self.rows_seen = total

    def damped(self, damping):
        """The matrix made safely invertible: dead features get a unit diagonal, then ``damping * mean(diag)`` is added."""
        h = self.matrix.clone()
        diag = torch.diagonal(h).clone()
        dead = diag == 0
        diag[dead] = 1.0
        torch.diagonal(h).copy_(diag + damping * diag.mean())
        return h


def _descending_stable(metric):
    n = metric.shape[0]
    jitter = torch.arange(n, device=metric.device, dtype=torch.float32) / n * 1e-12
    return torch.argsort(-(metric + jitter), stable=True)


def gptq_solve(w_t, hessian, *, bits=4, group_size=-1, symmetric=False, per_channel=True, activation_order=False, block=128):
    """GPTQ on ``w_t[out, in]`` with the (damped) Hessian ``[in, in]``.  Returns ``(codes int32 [out, in], scale
    [out, n_groups], zero uint8 [out, n_groups], g_idx int32 [in])``."""
    w = w_t.detach().float().clone()
    h = hessian.detach().float()
    in_features = w.shape[1]
    order = None
    if activation_order:
        metric = torch.diagonal(h).clone()
        metric[~torch.isfinite(metric)] = 0
        order = _descending_stable(metric)
        w = w[:, order]
        h = h[order][:, order]
    # upper Cholesky factor of H^-1: row j holds how an error in feature j spreads to the features after it
    spreader = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(h)), upper=True)
    codes = torch.zeros(w.shape, dtype=torch.int32, device=w.device)
    group = in_features if group_size == -1 else group_size
    grids, grid_start, grid = [], None, None
    for b0 in range(0, in_features, block):
        b1 = min(b0 + block, in_features)
        work = w[:, b0:b1].clone()          # in-block corrections happen on this copy; group ranges come from `w`
        errors = torch.zeros_like(work)
        local = spreader[b0:b1, b0:b1]
        for j in range(b1 - b0):
            feature = b0 + j
            start = (feature // group) * group
            if start != grid_start:
                grid = affine_parameters(w[:, start:min(start + group, in_features)] if group != in_features else w, bits, symmetric=symmetric,
                                         per_channel=per_channel, group_size=group_size)
                grids.append(grid)
                grid_start = start
            scale, zero, maxq = grid
            column = work[:, j]
            q = to_codes(column.unsqueeze(1), scale, zero, maxq)
            codes[:, feature] = q[:, 0].to(torch.int32)
            e = (column - from_codes(q, scale, zero)[:, 0]) / local[j, j]
            errors[:, j] = e
            if j + 1 < b1 - b0:
                work[:, j + 1:].addr_(e, local[j, j + 1:], alpha=-1.0)
        if b1 < in_features:
            w[:, b1:].sub_(errors @ spreader[b0:b1, b1:])
    g_idx = (torch.arange(in_features, device=w.device) // group).to(torch.int32)
    if order is not None:
        back = torch.argsort(order)
        g_idx = g_idx[back]
        codes = codes[:, back]
    scale = torch.cat([g[0] for g in grids], dim=1)
    zero = torch.cat([g[1] for g in grids], dim=1)
    return codes, scale, zero, g_idx


# ------------------------------------------------------------------------------------------------- AWQ
class ActivationProfile:
    """Running mean of ``|x|`` per input feature, plus the first rows seen (for the clipping search)."""

    def __init__(self, features, keep_sample=False, device=None):
        self.features = features
        self.magnitudes = torch.zeros(features, dtype=torch.float32, device=device)
        self.rows_seen = 0
        self.keep_sample = keep_sample
        self._sample, self._sample_rows = [], 0

    def add(self, x):
        if x is None:
            raise ValueError("Input tensor cannot be None.")
        if x.numel() == 0:
            raise ValueError("Input tensor cannot be empty.")
        x = x.reshape(-1, x.shape[-1]).float()
        if x.device != self.magnitudes.device:
            self.magnitudes = self.magnitudes.to(x.device)
        n = x.shape[0]
        total = self.rows_seen + n
        self.magnitudes.add_((x.abs().mean(dim=0) - self.magnitudes) * (n / total))
        self.rows_seen = total
        if self.keep_sample and self._sample_rows < MAX_CLIP_SAMPLE_ROWS:
            take = min(n, MAX_CLIP_SAMPLE_ROWS - self._sample_rows)
            self._sample.append(x[:take])
            self._sample_rows += take

    @property
    def sample(self):
        return torch.cat(self._sample, dim=0) if self._sample else None


def _fake_quantize(w, group_size):
    """Round ``w[out, in]`` to the 4-bit grouped grid and back."""
    codes, scale, zero, g_idx = round_to_nearest(w, 4, group_size)
    if group_size == -1:
        return from_codes(codes, scale, zero)
    return dequantize(codes, scale, zero, g_idx)


def _weight_salience(w, group_size):
    """Mean over output rows of ``|w|`` normalised by its group's (or row's) largest magnitude: ``[in]``."""
    out_features, in_features = w.shape
    mag = w.float().abs()
    if group_size and group_size > 0 and in_features % group_size == 0:
        grouped = mag.reshape(out_features, in_features // group_size, group_size)
        mag = (grouped / (grouped.amax(dim=2, keepdim=True) + 1e-6)).reshape(out_features, in_features)
    else:
        mag = mag / (mag.amax(dim=1, keepdim=True) + 1e-6)
    return mag.mean(dim=0)


def awq_channel_scales(w_t, activation_magnitudes, *, num_grid_points=20, group_size=-1):
    """Per-input-feature scales that minimise the activation-weighted error of 4-bit rounding, searched over the mixing
    exponent ``r = 0, 1/n, ..., 1``."""
    w = w_t.float()
    a = activation_magnitudes.float()
    a = torch.where(a < 1e-8, torch.ones_like(a), a)
    s = _weight_salience(w, group_size)
    s = torch.where(s < 1e-8, torch.ones_like(s), s)
    best, best_loss = torch.ones_like(a), None
    for i in range(num_grid_points + 1):
        r = i / num_grid_points
        scales = torch.clamp(a.pow(r) / s.pow(1.0 - r), min=1e-4)
        scales = scales / torch.clamp(torch.sqrt(scales.max() * scales.min()), min=1e-8)
        restored = _fake_quantize(w * scales, group_size) / scales
        loss = float((((w - restored) ** 2) * (a ** 2)).mean())
        if best_loss is None or loss < best_loss:
            best, best_loss = scales, loss
    return best


def awq_clip_ranges(w_scaled, activation_sample, scales, *, group_size=-1, n_grid=20, max_shrink=0.5, rows_per_pass=64):
    """Per (output row, group) the magnitude bound, among ``max * (1 - k * max_shrink / n_grid)``, whose clipped-and-rounded
    weights reproduce the group's partial outputs on the sample best.  Returns ``(bounds [out, n_groups, 1], group width,
    n_groups)``."""
    out_features, in_features = w_scaled.shape
    x = activation_sample.float().reshape(-1, in_features) / scales.float()
    width = group_size if (group_size and group_size > 0 and in_features % group_size == 0) else in_features
    n_groups = in_features // width
    xg = x.reshape(-1, n_groups, width)
    wg = w_scaled.float().reshape(out_features, n_groups, width)
    full = wg.abs().amax(dim=-1, keepdim=True)
    steps = max(1, int(n_grid))
    fq_group = width if n_groups > 1 else -1
    parts = []
    for start in range(0, out_features, rows_per_pass):
        w = wg[start:start + rows_per_pass]
        rows = w.shape[0]
        top = full[start:start + rows_per_pass]
        wanted = torch.einsum("rng,ong->orn", xg, w)
        best_bound, best_err = top, None
        for k in range(steps):
            bound = top * (1.0 - k * (max_shrink / n_grid))
            clipped = torch.maximum(torch.minimum(w, bound), -bound)
            rounded = _fake_quantize(clipped.reshape(rows, in_features), fq_group).reshape(rows, n_groups, width)
            err = ((torch.einsum("rng,ong->orn", xg, rounded) - wanted) ** 2).mean(dim=1).unsqueeze(-1)
            if best_err is None:
                best_err, best_bound = err, bound
            else:
                better = err < best_err
                best_err = torch.where(better, err, best_err)
                best_bound = torch.where(better, bound, best_bound)
        parts.append(best_bound)
    return torch.cat(parts, dim=0), width, n_groups


def awq_solve(w_t, activation_magnitudes, *, num_grid_points=20, group_size=-1, activation_sample=None, clip_n_grid=20, clip_max_shrink=0.5):
    """AWQ on ``w_t[out, in]``.  Returns ``(codes [out, in], scale, zero uint8, awq_scales [in], g_idx int32 [in])``; the
    layer computes ``x @ (dequantised / awq_scales)``.  ``activation_sample`` switches the clipping search on."""
    w = w_t.detach().float()
    out_features, in_features = w.shape
    scales = awq_channel_scales(w, activation_magnitudes, num_grid_points=num_grid_points, group_size=group_size)
    scaled = w * scales
    if activation_sample is not None:
        bounds, width, n_groups = awq_clip_ranges(scaled, activation_sample, scales, group_size=group_size, n_grid=clip_n_grid, max_shrink=clip_max_shrink)
        grouped = scaled.reshape(out_features, n_groups, width)
        scaled = torch.maximum(torch.minimum(grouped, bounds), -bounds).reshape(out_features, in_features)
    codes, scale, zero, g_idx = round_to_nearest(scaled, 4, group_size)
    return codes, scale, zero, scales, g_idx
