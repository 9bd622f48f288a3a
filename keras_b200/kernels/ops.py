"""Python side of the sm_100a kernels: ``ctypes`` launch wrappers and autograd functions."""

import ctypes

import torch

from keras_b200.kernels import loader

_vp = ctypes.c_void_p
_ll = ctypes.c_longlong
_i = ctypes.c_int
_f = ctypes.c_float
_d = ctypes.c_double


def _p(t):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


def _dt(t):
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError(f"unsupported dtype {t.dtype}")


import threading

_TL = threading.local()


def _stream():
    """Current stream handle; also binds this thread to the current device on first use."""
    dev = torch.cuda.current_device()
    if getattr(_TL, "dev", None) != dev:
        loader.get().kb200_bind_device(_i(dev))
        _TL.dev = dev
    return _vp(torch.cuda.current_stream().cuda_stream)


def _lib():
    lib = loader.get()
    if lib is None:
        raise RuntimeError("The sm_100a kernel library needs a CUDA device.")
    return lib


_LAUNCHES = [0]


def launch_count():
    """Number of kernel-launcher calls made by this process so far."""
    return _LAUNCHES[0]


def check_stream_kernels():
    """Raise if a bounded wait ran out inside a bulk-copy ring kernel (BatchNorm streaming passes) since the last check.
    Synchronises the device."""
    lib = loader.get()
    if lib is None or not hasattr(lib, "kb200_bn_stream_status"):
        return
    lib.kb200_bn_stream_status.restype = ctypes.c_int
    code = lib.kb200_bn_stream_status()
    if code > 0:
        raise RuntimeError(f"a BatchNorm streaming kernel gave up waiting on its copy pipeline (wait {code}); results of that pass are incomplete")


def add_launches(n):
    """Account for launcher calls that ran without passing through Python (a replayed CUDA graph of them)."""
    _LAUNCHES[0] += n


def _check(code, what):
    _LAUNCHES[0] += 1
    if code != 0:
        msg = b""
        try:
            fn = _lib().kb200_last_error
            fn.restype = ctypes.c_char_p
            msg = fn() or b""
        except Exception:
            pass
        raise RuntimeError(f"{what} failed with code {code}: {msg.decode(errors='ignore')}")


# ------------------------------------------------------------------------------ max pooling
class FusedMaxPool2D(torch.autograd.Function):
    """Channels-last 2-D max pooling with the padding folded in (``pad_mode`` 1: zeros, 0: ignored)."""

    @staticmethod
    def forward(ctx, x, pool, strides, pads, out_hw, pad_mode):
        lib = _lib()
        x = x.contiguous()
        N, H, W, C = x.shape
        OH, OW = out_hw
        y = torch.empty((N, OH, OW, C), dtype=x.dtype, device=x.device)
        idx = torch.empty((N, OH, OW, C), dtype=torch.uint8, device=x.device)
        _check(lib.kb200_maxpool2d_fwd(_p(x), _p(y), _p(idx), _i(N), _i(H), _i(W), _i(C), _i(OH), _i(OW), _i(pool[0]), _i(pool[1]), _i(strides[0]),
                                       _i(strides[1]), _i(pads[0]), _i(pads[1]), _i(pad_mode), _i(_dt(x)), _stream()), "maxpool_fwd")
        ctx.save_for_backward(idx)
        ctx.geom = (N, H, W, C, OH, OW, pool, strides, pads, _dt(x))
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        (idx,) = ctx.saved_tensors
        N, H, W, C, OH, OW, pool, strides, pads, dt = ctx.geom
        dy = dy.contiguous()
        dx = torch.empty((N, H, W, C), dtype=dy.dtype, device=dy.device)
        _check(lib.kb200_maxpool2d_bwd(_p(dy), _p(idx), _p(dx), _i(N), _i(H), _i(W), _i(C), _i(OH), _i(OW), _i(pool[0]), _i(pool[1]), _i(strides[0]),
                                       _i(strides[1]), _i(pads[0]), _i(pads[1]), _i(dt), _stream()), "maxpool_bwd")
        return dx, None, None, None, None, None


class FusedAvgPool2D(torch.autograd.Function):
    """Channels-last 2-D average pooling; window elements outside the image do not count (as ``padding="same"`` means in
    keras/src/backend/torch/nn.py:449-533)."""

    @staticmethod
    def forward(ctx, x, pool, strides, pads, out_hw):
        lib = _lib()
        x = x.contiguous()
        N, H, W, C = x.shape
        OH, OW = out_hw
        y = torch.empty((N, OH, OW, C), dtype=x.dtype, device=x.device)
        _check(lib.kb200_avgpool2d_fwd(_p(x), _p(y), _i(N), _i(H), _i(W), _i(C), _i(OH), _i(OW), _i(pool[0]), _i(pool[1]), _i(strides[0]), _i(strides[1]),
                                       _i(pads[0]), _i(pads[1]), _i(_dt(x)), _stream()), "avgpool_fwd")
        ctx.geom = (N, H, W, C, OH, OW, pool, strides, pads)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        N, H, W, C, OH, OW, pool, strides, pads = ctx.geom
        dy = dy.contiguous()
        dx = torch.empty((N, H, W, C), dtype=dy.dtype, device=dy.device)
        _check(lib.kb200_avgpool2d_bwd(_p(dy), _p(dx), _i(N), _i(H), _i(W), _i(C), _i(OH), _i(OW), _i(pool[0]), _i(pool[1]), _i(strides[0]), _i(strides[1]),
                                       _i(pads[0]), _i(pads[1]), _i(_dt(dy)), _stream()), "avgpool_bwd")
        return dx, None, None, None, None


class FusedGlobalAvgPool(torch.autograd.Function):
    """Mean over the pixel axes of a channels-last tensor: ``[N, *spatial, C] -> [N, C]``."""

    @staticmethod
    def forward(ctx, x):
        lib = _lib()
        x = x.contiguous()
        N, C = x.shape[0], x.shape[-1]
        P = x.numel() // (N * C)
        y = torch.empty((N, C), dtype=x.dtype, device=x.device)
        _check(lib.kb200_global_avgpool_fwd(_p(x), _p(y), _i(N), _i(P), _i(C), _i(_dt(x)), _stream()), "global_avgpool_fwd")
        ctx.shape = tuple(x.shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        shape = ctx.shape
        N, C = shape[0], shape[-1]
        P = 1
        for d in shape[1:-1]:
            P *= d
        dy = dy.contiguous()
        dx = torch.empty(shape, dtype=dy.dtype, device=dy.device)
        _check(lib.kb200_global_avgpool_bwd(_p(dy), _p(dx), _i(N), _i(P), _i(C), _i(_dt(dy)), _stream()), "global_avgpool_bwd")
        return dx


# ------------------------------------------------------------------------------ softmax
class FusedSoftmax(torch.autograd.Function):
    """softmax / log-softmax over the last axis of a contiguous tensor; ``mask`` (bool, same shape, or ``None``) marks the
    elements that take part: the others get ``masked_add`` added before the exponential."""

    @staticmethod
    def forward(ctx, x, mask, masked_add, log_mode):
        lib = _lib()
        x = x.contiguous()
        C = x.shape[-1]
        rows = x.numel() // C
        y = torch.empty_like(x)
        m8 = None
        if mask is not None:
            m8 = mask.expand(x.shape).contiguous().view(torch.uint8) if mask.dtype == torch.bool else (mask != 0).expand(x.shape).contiguous().view(torch.uint8)
        _check(lib.kb200_softmax_fwd(_p(x), _p(m8), _p(y), _ll(rows), _i(C), _f(masked_add), _i(1 if log_mode else 0), _i(_dt(x)), _stream()), "softmax_fwd")
        ctx.save_for_backward(y)
        ctx.log_mode = log_mode
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        (y,) = ctx.saved_tensors
        C = y.shape[-1]
        rows = y.numel() // C
        dy = dy.to(y.dtype).contiguous()
        dx = torch.empty_like(y)
        _check(lib.kb200_softmax_bwd(_p(y), _p(dy), _p(dx), _ll(rows), _i(C), _i(1 if ctx.log_mode else 0), _i(_dt(y)), _stream()), "softmax_bwd")
        return dx, None, None, None


# ------------------------------------------------------------------------------ embedding
class FusedEmbedding(torch.autograd.Function):
    """``table[ids]`` in ``out_dtype``.  ``table`` is the fp32 parameter or its bf16 shadow read; ``target`` is the fp32
    parameter when its gradient lives in persistent storage: the scatter-add then goes straight into it."""

    @staticmethod
    def forward(ctx, table, ids, out_dtype, target):
        lib = _lib()
        V, D = table.shape
        ids64 = ids.reshape(-1).to(torch.int64).contiguous()
        n = ids64.numel()
        src = table.detach()
        if not src.is_contiguous():
            src = src.contiguous()
        out = torch.empty((n, D), dtype=out_dtype, device=table.device)
        _check(lib.kb200_embedding_fwd(_p(src), _p(ids64), _p(out), _ll(n), _i(D), _ll(V), _i(_dt(src)), _i(_dt(out)), _stream()), "embedding_fwd")
        ctx.save_for_backward(ids64)
        ctx.table_shape, ctx.table_dtype, ctx.target = (V, D), table.dtype, target
        ctx.set_materialize_grads(False)
        return out.reshape(tuple(ids.shape) + (D,))

    @staticmethod
    def backward(ctx, dout):
        if dout is None:
            return None, None, None, None
        from keras_b200.kernels import shadow

        lib = _lib()
        (ids64,) = ctx.saved_tensors
        V, D = ctx.table_shape
        if dout.dtype not in (torch.float32, torch.bfloat16):
            dout = dout.float()
        dout = dout.reshape(-1, D).contiguous()
        slot = shadow.grad_slot(ctx.target, (V, D))
        acc = slot.view(V, D) if slot is not None else torch.zeros((V, D), dtype=torch.float32, device=dout.device)
        _check(lib.kb200_embedding_bwd(_p(dout), _p(ids64), _p(acc), _ll(ids64.numel()), _i(D), _ll(V), _i(_dt(dout)), _stream()), "embedding_bwd")
        if slot is not None:
            return None, None, None, None  # already inside the parameter's gradient
        return acc.to(ctx.table_dtype), None, None, None


def int8_quantize_rows(x2, eps, qmax=127.0):
    """Per-row dynamic quantisation of a contiguous 2-D bf16 / fp32 tensor: ``(codes int8, scale [rows, 1] in x's dtype,
    1 / scale fp32 [rows])`` in one kernel."""
    lib = _lib()
    rows, K = x2.shape
    q = torch.empty((rows, K), dtype=torch.int8, device=x2.device)
    scale = torch.empty((rows, 1), dtype=x2.dtype, device=x2.device)
    inv = torch.empty((rows,), dtype=torch.float32, device=x2.device)
    _check(lib.kb200_int8_quantize_rows(_p(x2), _p(q), _p(scale), _p(inv), _ll(rows), _i(K), _f(eps), _f(qmax), _i(_dt(x2)), _stream()), "int8_quantize_rows")
    return q, scale, inv


def resize_nhwc(x, out_hw, nearest, out_dtype=None):
    """Bilinear (half-pixel centres, no antialiasing) or nearest resize of a contiguous NHWC tensor of uint8, bf16 or fp32."""
    lib = _lib()
    codes = {torch.float32: 0, torch.bfloat16: 1, torch.uint8: 2}
    x = x.contiguous()
    out_dtype = out_dtype or x.dtype
    N, H, W, C = x.shape
    y = torch.empty((N, out_hw[0], out_hw[1], C), dtype=out_dtype, device=x.device)
    _check(lib.kb200_resize_nhwc(_p(x), _p(y), _i(N), _i(H), _i(W), _i(C), _i(out_hw[0]), _i(out_hw[1]), _i(1 if nearest else 0), _i(codes[x.dtype]),
                                 _i(codes[out_dtype]), _stream()), "resize_nhwc")
    return y


# ------------------------------------------------------------------------------ batch norm
class FusedBatchNormAct(torch.autograd.Function):
    """y = relu?(batchnorm_train(x) (+ residual)) for channels-last x, with moving-stat update."""

    @staticmethod
    def forward(ctx, x, gamma, beta, residual, moving_mean, moving_var, momentum, eps, relu, pre_bias=None, conv_stats=None, merge=None):
        lib = _lib()
        C = x.shape[-1]
        M = x.numel() // C
        x = x.contiguous()
        dev = x.device
        stats = torch.empty(4 * C, dtype=torch.float32, device=dev)
        mean, invstd, scale, shift = stats[:C], stats[C:2 * C], stats[2 * C:3 * C], stats[3 * C:]
        y = torch.empty_like(x)
        st = _stream()
        dt = _dt(x)
        if conv_stats is not None and conv_stats.count == M:
            # the producing convolution's epilogue already summed x and x^2 per channel
            cs = conv_stats
            _check(lib.kb200_bn_finalize_partials(_p(cs.partials), _i(cs.grid), _i(cs.n_tiles), _i(cs.bn), _i(cs.ld), _p(gamma), _p(beta), _p(pre_bias),
                                                  _p(moving_mean), _p(moving_var), _f(momentum), _f(eps), _ll(M), _i(C), _p(mean), _p(invstd), _p(scale),
                                                  _p(shift), st), "bn_finalize_partials")
        else:
            sums = torch.empty(2 * C, dtype=torch.float32, device=dev)
            _check(lib.kb200_bn_stats(_p(x), _ll(M), _i(C), _i(dt), _p(sums), st), "bn_stats")
            _check(lib.kb200_bn_finalize(_p(sums), _p(gamma), _p(beta), _p(pre_bias), _p(moving_mean), _p(moving_var), _f(momentum), _f(eps), _ll(M), _i(C),
                                         _p(mean), _p(invstd), _p(scale), _p(shift), st), "bn_finalize")
        res = residual.contiguous() if residual is not None else None
        bits = None
        if relu:
            bits = torch.empty(M * (C // (8 if dt == 1 else 4)), dtype=torch.uint8, device=dev)
            _check(lib.kb200_bn_apply_mask(_p(x), _p(res), _p(y), _p(bits), _p(scale), _p(shift), _ll(M), _i(C), _i(1), _i(dt), st), "bn_apply")
        else:
            _check(lib.kb200_bn_apply(_p(x), _p(res), _p(y), _p(scale), _p(shift), _ll(M), _i(C), _i(0), _i(dt), st), "bn_apply")
        ctx.save_for_backward(x, bits, gamma, stats)
        # fp32 leaf parameters: their gradients can be added into persistent storage by the coefficient kernel
        ctx.leaves = (gamma if gamma is not None and gamma.is_leaf and gamma.requires_grad else None,
                      beta if beta is not None and beta.is_leaf and beta.requires_grad else None)
        ctx.relu = relu
        ctx.has_res = residual is not None
        ctx.merge = merge if residual is not None else None  # grad_merge.MergeSlot of the residual activation
        ctx.res_shape = tuple(residual.shape) if residual is not None else None
        ctx.dims = (M, C)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        x, bits, gamma, stats = ctx.saved_tensors
        M, C = ctx.dims
        mean, invstd = stats[:C], stats[C:2 * C]
        dy = dy.contiguous()
        dev = x.device
        sums = torch.empty(5 * C, dtype=torch.float32, device=dev)
        coef = sums[2 * C:]
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        st = _stream()
        dt = _dt(x)
        _check(lib.kb200_bn_bwd_reduce_mask(_p(dy), _p(x), _p(bits), _p(mean), _p(invstd), _ll(M), _i(C), _i(dt), _p(sums), st), "bn_bwd_reduce")
        from keras_b200.kernels import shadow

        slot_g, slot_b = shadow.grad_slot(ctx.leaves[0], (C,)), shadow.grad_slot(ctx.leaves[1], (C,))
        _check(lib.kb200_bn_bwd_apply_mask_acc(_p(dy), _p(x), _p(bits), _p(mean), _p(invstd), _p(gamma), _p(sums), _p(coef), _p(dx), _p(dres),
                                               _p(slot_g), _p(slot_b), _ll(M), _i(C), _i(dt), st), "bn_bwd_apply")
        dgamma = sums[C:2 * C] if gamma is not None and slot_g is None else None
        dbeta = sums[:C] if slot_b is None else None
        if dres is not None and ctx.merge is not None:
            from keras_b200.kernels import grad_merge

            dres = dres.view(ctx.res_shape)
            other = grad_merge.target(ctx.merge, dres.shape, dres.dtype)
            if other is not None:
                other.add_(dres)  # the other consumer of the residual activation ran first: its tensor carries the sum
                dres = None
            else:
                grad_merge.offer(ctx.merge, dres)
        return dx, dgamma, dbeta, dres, None, None, None, None, None, None, None, None


def bn_inference(x, scale, shift, residual, relu):
    """y = relu?(x*scale + shift (+ residual)) with per-channel fp32 scale/shift (no autograd)."""
    lib = _lib()
    C = x.shape[-1]
    M = x.numel() // C
    x = x.contiguous()
    y = torch.empty_like(x)
    res = residual.contiguous() if residual is not None else None
    _check(lib.kb200_bn_apply(_p(x), _p(res), _p(y), _p(scale), _p(shift), _ll(M), _i(C), _i(1 if relu else 0), _i(_dt(x)), _stream()), "bn_apply")
    return y


# ------------------------------------------------------------------- layer norm / rms norm
class FusedNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        lib = _lib()
        D = x.shape[-1]
        rows = x.numel() // D
        x = x.contiguous()
        y = torch.empty_like(x)
        stats = torch.empty(2 * rows, dtype=torch.float32, device=x.device)
        mean, rstd = stats[:rows], stats[rows:]
        g = gamma.float().contiguous() if gamma is not None else None
        b = beta.float().contiguous() if beta is not None else None
        _check(lib.kb200_norm_fwd(_p(x), _p(g), _p(b), _p(y), _p(mean), _p(rstd), _ll(rows), _i(D), _f(eps), _i(1 if rms else 0), _i(_dt(x)), _stream()), "norm_fwd")
        ctx.save_for_backward(x, g, stats)
        ctx.rms = rms
        ctx.has_beta = beta is not None
        # fp32 leaf parameters handed in directly: their gradients can be added into persistent storage by the reduction
        ctx.leaves = (gamma if gamma is not None and gamma.is_leaf and gamma.requires_grad else None,
                      beta if beta is not None and beta.is_leaf and beta.requires_grad else None)
        ctx.gamma_dtype = gamma.dtype if gamma is not None else None
        ctx.beta_dtype = beta.dtype if beta is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        x, g, stats = ctx.saved_tensors
        D = x.shape[-1]
        rows = x.numel() // D
        mean, rstd = stats[:rows], stats[rows:]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        lib.kb200_norm_bwd_blocks.restype = ctypes.c_int
        nb = lib.kb200_norm_bwd_blocks(_ll(rows))
        pdg = torch.empty((nb, D), dtype=torch.float32, device=x.device)
        pdb = torch.empty((nb, D), dtype=torch.float32, device=x.device) if ctx.has_beta else None
        from keras_b200.kernels import shadow

        slot_g = shadow.grad_slot(ctx.leaves[0], (D,)) if g is not None else None
        slot_b = shadow.grad_slot(ctx.leaves[1], (D,)) if ctx.has_beta else None
        if g is not None and slot_g is not None and (slot_b is not None or not ctx.has_beta):
            _check(lib.kb200_norm_bwd(_p(dy), _p(x), _p(g), _p(mean), _p(rstd), _p(dx), _p(pdg), _p(pdb), _p(slot_g), _p(slot_b), _ll(rows), _i(D),
                                      _i(1 if ctx.rms else 0), _i(_dt(x)), _i(1), _stream()), "norm_bwd")
            return dx, None, None, None, None
        dgamma = torch.empty(D, dtype=torch.float32, device=x.device) if g is not None else None
        dbeta = torch.empty(D, dtype=torch.float32, device=x.device) if ctx.has_beta else None
        _check(lib.kb200_norm_bwd(_p(dy), _p(x), _p(g), _p(mean), _p(rstd), _p(dx), _p(pdg), _p(pdb), _p(dgamma), _p(dbeta), _ll(rows), _i(D),
                                  _i(1 if ctx.rms else 0), _i(_dt(x)), _i(0), _stream()), "norm_bwd")
        if dgamma is not None and ctx.gamma_dtype != torch.float32:
            dgamma = dgamma.to(ctx.gamma_dtype)
        if dbeta is not None and ctx.beta_dtype != torch.float32:
            dbeta = dbeta.to(ctx.beta_dtype)
        return dx, dgamma, dbeta, None, None


def column_sum(x, accumulate_into=None):
    """fp32 sums over the rows of a 2-D bf16/fp32 CUDA tensor (bias gradients); falls back to torch for other layouts.
    ``accumulate_into``: an fp32 vector the sums are added to (returned) instead of a fresh result."""
    vn = 8 if x.dtype == torch.bfloat16 else 4
    if (x.ndim != 2 or not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32) or x.stride(1) != 1 or x.shape[1] % vn or x.stride(0) % vn
            or x.data_ptr() % 16 or x.shape[0] < 256):
        sums = x.sum(0, dtype=torch.float32)
        return sums if accumulate_into is None else accumulate_into.add_(sums)
    lib = _lib()
    rows, cols = x.shape
    lib.kb200_colsum_slabs.restype = ctypes.c_int
    slabs = lib.kb200_colsum_slabs(_ll(rows), _i(cols), _i(_dt(x)))
    partial = torch.empty((slabs, cols), dtype=torch.float32, device=x.device)
    out = torch.empty(cols, dtype=torch.float32, device=x.device) if accumulate_into is None else accumulate_into
    _check(lib.kb200_colsum(_p(x), _ll(x.stride(0)), _ll(rows), _i(cols), _p(partial), _p(out), _i(_dt(x)), _i(0 if accumulate_into is None else 1),
                            _stream()), "colsum")
    return out


# ----------------------------------------------------------------- softmax cross-entropy
class FusedSoftmaxXent(torch.autograd.Function):
    """Per-row loss in float32 from logits of any float dtype.  Logits may be the leading columns of a wider buffer
    (rows with a uniform pitch, as a padded GEMM returns them); the gradient then has the same pitch and zeroed padding."""

    @staticmethod
    def forward(ctx, logits, labels):
        lib = _lib()
        V = logits.shape[-1]
        rows = logits.numel() // V
        flat = logits.reshape(rows, V)  # a view whenever the leading dimensions collapse
        if flat.stride(1) != 1 or (rows > 1 and flat.stride(0) < V):
            flat = flat.contiguous()
        ld = flat.stride(0) if rows > 1 else V
        labels64 = labels.reshape(-1).to(torch.int64).contiguous()
        out = torch.empty(2 * rows, dtype=torch.float32, device=logits.device)
        loss, lse = out[:rows], out[rows:]
        _check(lib.kb200_xent_fwd(_p(flat), _p(labels64), _p(loss), _p(lse), _ll(rows), _i(V), _ll(ld), _i(_dt(flat)), _stream()), "xent_fwd")
        ctx.save_for_backward(flat, labels64, lse)
        ctx.logits_shape = tuple(logits.shape)
        ctx.ld = ld
        return loss.reshape(labels.shape)

    @staticmethod
    def backward(ctx, dloss):
        lib = _lib()
        flat, labels64, lse = ctx.saved_tensors
        rows, V = flat.shape
        ld = ctx.ld
        dl = dloss.reshape(-1).float().contiguous()
        buf = torch.empty((rows, ld), dtype=flat.dtype, device=flat.device)
        zero_to = ld if ld - V < 16 else V
        _check(lib.kb200_xent_bwd(_p(flat), _p(labels64), _p(lse), _p(dl), _p(buf), _ll(rows), _i(V), _ll(ld), _i(zero_to), _i(_dt(flat)), _stream()),
               "xent_bwd")
        dlogits = buf if ld == V else buf[:, :V]
        return dlogits.reshape(ctx.logits_shape), None


# ------------------------------------------------------------------------ fused optimizers
class OptimizerPlan:
    """Device-resident descriptor + chunk tables for one (optimizer, variable list) pair."""

    def __init__(self, params, grads, slot0, slot1, shadows, decays):
        lib = _lib()
        lib.kb200_opt_chunk_elems.restype = ctypes.c_int
        lib.kb200_opt_desc_bytes.restype = ctypes.c_int
        chunk = lib.kb200_opt_chunk_elems()
        assert lib.kb200_opt_desc_bytes() == 56
        import numpy as np

        n = len(params)
        desc = np.zeros(n, dtype=[("param", "<u8"), ("grad", "<u8"), ("slot0", "<u8"), ("slot1", "<u8"), ("shadow", "<u8"), ("numel", "<i8"), ("decay", "<f4"), ("pad", "<i4")])
        chunks = []
        for i, p in enumerate(params):
            desc[i]["param"] = p.data_ptr()
            desc[i]["grad"] = grads[i].data_ptr()
            desc[i]["slot0"] = slot0[i].data_ptr() if slot0 is not None and slot0[i] is not None else 0
            desc[i]["slot1"] = slot1[i].data_ptr() if slot1 is not None and slot1[i] is not None else 0
            desc[i]["shadow"] = shadows[i].data_ptr() if shadows is not None and shadows[i] is not None else 0
            desc[i]["numel"] = p.numel()
            desc[i]["decay"] = decays[i]
            for start in range(0, p.numel(), chunk):
                chunks.append((i, 0, start))
        ch = np.array(chunks, dtype=[("tensor", "<i4"), ("pad", "<i4"), ("start", "<i8")]) if chunks else np.zeros(0, dtype=[("tensor", "<i4"), ("pad", "<i4"), ("start", "<i8")])
        dev = params[0].device
        self.desc_host = desc
        self.desc = torch.from_numpy(desc.view(np.uint8).copy()).to(dev)
        self.chunks = torch.from_numpy(ch.view(np.uint8).copy()).to(dev)
        self.n_chunks = len(chunks)
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        self.keep = (params, grads, slot0, slot1, shadows)

    def set_decays(self, decays):
        """Refresh the per-tensor weight-decay coefficients (0 for tensors excluded from decay)."""
        import numpy as np

        changed = False
        for i, d in enumerate(decays):
            if self.desc_host[i]["decay"] != np.float32(d):
                self.desc_host[i]["decay"] = d
                changed = True
        if changed:
            self.desc.copy_(torch.from_numpy(self.desc_host.view(np.uint8).copy()), non_blocking=True)

    def adam(self, alpha, beta1, beta2, eps, lr=0.0, grad_scale=1.0, zero_grad=True, check_inf=False, lr_tensor=None, step_tensor=None):
        """``lr_tensor`` (fp32 scalar) and ``step_tensor`` (int32 count of completed updates), both on the device: the kernel
        reads them and derives the bias-corrected step size itself; ``alpha`` and ``lr`` are then ignored."""
        lib = _lib()
        _check(lib.kb200_fused_adam(_p(self.desc), _p(self.chunks), _i(self.n_chunks), _f(alpha), _f(lr), _d(beta1), _d(beta2), _f(eps),
                                    _f(grad_scale), _i(1 if zero_grad else 0), _p(self.found_inf) if check_inf else _vp(0), _p(lr_tensor),
                                    _p(step_tensor), _stream()), "fused_adam")

    def sgd(self, lr, momentum, nesterov, grad_scale=1.0, zero_grad=True, check_inf=False, lr_tensor=None):
        lib = _lib()
        _check(lib.kb200_fused_sgd(_p(self.desc), _p(self.chunks), _i(self.n_chunks), _f(lr), _f(momentum), _i(1 if nesterov else 0), _f(grad_scale),
                                   _i(1 if zero_grad else 0), _p(self.found_inf) if check_inf else _vp(0), _p(lr_tensor), _stream()), "fused_sgd")


    RULES = {"rmsprop": 0, "adagrad": 1, "adadelta": 2, "adamax": 3, "nadam": 4, "lion": 5}

    def rule(self, name, lr, consts, step_scalars=(), beta1=0.0, beta2=0.0, flags=0, grad_scale=1.0, zero_grad=True, lr_tensor=None, step_tensor=None,
             u_product=None):
        """One launch of the rule kernel ``name`` over every tensor of the plan.  ``consts``: up to four rule constants;
        ``step_scalars``: up to four step-dependent scalars by value, ignored by the rules that derive them from
        ``step_tensor`` (Adamax, Nadam); ``u_product``: Nadam's device-resident running product, advanced by the kernel
        when ``step_tensor`` is given."""
        lib = _lib()
        c = (ctypes.c_float * 4)(*(list(consts) + [0.0] * (4 - len(consts))))
        k = (ctypes.c_float * 4)(*(list(step_scalars) + [0.0] * (4 - len(step_scalars))))
        scratch = None
        if name == "nadam" and step_tensor is not None:
            scratch = getattr(self, "_scratch", None)
            if scratch is None:
                scratch = self._scratch = torch.zeros(4, dtype=torch.float32, device=self.desc.device)
        _check(lib.kb200_fused_rule(_p(self.desc), _p(self.chunks), _i(self.n_chunks), _i(self.RULES[name]), _f(lr), c, k, _d(beta1), _d(beta2), _i(flags),
                                    _f(grad_scale), _i(1 if zero_grad else 0), _vp(0), _p(lr_tensor), _p(step_tensor), _p(u_product), _p(scratch),
                                    _stream()), "fused_rule")


def cast_f32_to_bf16(src, dst):
    lib = _lib()
    _check(lib.kb200_cast_f32_bf16(_p(src), _p(dst), _ll(src.numel()), _stream()), "cast_f32_bf16")
