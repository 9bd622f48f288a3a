"""Routing of hot ops to the sm_100a kernels.

Each function returns ``None`` (or ``False``) when the call does not qualify (CPU tensor,
unsupported dtype or shape, kernels disabled by ``KERAS_B200_DISABLE_FUSED_KERNELS=1``, symbolic
tracing on the meta device); the caller then uses its library path.  On a CUDA device the kernel
library must be loadable: a missing build raises instead of silently falling back.
"""

import torch

from keras_b200.core import config

_FLOAT_IO = (torch.float32, torch.bfloat16)


def enabled(t):
    return isinstance(t, torch.Tensor) and t.is_cuda and config.fused_kernels_enabled()


def _ops():
    from keras_b200.kernels import ops

    return ops


# ------------------------------------------------------------------------------------ GEMM
def matmul(a, b):
    if not (enabled(a) and enabled(b)):
        return None
    from keras_b200.kernels import gemm

    return gemm.matmul(a, b)


def dense(x, kernel, bias, activation_name, kernel_shape=None):
    if not enabled(x):
        return None
    from keras_b200.kernels import gemm

    return gemm.dense(x, kernel, bias, activation_name, kernel_shape)


_I8_TRANSPOSED = {}


_I8_COL_SCALE = {}


def int8_quantize_rows(x, quantizer):
    """Dynamic abs-max quantisation of ``x`` over its last axis in one kernel: ``(codes, scale, 1 / scale as fp32)`` with the
    leading shape of ``x``, or ``None`` when ``quantizer`` is not the plain symmetric int8 one."""
    from keras_b200 import quantizers

    if not enabled(x) or x.dtype not in _FLOAT_IO or x.ndim < 2 or x.numel() == 0 or type(quantizer) is not quantizers.AbsMaxQuantizer:
        return None
    if tuple(quantizer.value_range) != (-127, 127) or quantizer.output_dtype != "int8":
        return None
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    q, scale, inv = _ops().int8_quantize_rows(x2, float(quantizer.epsilon))
    lead = tuple(x.shape[:-1])
    return q.reshape(lead + (x.shape[-1],)), scale.reshape(lead + (1,)), inv


def _i8_operands(kernel, kernel_scale):
    """Per int8 kernel [K, N], cached: the kernel transposed to [Np, K] (the GEMM wants both operands K-major; N padded to
    a multiple of 8 with zero rows) and 1 / kernel_scale as fp32 [Np]."""
    K, N = kernel.shape
    Np = (N + 7) // 8 * 8
    key = kernel.data_ptr()
    hit = _I8_TRANSPOSED.get(key)
    if hit is None or hit[0] != kernel._version or hit[1].shape != (Np, K):
        if len(_I8_TRANSPOSED) > 256:
            _I8_TRANSPOSED.clear()
        bt = kernel.t().contiguous()
        if Np != N:
            bt = torch.nn.functional.pad(bt, (0, 0, 0, Np - N))
        hit = (kernel._version, bt)
        _I8_TRANSPOSED[key] = hit
    ckey = kernel_scale.data_ptr()
    chit = _I8_COL_SCALE.get(ckey)
    if chit is None or chit[0] != kernel_scale._version or chit[1].numel() != Np:
        if len(_I8_COL_SCALE) > 256:
            _I8_COL_SCALE.clear()
        col = torch.reciprocal(kernel_scale.detach().reshape(-1).float())
        if Np != N:
            col = torch.nn.functional.pad(col, (0, Np - N))
        chit = (kernel_scale._version, col)
        _I8_COL_SCALE[ckey] = chit
    return hit[1], chit[1], Np


def int8_matmul(q_inputs, kernel, inputs_scale, kernel_scale, out_dtype=torch.bfloat16, inv_inputs_scale=None, bias=None, act=0):
    """``act((q_inputs @ kernel) / (inputs_scale * kernel_scale) + bias)`` on the int8 tensor-core GEMM, or ``None``.

    ``q_inputs``: int8 [..., K] with per-row ``inputs_scale`` [..., 1]; ``kernel``: int8 [K, N] with ``kernel_scale`` [N];
    ``inv_inputs_scale``: 1 / inputs_scale as fp32 [rows] when the caller already has it; ``bias``: fp32 [N] added in the
    epilogue; ``act``: activation code of the GEMM epilogue."""
    if not (enabled(q_inputs) and enabled(kernel)) or q_inputs.dtype != torch.int8 or kernel.dtype != torch.int8 or kernel.ndim != 2:
        return None
    K, N = kernel.shape
    a2 = q_inputs.reshape(-1, K)
    M = a2.shape[0]
    if K % 16 or M < 16 or not a2.is_contiguous() or (inputs_scale is None and inv_inputs_scale is None) or kernel_scale.numel() != N:
        return None
    row_scale = inv_inputs_scale if inv_inputs_scale is not None else torch.reciprocal(inputs_scale.reshape(-1).float())
    if row_scale.numel() != M:
        return None
    from keras_b200.kernels import gemm as kgemm

    ops = _ops()
    bt, col_scale, Np = _i8_operands(kernel, kernel_scale)
    if bias is not None:
        bias = bias.detach().reshape(-1).float()
        if Np != N:
            bias = torch.nn.functional.pad(bias, (0, Np - N))
    out = torch.empty((M, Np), dtype=out_dtype, device=a2.device)
    err = kgemm._err_flag(a2.device)
    code = ops._lib().kb200_gemm_i8(ops._p(a2), ops._p(bt), ops._p(out), ops._p(bias), ops._p(row_scale), ops._p(col_scale), ops._i(M), ops._i(Np), ops._i(K),
                                    ops._ll(a2.stride(0)), ops._ll(bt.stride(0)), ops._ll(out.stride(0)), ops._i(act),
                                    ops._i(1 if out_dtype == torch.float32 else 0), ops._p(err), ops._stream())
    ops._check(code, "gemm_i8")
    if Np != N:
        out = out[:, :N]
    return out.reshape(tuple(q_inputs.shape[:-1]) + (N,))


def int8_dense(inputs, kernel, kernel_scale, quantizer, bias, activation_name):
    """Inference form of an int8 Dense layer in two launches: per-row quantisation of the activations, then the int8 GEMM
    whose epilogue de-scales, adds the bias and applies the activation.  Returns ``(output, activation_applied)`` or ``None``
    (gradients are needed, or the call does not qualify)."""
    if not enabled(inputs) or (torch.is_grad_enabled() and inputs.requires_grad) or inputs.dtype not in _FLOAT_IO:
        return None
    quantised = int8_quantize_rows(inputs, quantizer)
    if quantised is None:
        return None
    from keras_b200.kernels import gemm as kgemm

    q, _, inv = quantised
    name = {"gelu": "gelu_erf"}.get(activation_name, activation_name)
    act = kgemm._ACT.get(name)
    out = int8_matmul(q, kernel, None, kernel_scale, out_dtype=inputs.dtype, inv_inputs_scale=inv, bias=bias, act=act or 0)
    if out is None:
        return None
    return out, act is not None


def fp8_matmul(layer, inputs, kernel, equation, training, bias=None):
    """float8-policy product on the fp8 tensor-core GEMM (plain matmul on the last axis only); ``None`` otherwise.  ``bias``
    (optional) is added by the GEMM's epilogue."""
    if equation is not None or not enabled(inputs):
        return None
    from keras_b200.kernels import fp8

    return fp8.linear(layer, inputs, kernel, training, bias=bias)


def conv(x, kernel, strides, padding, data_format, dilation):
    if not (enabled(x) and enabled(kernel)) or x.ndim != 4:
        return None
    from keras_b200.kernels import conv as conv_mod

    return conv_mod.conv(x, kernel, strides, padding, data_format, dilation)


# ------------------------------------------------------------------------- normalisation
def layer_norm(x, gamma, beta, eps):
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.shape[-1] > 8192 or x.numel() == 0:
        return None
    return _ops().FusedNorm.apply(x, gamma, beta, float(eps), False)


def rms_norm(x, scale, eps):
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.shape[-1] > 8192 or x.numel() == 0:
        return None
    return _ops().FusedNorm.apply(x, scale, None, float(eps), True)


def batch_norm(layer, inputs, training, residual=None, relu=False, pre_bias=None, conv_stats=None):
    """Fused channels-last BatchNorm (+residual)(+ReLU).  Returns ``None`` when not applicable.

    ``conv_stats``: partial sums of ``inputs`` left by the producing convolution kernel (training mode only); the
    statistics pass over ``inputs`` is then skipped."""
    x = inputs
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.ndim < 2:
        return None
    axis = layer.axis % x.ndim
    if axis != x.ndim - 1:
        return None
    C = x.shape[-1]
    vec = 8 if x.dtype == torch.bfloat16 else 4
    if C % vec != 0 or x.numel() == 0:
        return None
    gamma = layer.gamma._value if layer.scale else None
    beta = layer.beta._value if layer.center else None
    if (gamma is not None and gamma.dtype != torch.float32) or (beta is not None and beta.dtype != torch.float32):
        return None
    mm, mv = layer.moving_mean._value, layer.moving_variance._value
    if mm.dtype != torch.float32:
        return None
    ops = _ops()
    if training:
        if beta is None:
            beta = torch.zeros(C, dtype=torch.float32, device=x.device)
        from keras_b200.kernels import grad_merge

        return ops.FusedBatchNormAct.apply(x, gamma, beta, residual, mm, mv, float(layer.momentum), float(layer.epsilon), bool(relu), pre_bias, conv_stats,
                                           grad_merge.slot_of(residual))
    if torch.is_grad_enabled() and (x.requires_grad or (gamma is not None and gamma.requires_grad and layer.trainable)):
        return None
    with torch.no_grad():
        inv = torch.rsqrt(mv + layer.epsilon)
        scale = inv * gamma if gamma is not None else inv
        shift = -mm * scale if pre_bias is None else (pre_bias.float() - mm) * scale
        if beta is not None:
            shift = shift + beta
    return ops.bn_inference(x, scale.contiguous(), shift.contiguous(), residual, relu)


def max_pool2d(x, pool_size, strides, padding, zero_pad=None):
    """Channels-last 2-D max pooling; ``zero_pad=((top, bottom), (left, right))`` folds a preceding ZeroPadding2D.

    Returns ``None`` when not applicable."""
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.ndim != 4 or x.numel() == 0:
        return None
    N, H, W, C = x.shape
    if C % (8 if x.dtype == torch.bfloat16 else 4) != 0 or pool_size[0] * pool_size[1] > 255:
        return None
    if zero_pad is not None:
        if padding != "valid":
            return None
        (pt, pb), (pl, pr) = zero_pad
        OH = (H + pt + pb - pool_size[0]) // strides[0] + 1
        OW = (W + pl + pr - pool_size[1]) // strides[1] + 1
        mode = 1
    elif padding == "same":
        OH, OW = -(-H // strides[0]), -(-W // strides[1])
        pt = max((OH - 1) * strides[0] + pool_size[0] - H, 0) // 2
        pl = max((OW - 1) * strides[1] + pool_size[1] - W, 0) // 2
        mode = 0
    else:
        OH = (H - pool_size[0]) // strides[0] + 1
        OW = (W - pool_size[1]) // strides[1] + 1
        pt = pl = 0
        mode = 0
    if OH <= 0 or OW <= 0:
        return None
    return _ops().FusedMaxPool2D.apply(x, tuple(pool_size), tuple(strides), (pt, pl), (OH, OW), mode)


def avg_pool2d(x, pool_size, strides, padding):
    """Channels-last 2-D average pooling (padding excluded from the average) or ``None``."""
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.ndim != 4 or x.numel() == 0:
        return None
    N, H, W, C = x.shape
    if C % (8 if x.dtype == torch.bfloat16 else 4) != 0:
        return None
    if padding == "same":
        OH, OW = -(-H // strides[0]), -(-W // strides[1])
        pt = max((OH - 1) * strides[0] + pool_size[0] - H, 0) // 2
        pl = max((OW - 1) * strides[1] + pool_size[1] - W, 0) // 2
    else:
        OH = (H - pool_size[0]) // strides[0] + 1
        OW = (W - pool_size[1]) // strides[1] + 1
        pt = pl = 0
    if OH <= 0 or OW <= 0:
        return None
    return _ops().FusedAvgPool2D.apply(x, tuple(pool_size), tuple(strides), (pt, pl), (OH, OW))


def global_avg_pool(x):
    """Mean over all axes between the first and the last of a channels-last tensor, ``[N, ..., C] -> [N, C]``, or ``None``."""
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.ndim < 3 or x.numel() == 0:
        return None
    if x.shape[-1] % (8 if x.dtype == torch.bfloat16 else 4) != 0:
        return None
    return _ops().FusedGlobalAvgPool.apply(x)


def softmax(x, mask=None, masked_add=0.0, log=False):
    """softmax / log-softmax over the last axis in the input's dtype (fp32 arithmetic), or ``None``."""
    if not enabled(x) or x.dtype not in _FLOAT_IO or x.ndim < 1 or x.numel() == 0 or x.shape[-1] > (1 << 24):
        return None
    if mask is not None and not (isinstance(mask, torch.Tensor) and mask.is_cuda):
        return None
    return _ops().FusedSoftmax.apply(x, mask, float(masked_add), bool(log))


def embedding(variable, table, ids, out_dtype):
    """``table[ids]`` cast to ``out_dtype`` in one gather kernel, with a scatter-add gradient, or ``None``.

    ``variable`` is the ``Variable`` the table was read from (or ``None``)."""
    if not enabled(table) or not isinstance(ids, torch.Tensor) or not ids.is_cuda or table.ndim != 2 or table.dtype not in _FLOAT_IO:
        return None
    if out_dtype not in _FLOAT_IO or table.shape[1] % 8 or ids.dtype not in (torch.int32, torch.int64) or ids.numel() == 0:
        return None
    if getattr(variable, "_shard_slices", None) is not None:
        return None
    from keras_b200.kernels import gemm

    target = gemm._grad_target(variable, table) if variable is not None else None
    return _ops().FusedEmbedding.apply(table, ids, out_dtype, target)


def resize(x, out_hw, interpolation):
    """NHWC bilinear / nearest resize without antialiasing, or ``None``."""
    if not enabled(x) or x.ndim != 4 or x.dtype not in (torch.float32, torch.bfloat16, torch.uint8) or x.numel() == 0:
        return None
    if interpolation not in ("bilinear", "nearest") or (torch.is_grad_enabled() and x.requires_grad):
        return None
    return _ops().resize_nhwc(x, out_hw, interpolation == "nearest")


def softmax_cross_entropy(logits, labels):
    if not enabled(logits) or logits.dtype not in _FLOAT_IO or logits.numel() == 0:
        return None
    if logits.shape[-1] < 64:
        return None
    return _ops().FusedSoftmaxXent.apply(logits, labels)


def flash_attention(q, k, v, mask, scale, is_causal):
    if not enabled(q):
        return None
    from keras_b200.kernels import attention

    return attention.flash_attention(q, k, v, mask, scale, is_causal)


# ---------------------------------------------------------------------------- optimizers
def _plan_for(opt, grads, variables, slot_lists):
    if not variables:
        return None
    p0 = variables[0]._value
    if not enabled(p0):
        return None
    params = [v._value for v in variables]
    for p, g in zip(params, grads):
        if p.dtype != torch.float32 or g.dtype != torch.float32 or not g.is_contiguous() or not p.is_contiguous() or not p.is_cuda:
            return None
    key = (tuple(id(v) for v in variables), tuple(g.data_ptr() for g in grads), tuple(p.data_ptr() for p in params))
    cache = getattr(opt, "_fused_plan", None)
    if cache is not None and cache[0] == key:
        return cache[1]
    slots = []
    for lst in slot_lists:
        if lst is None:
            slots.append(None)
        else:
            slots.append([lst[opt._get_variable_index(v)]._value for v in variables])
    shadows = None
    from keras_b200.kernels import shadow

    shadows = shadow.shadows_for(variables)
    plan = _ops().OptimizerPlan(params, list(grads), slots[0], slots[1] if len(slots) > 1 else None, shadows, [0.0] * len(params))
    opt._fused_plan = (key, plan)
    return plan


def _decays(opt, variables):
    """Per-variable decoupled weight-decay coefficient (0 where the variable is excluded), or ``None`` without decay."""
    wd = opt.weight_decay
    if wd is None:
        return None
    return [float(wd) if opt._use_weight_decay(v) else 0.0 for v in variables]


def _consumes_gradients(opt):
    """True while the caller of ``apply`` is this package's training step, whose gradients live in its own persistent storage:
    the update kernel then zeroes them as it reads them.  Gradients handed to ``optimizer.apply`` by user code are left as they
    are (a custom loop may log or reuse them afterwards)."""
    return bool(getattr(opt, "_gradients_are_step_storage", False))


def _device_scalars(opt):
    """(learning-rate tensor, iteration tensor) when both live on the device in the types the kernels read: the update
    then takes its step scalars from device memory and a captured replay of it stays correct as they change."""
    lr = getattr(opt._learning_rate, "_value", None)
    it = getattr(opt._iterations, "_value", None)
    if (isinstance(lr, torch.Tensor) and isinstance(it, torch.Tensor) and lr.is_cuda and it.is_cuda and lr.dtype == torch.float32
            and it.dtype == torch.int32 and lr.numel() == 1 and it.numel() == 1):
        return lr, it
    return None, None


def fused_sgd(opt, grads, variables, lr):
    if opt.gradient_accumulation_steps:
        return False
    slot0 = opt.momentums if opt.momentum != 0 else None
    plan = _plan_for(opt, grads, variables, [slot0])
    if plan is None:
        return False
    d = _decays(opt, variables)
    if d is not None:
        plan.set_decays(d)
    scale = 1.0 / opt.loss_scale_factor if opt.loss_scale_factor else 1.0
    lr_t, _ = _device_scalars(opt)
    plan.sgd(lr, opt.momentum, opt.nesterov, grad_scale=scale, zero_grad=_consumes_gradients(opt), lr_tensor=lr_t)
    opt._fused_zeroed_grads = _consumes_gradients(opt)
    opt._step_scalars_on_device = lr_t is not None
    return True


def fused_adam(opt, grads, variables, lr):
    if opt.gradient_accumulation_steps:
        return False
    plan = _plan_for(opt, grads, variables, [opt._momentums, opt._velocities])
    if plan is None:
        return False
    d = _decays(opt, variables)
    if d is not None:
        plan.set_decays(d)
    scale = 1.0 / opt.loss_scale_factor if opt.loss_scale_factor else 1.0
    lr_t, step_t = _device_scalars(opt)
    if lr_t is not None:
        plan.adam(0.0, opt.beta_1, opt.beta_2, opt.epsilon, grad_scale=scale, zero_grad=_consumes_gradients(opt), lr_tensor=lr_t, step_tensor=step_t)
    else:
        plan.adam(opt._alpha(lr), opt.beta_1, opt.beta_2, opt.epsilon, lr=lr, grad_scale=scale, zero_grad=_consumes_gradients(opt))
    opt._fused_zeroed_grads = _consumes_gradients(opt)
    opt._step_scalars_on_device = lr_t is not None
    return True


def fused_rule(opt, grads, variables, lr, name, slot_lists, consts, step_scalars=(), beta1=0.0, beta2=0.0, flags=0, u_product=None,
               needs_step=False):
    """RMSprop / Adagrad / Adadelta / Adamax / Nadam / Lion: the whole variable list in one launch.  ``needs_step``: the rule
    has step-dependent scalars, taken from the device-resident iteration counter when there is one (the launch then
    stays valid inside a recorded step) and from ``step_scalars`` otherwise."""
    if opt.gradient_accumulation_steps:
        return False
    plan = _plan_for(opt, grads, variables, slot_lists)
    if plan is None:
        return False
    d = _decays(opt, variables)
    if d is not None:
        plan.set_decays(d)
    scale = 1.0 / opt.loss_scale_factor if opt.loss_scale_factor else 1.0
    lr_t, step_t = _device_scalars(opt)
    if u_product is not None and not (u_product.is_cuda and u_product.dtype == torch.float32 and u_product.numel() == 1):
        step_t = None
    plan.rule(name, lr, consts, step_scalars, beta1=beta1, beta2=beta2, flags=flags, grad_scale=scale, zero_grad=_consumes_gradients(opt), lr_tensor=lr_t,
              step_tensor=step_t if needs_step else None, u_product=u_product if (needs_step and step_t is not None) else None)
    opt._fused_zeroed_grads = _consumes_gradients(opt)
    opt._step_scalars_on_device = lr_t is not None and (not needs_step or step_t is not None)
    return True
