"""Quantization math and helpers (``keras.quantizers``).

Formulas follow keras/src/quantizers/quantizers.py (abs-max :70-121, fake-quant, float8 scale /
amax history :585-621, int4 nibble packing).  The int8 and float8 matmuls route to the sm_100a
kernels on a B200 and to plain torch elsewhere; both reproduce the reference numerics:
dynamic per-row activation quantisation for int8, delayed per-tensor scaling for float8 with the
new scale / history handed to the optimizer *as gradients* of the bookkeeping variables.
"""

import numpy as np
import torch

from keras_b200.core import config as _config
from keras_b200.core.dtypes import standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_numpy, convert_to_tensor
from keras_b200.quantizers.quantization_config import (  # noqa: F401
    AWQConfig, Float8QuantizationConfig, GPTQConfig, Int4QuantizationConfig, Int8QuantizationConfig,
    QuantizationConfig, TernaryQuantizationConfig, validate_and_resolve_config,
)

E4M3_MAX = 448.0
E5M2_MAX = 57344.0


@keras_export(["keras.Quantizer", "keras.quantizers.Quantizer"])
class Quantizer:
    def __init__(self, output_dtype="int8"):
        self.output_dtype = output_dtype

    def __call__(self, x):
        return x

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def get_config(self):
        raise NotImplementedError(f"{self} does not implement get_config()")


@keras_export("keras.quantizers.abs_max_quantize")
def abs_max_quantize(inputs, axis, value_range=(-127, 127), dtype="int8", epsilon=None, to_numpy=False):
    eps = _config.epsilon() if epsilon is None else epsilon
    if to_numpy:
        original = standardize_dtype(inputs.dtype)
        x = convert_to_numpy(inputs).astype("float32") if original == "bfloat16" else convert_to_numpy(inputs)
        ax = tuple(axis) if isinstance(axis, (list, tuple)) else axis
        scale = np.divide(value_range[1], np.add(np.max(np.abs(x), axis=ax, keepdims=True), eps))
        out = np.clip(np.round(np.multiply(x, scale)), value_range[0], value_range[1]).astype(dtype)
        return convert_to_tensor(out), convert_to_tensor(scale, dtype=original)
    x = convert_to_tensor(inputs)
    ax = tuple(axis) if isinstance(axis, (list, tuple)) else axis
    scale = (value_range[1] / (torch.amax(torch.abs(x), dim=ax, keepdim=True) + eps)).to(x.dtype)
    out = torch.clip(torch.round(x * scale), value_range[0], value_range[1]).to(to_torch_dtype(dtype))
    return out, scale


@keras_export("keras.quantizers.AbsMaxQuantizer")
class AbsMaxQuantizer(Quantizer):
    def __init__(self, axis=None, value_range=(-127, 127), epsilon=None, output_dtype="int8"):
        super().__init__(output_dtype=output_dtype)
        if isinstance(axis, (list, tuple)):
            axis = tuple(axis)
        self.axis = axis
        self.value_range = tuple(value_range)
        self.epsilon = _config.epsilon() if epsilon is None else epsilon

    def __call__(self, x, axis=None, to_numpy=False):
        ax = self.axis if axis is None else axis
        return abs_max_quantize(x, ax, self.value_range, self.output_dtype, self.epsilon, to_numpy)

    def get_config(self):
        return {"axis": self.axis, "value_range": self.value_range, "epsilon": self.epsilon, "output_dtype": self.output_dtype}


@keras_export("keras.quantizers.abs_max_quantize_grouped_with_zero_point")
def abs_max_quantize_grouped_with_zero_point(inputs, block_size, value_range=(-8, 7), dtype="int8", to_numpy=False):
    """Asymmetric group-wise quantisation of a ``(in, out)`` kernel along ``in``."""
    x = convert_to_tensor(inputs).to(torch.float32)
    in_dim, out_dim = x.shape
    groups = -(-in_dim // block_size)
    pad = groups * block_size - in_dim
    if pad:
        x = torch.nn.functional.pad(x, (0, 0, 0, pad))
    g = x.reshape(groups, block_size, out_dim)
    lo, hi = g.amin(dim=1), g.amax(dim=1)
    qmin, qmax = value_range
    scale = (hi - lo) / (qmax - qmin)
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    zero = torch.round(qmin - lo / scale)
    q = torch.clip(torch.round(g / scale[:, None, :] + zero[:, None, :]), qmin, qmax).reshape(groups * block_size, out_dim)[:in_dim]
    return q.to(to_torch_dtype(dtype)), scale, zero.to(torch.int8)


@keras_export("keras.quantizers.fake_quant_with_min_max_vars")
def fake_quant_with_min_max_vars(inputs, min_vals, max_vals, num_bits=8, narrow_range=False, axis=None):
    """Quantize-dequantize with a straight-through gradient for in-range values."""
    x = convert_to_tensor(inputs)
    lo = convert_to_tensor(min_vals).to(x.dtype)
    hi = convert_to_tensor(max_vals).to(x.dtype)
    if axis is not None and lo.ndim == 1:
        shape = [1] * x.ndim
        shape[axis] = -1
        lo, hi = lo.reshape(shape), hi.reshape(shape)
    qmin = 1.0 if narrow_range else 0.0
    qmax = float(2 ** num_bits - 1)
    scale = (hi - lo) / (qmax - qmin)
    inv = (qmax - qmin) / (hi - lo)
    zp_from_min = qmin - lo / scale
    nudged_zp = torch.where(zp_from_min < qmin, torch.full_like(lo, qmin), torch.where(zp_from_min > qmax, torch.full_like(lo, qmax), torch.round(zp_from_min)))
    nudged_min = (qmin - nudged_zp) * scale
    nudged_max = (qmax - nudged_zp) * scale
    clamped = torch.minimum(torch.maximum(x, nudged_min), nudged_max)
    q = torch.floor((clamped - nudged_min) * inv + 0.5) * scale + nudged_min
    mask = ((x >= nudged_min) & (x <= nudged_max)).to(x.dtype)
    # straight-through estimator: forward value q, gradient = mask
    return (x * mask).detach() * 0 + (x * mask - (x * mask).detach()) + q.detach()


@keras_export("keras.quantizers.compute_float8_scale")
def compute_float8_scale(amax, scale, dtype_max, margin=0):
    amax, scale = convert_to_tensor(amax), convert_to_tensor(scale)
    old_sf = torch.reciprocal(scale)
    sf = (dtype_max / amax) / (2 ** margin)
    sf = torch.where(amax > 0.0, sf, old_sf)
    sf = torch.where(torch.isfinite(amax), sf, old_sf)
    return torch.reciprocal(sf)


@keras_export("keras.quantizers.compute_float8_amax_history")
def compute_float8_amax_history(x, amax_history):
    x, amax_history = convert_to_tensor(x), convert_to_tensor(amax_history)
    new = torch.roll(amax_history, shifts=-1)
    new = new.clone()
    new[0] = torch.amax(torch.abs(x)).to(amax_history.dtype)
    return new


@keras_export("keras.quantizers.quantize_and_dequantize")
def quantize_and_dequantize(inputs, scale, quantized_dtype, compute_dtype):
    x = convert_to_tensor(inputs)
    ctd = to_torch_dtype(compute_dtype)
    qtd = to_torch_dtype(quantized_dtype)
    qmax = E4M3_MAX if qtd == torch.float8_e4m3fn else E5M2_MAX
    s = convert_to_tensor(scale).to(ctd)
    y = torch.clip(x.to(ctd) / s, -qmax, qmax).to(qtd)
    return y.to(ctd) * s


def _pack_nibbles(arr, axis, per_byte, bits):
    a = convert_to_numpy(arr)
    a = np.moveaxis(a, axis % a.ndim, 0)
    n = a.shape[0]
    pad = (-n) % per_byte
    if pad:
        a = np.concatenate([a, np.zeros((pad,) + a.shape[1:], dtype=a.dtype)], axis=0)
    mask = (1 << bits) - 1
    u = a.astype(np.uint8) & mask
    packed = np.zeros((a.shape[0] // per_byte,) + a.shape[1:], dtype=np.uint8)
    for i in range(per_byte):
        packed |= (u[i::per_byte] << (bits * i)).astype(np.uint8)
    return packed, n


@keras_export("keras.quantizers.pack_int4")
def pack_int4(arr, axis=0, dtype="int8"):
    if dtype not in ("int8", "uint8"):
        raise ValueError(f"Expected dtype to be 'int8' or 'uint8', but got '{dtype}'.")
    if standardize_dtype(arr.dtype) != dtype:
        raise TypeError(f"Expected {dtype} tensor for packing, got {standardize_dtype(arr.dtype)}.")
    packed, n = _pack_nibbles(arr, axis, 2, 4)
    packed = np.moveaxis(packed.view(np.dtype(dtype)), 0, axis % packed.ndim)
    return convert_to_tensor(packed), tuple(packed.shape), n


@keras_export("keras.quantizers.unpack_int4")
def unpack_int4(packed, orig_len, axis=0, dtype="int8"):
    if dtype not in ("int8", "uint8"):
        raise ValueError(f"Expected dtype to be 'int8' or 'uint8', but got '{dtype}'.")
    p = convert_to_tensor(packed)
    if p.dtype not in (torch.int8, torch.uint8):
        raise TypeError(f"Expected int8 or uint8 tensor for unpacking, got {p.dtype}")
    p = torch.movedim(p, axis % p.ndim, 0).to(torch.int16)
    low, high = p & 0x0F, (p >> 4) & 0x0F
    if dtype == "int8":
        low = torch.where(low > 7, low - 16, low)
        high = torch.where(high > 7, high - 16, high)
    out = torch.stack([low, high], dim=1).reshape((-1,) + tuple(p.shape[1:]))[:orig_len]
    return torch.movedim(out.to(to_torch_dtype(dtype)), 0, axis % out.ndim)


@keras_export("keras.quantizers.pack_int2")
def pack_int2(arr, axis=0, dtype="int8"):
    packed, n = _pack_nibbles(arr, axis, 4, 2)
    packed = np.moveaxis(packed.view(np.dtype(dtype)), 0, axis % packed.ndim)
    return convert_to_tensor(packed), tuple(packed.shape), n


@keras_export("keras.quantizers.unpack_int2")
def unpack_int2(packed, orig_len, axis=0, dtype="int8"):
    p = torch.movedim(convert_to_tensor(packed), axis % packed.ndim, 0).to(torch.int16)
    parts = []
    for i in range(4):
        v = (p >> (2 * i)) & 0x03
        if dtype == "int8":
            v = torch.where(v > 1, v - 4, v)
        parts.append(v)
    out = torch.stack(parts, dim=1).reshape((-1,) + tuple(p.shape[1:]))[:orig_len]
    return torch.movedim(out.to(to_torch_dtype(dtype)), 0, axis % out.ndim)


@keras_export("keras.quantizers.pack_ternary")
def pack_ternary(arr, axis=0):
    """Pack values in {-1, 0, +1} at five per ``uint8`` byte (base 3: ``d0 + 3 d1 + 9 d2 + 27 d3 + 81 d4`` with
    ``d = t + 1``), the layout of keras/src/quantizers/quantizers.py:1179-1260.  Returns ``(packed, packed_shape, orig_len)``."""
    a = convert_to_numpy(convert_to_tensor(arr))
    axis = axis % a.ndim
    a = np.moveaxis(a, axis, 0)
    n = a.shape[0]
    pad = (-n) % 5
    if pad:
        a = np.concatenate([a, np.zeros((pad,) + a.shape[1:], dtype=a.dtype)], axis=0)
    d = (np.clip(np.rint(a), -1, 1) + 1).astype(np.uint8).reshape((-1, 5) + a.shape[1:])
    weights = np.array([1, 3, 9, 27, 81], dtype=np.uint8).reshape((1, 5) + (1,) * (a.ndim - 1))
    packed = (d * weights).sum(axis=1).astype(np.uint8)
    packed = np.moveaxis(packed, 0, axis)
    return convert_to_tensor(packed), tuple(packed.shape), n


@keras_export("keras.quantizers.unpack_ternary")
def unpack_ternary(packed, orig_len, axis=0):
    p = convert_to_tensor(packed)
    axis = axis % p.ndim
    p = torch.movedim(p, axis, 0).to(torch.int16)
    digits = []
    for _ in range(5):
        digits.append(p % 3)
        p = p // 3
    out = torch.stack(digits, dim=1).reshape((-1,) + tuple(digits[0].shape[1:]))[:orig_len]
    return torch.movedim((out - 1).to(torch.int8), 0, axis)


# --- layer-level helpers shared by Dense / EinsumDense / Embedding ---------------------------

class _Int8MatmulFn(torch.autograd.Function):
    """int8 x int8 → int32 matmul, de-scaled; gradient flows to the activations only."""

    @staticmethod
    def forward(ctx, inputs, kernel, kernel_scale, quantizer, equation):
        compute = inputs.dtype
        inv_scale = None
        if quantizer is not None:
            fused_q = None
            if equation is None and inputs.is_cuda:
                from keras_b200.kernels import dispatch

                fused_q = dispatch.int8_quantize_rows(inputs, quantizer)
            if fused_q is not None:
                q_in, in_scale, inv_scale = fused_q
            else:
                q_in, in_scale = quantizer(inputs, axis=-1 if equation is None else quantizer.axis)
        else:
            q_in, in_scale = inputs, None
        ctx.save_for_backward(kernel, kernel_scale)
        ctx.compute = compute
        ctx.equation = equation
        if equation is None:
            from keras_b200.kernels import dispatch

            fused = None
            if quantizer is not None and compute in (torch.bfloat16, torch.float32):
                fused = dispatch.int8_matmul(q_in, kernel, in_scale, kernel_scale, out_dtype=compute, inv_inputs_scale=inv_scale)
            if fused is not None:
                return fused
            lead = q_in.shape[:-1]
            a2 = q_in.reshape(-1, q_in.shape[-1])
            if a2.is_cuda and a2.dtype == torch.int8 and a2.shape[0] > 16 and a2.shape[0] % 8 == 0 and a2.shape[1] % 8 == 0 and kernel.shape[1] % 8 == 0:
                acc = torch._int_mm(a2, kernel)
            elif a2.is_cuda:
                acc = torch.matmul(a2.to(torch.float32), kernel.to(torch.float32))
            else:
                acc = torch.matmul(a2.to(torch.int32), kernel.to(torch.int32))
            acc = acc.reshape(tuple(lead) + (kernel.shape[1],))
            out_scale = kernel_scale * in_scale if in_scale is not None else kernel_scale
            return (acc.to(compute) / out_scale).to(compute)
        raise NotImplementedError

    @staticmethod
    def backward(ctx, upstream):
        kernel, kernel_scale = ctx.saved_tensors
        float_kernel = kernel.to(ctx.compute) / kernel_scale.to(ctx.compute)
        return torch.matmul(upstream, float_kernel.t()), None, None, None, None


def int8_dense_forward(inputs, kernel, kernel_scale, inputs_quantizer):
    return _Int8MatmulFn.apply(convert_to_tensor(inputs), kernel, kernel_scale, inputs_quantizer, None)


def float8_build(layer, amax_history_length=None):
    """Create the six delayed-scaling variables (keras/src/layers/core/dense.py:895-936)."""
    from keras_b200.dtype_policies import QuantizedFloat8DTypePolicy

    policy = layer._resolved_policy()
    length = amax_history_length or getattr(policy, "amax_history_length", QuantizedFloat8DTypePolicy.default_amax_history_length)
    scale_kw = dict(shape=(), initializer="ones", dtype="float32", trainable=True, autocast=False, overwrite_with_gradient=True)
    hist_kw = dict(shape=(length,), initializer="zeros", dtype="float32", trainable=True, autocast=False, overwrite_with_gradient=True)
    layer.inputs_scale = layer.add_weight(name="inputs_scale", **scale_kw)
    layer.inputs_amax_history = layer.add_weight(name="inputs_amax_history", **hist_kw)
    layer.kernel_scale = layer.add_weight(name="kernel_scale", **scale_kw)
    layer.kernel_amax_history = layer.add_weight(name="kernel_amax_history", **hist_kw)
    layer.outputs_grad_scale = layer.add_weight(name="outputs_grad_scale", **scale_kw)
    layer.outputs_grad_amax_history = layer.add_weight(name="outputs_grad_amax_history", **hist_kw)


class _QDQOperand(torch.autograd.Function):
    """QDQ to e4m3 in forward; backward passes the gradient through and returns the *new*
    scale / amax history as the "gradients" of the bookkeeping variables."""

    @staticmethod
    def forward(ctx, x, scale, history, training, compute_dtype):
        if training:
            ctx.new_scale = compute_float8_scale(torch.amax(history, dim=0), scale, E4M3_MAX)
            ctx.new_history = compute_float8_amax_history(x, history)
        else:
            ctx.new_scale = ctx.new_history = None
        return quantize_and_dequantize(x, scale, "float8_e4m3fn", compute_dtype)

    @staticmethod
    def backward(ctx, upstream):
        return upstream, ctx.new_scale, ctx.new_history, None, None


class _QDQOutputGrad(torch.autograd.Function):
    """Identity in forward; QDQ of the incoming gradient to e5m2 in backward."""

    @staticmethod
    def forward(ctx, out, scale, history, compute_dtype):
        ctx.save_for_backward(scale, history)
        ctx.compute_dtype = compute_dtype
        return out.view_as(out)

    @staticmethod
    def backward(ctx, upstream):
        scale, history = ctx.saved_tensors
        new_scale = compute_float8_scale(torch.amax(history, dim=0), scale, E5M2_MAX)
        qdq = quantize_and_dequantize(upstream, scale, "float8_e5m2", ctx.compute_dtype)
        new_history = compute_float8_amax_history(upstream, history)
        return qdq, new_scale, new_history, None


def float8_matmul(layer, inputs, kernel, equation, training, bias=None):
    """``inputs (x) kernel`` with e4m3 operands and e5m2 output gradient, delayed scaling.

    ``equation`` None means a plain matmul on the last axis, else an einsum equation.  With ``bias`` (a variable of the
    output width) the result is ``(output, bias_added)``: the fp8 tensor-core path adds it in its epilogue, the emulated
    path leaves it to the caller.
    """
    from keras_b200.kernels import dispatch

    inputs = convert_to_tensor(inputs)
    compute = layer.compute_dtype
    training = bool(training)
    fused = dispatch.fp8_matmul(layer, inputs, kernel, equation, training, bias=bias)
    if fused is not None:
        return fused if bias is None else (fused, True)
    a = _QDQOperand.apply(inputs, layer.inputs_scale._value, layer.inputs_amax_history._value, training, compute)
    b = _QDQOperand.apply(kernel, layer.kernel_scale._value, layer.kernel_amax_history._value, training, compute)
    out = None
    if equation is None:
        out = dispatch.matmul(a, b.to(a.dtype))  # own bf16 GEMM (handles widths that are not multiples of 8), else the library
    if out is None:
        out = torch.matmul(a, b.to(a.dtype)) if equation is None else torch.einsum(equation, a, b.to(a.dtype))
    out = _QDQOutputGrad.apply(out, layer.outputs_grad_scale._value, layer.outputs_grad_amax_history._value, compute)
    return out if bias is None else (out, False)


def set_quantized_policy(layer, mode):
    from keras_b200 import dtype_policies
    from keras_b200.dtype_policies.dtype_policy_map import DTypePolicyMap

    if layer.dtype_policy.quantization_mode is None:
        source = layer._resolved_policy().name
        policy = dtype_policies.get(f"{mode}_from_{source}")
        if isinstance(layer._dtype_policy, DTypePolicyMap) and layer.path:
            layer._dtype_policy[layer.path] = policy
        else:
            layer._dtype_policy = policy


ALL_OBJECTS = [Quantizer, AbsMaxQuantizer]
_LOOKUP = {c.__name__: c for c in ALL_OBJECTS}
_LOOKUP.update({"abs_max_quantizer": AbsMaxQuantizer})


@keras_export("keras.quantizers.serialize")
def serialize(quantizer):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(quantizer)


@keras_export("keras.quantizers.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=_LOOKUP, custom_objects=custom_objects)


@keras_export("keras.quantizers.get")
def get(identifier, **kwargs):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        obj = _LOOKUP.get(identifier)
    else:
        obj = identifier
    if callable(obj):
        return obj(**kwargs) if isinstance(obj, type) else obj
    raise ValueError(f"Could not interpret quantizer identifier: {identifier}")

from keras_b200.quantizers.report import QuantizationReport  # noqa: F401,E402
