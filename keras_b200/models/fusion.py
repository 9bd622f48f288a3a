"""Graph-level fusion for ``Functional`` models.

The executor of a ``Functional`` walks its nodes in order; this module finds, once per model,
the node patterns that a single sm_100a kernel can execute:

* ``BatchNormalization → ReLU``                         → BN apply with fused ReLU
* ``BatchNormalization → Add(other) [→ ReLU]``          → BN apply with fused residual add (and ReLU)

(the residual bottleneck of keras/src/applications/resnet.py:219-273 is conv→BN→ReLU ×2, conv→BN,
Add, ReLU).  A fused BN is *deferred*: its node records the input, and the kernel runs when the
consumer node is reached so the residual operand is available.  Patterns only fire on CUDA tensors
with a channels-last BN; otherwise execution is node by node as written.
"""

import torch

from keras_b200.layers.activations.activation_layers import Activation, ReLU
from keras_b200.layers.merging.merging_layers import Add
from keras_b200.layers.normalization.normalization_layers import BatchNormalization


class Deferred:
    __slots__ = ("layer", "x", "pre_bias", "stats", "shape", "dtype", "device", "ndim")

    def __init__(self, layer, x, pre_bias=None, stats=None):
        self.layer, self.x, self.pre_bias, self.stats = layer, x, pre_bias, stats
        self.shape, self.dtype, self.device, self.ndim = x.shape, x.dtype, x.device, x.ndim


class Padded:
    """Input of a folded ZeroPadding2D: the consumer applies ``pairs`` itself."""

    __slots__ = ("x", "pairs")

    def __init__(self, x, pairs):
        self.x, self.pairs = x, pairs


class NoBias:
    """Output of a convolution whose bias add was folded into the following BatchNormalization."""

    __slots__ = ("x", "bias", "stats")

    def __init__(self, x, bias, stats=None):
        self.x, self.bias, self.stats = x, bias, stats


def _is_relu(op):
    if isinstance(op, ReLU):
        return op.max_value is None and op.negative_slope == 0.0 and op.threshold == 0.0
    if isinstance(op, Activation):
        return getattr(op.activation, "__name__", "") == "relu"
    return False


def build_plan(function):
    """Return {id(node): role} with roles 'defer_bn', 'consume_add', 'consume_relu', 'maybe_identity'."""
    nodes = function._ordered_nodes()
    in_graph = set(id(n) for n in nodes)
    consumers = {}
    for n in nodes:
        for t in n.input_tensors:
            consumers.setdefault(id(t), []).append(n)
    output_ids = {id(t) for t in function._outputs}
    plan = {}
    for n in nodes:
        op = n.operation
        if not isinstance(op, BatchNormalization) or op.renorm or op.synchronized or len(n.outputs) != 1:
            continue
        out = n.outputs[0]
        if id(out) in output_ids:
            continue
        cons = consumers.get(id(out), [])
        if len(cons) != 1:
            continue
        c = cons[0]
        if plan.get(id(c)) in ("consume_add", "consume_add_relu"):
            # second BN operand of an already planned Add: deferred too, so that its producing convolution can
            # drop its bias; the executor materialises it before the fused BN+Add of the first operand
            plan[id(n)] = "defer_bn"
            continue
        if id(c) in plan:
            continue
        if _is_relu(c.operation) and len(c.input_tensors) == 1:
            plan[id(n)] = "defer_bn"
            plan[id(c)] = "consume_relu"
        elif isinstance(c.operation, Add) and len(c.input_tensors) == 2 and len(c.outputs) == 1:
            other = [t for t in c.input_tensors if t is not out]
            if len(other) != 1 or tuple(other[0].shape) != tuple(out.shape):
                continue
            plan[id(n)] = "defer_bn"
            plan[id(c)] = "consume_add"
            add_out = c.outputs[0]
            cc = consumers.get(id(add_out), [])
            if id(add_out) not in output_ids and len(cc) == 1 and _is_relu(cc[0].operation) and id(cc[0]) not in plan:
                plan[id(c)] = "consume_add_relu"
                plan[id(cc[0])] = "identity"
    # Convolution bias feeding a fused BN: the normalised output does not depend on it (training
    # mode) and its gradient is exactly zero, so the add and the bias-gradient reduction are dropped;
    # the bias only enters the moving-mean update (and the shift in inference mode).
    from keras_b200.layers.convolutional.base_conv import BaseConv

    producers = {}
    for n in nodes:
        for t in n.outputs:
            producers[id(t)] = n
    for n in nodes:
        if plan.get(id(n)) != "defer_bn":
            continue
        src = producers.get(id(n.input_tensors[0]))
        if src is None or id(src) in plan:
            continue
        op = src.operation
        if not isinstance(op, BaseConv) or op.lora_enabled or op.data_format != "channels_last":
            continue
        if getattr(op.activation, "__name__", "linear") != "linear" or op.activity_regularizer is not None:
            continue
        out = src.outputs[0]
        if id(out) in output_ids or len(consumers.get(id(out), [])) != 1 or len(src.input_tensors) != 1:
            continue
        if n.operation.axis % len(out.shape) != len(out.shape) - 1:
            continue
        plan[id(src)] = "conv_fold_bias"
    # ZeroPadding2D in front of a max pooling or of a bias-folded convolution ("valid" padding): the padded copy
    # is never made; the pooling kernel and the convolution take the padding as a parameter.
    from keras_b200.layers.pooling.pooling import MaxPooling2D
    from keras_b200.layers.reshaping.reshaping_layers import ZeroPadding2D

    for n in nodes:
        op = n.operation
        if not isinstance(op, ZeroPadding2D) or op.data_format != "channels_last" or id(n) in plan or len(n.input_tensors) != 1:
            continue
        out = n.outputs[0]
        cons = consumers.get(id(out), [])
        if id(out) in output_ids or len(cons) != 1:
            continue
        c = cons[0]
        cop = c.operation
        if isinstance(cop, MaxPooling2D) and cop.padding == "valid" and cop.data_format == "channels_last" and id(c) not in plan:
            plan[id(n)] = "pad_fold"
            plan[id(c)] = "pool_padded"
        elif plan.get(id(c)) == "conv_fold_bias" and cop.rank == 2 and cop.padding == "valid" and all(lo == hi for lo, hi in op.padding):
            plan[id(n)] = "pad_fold"
    # Activations read by exactly two consumers that can share one gradient buffer (kernels/grad_merge.py): a bias-folded
    # convolution reading the tensor itself, plus either a second such convolution (projection shortcut) or the fused
    # BatchNorm+Add that takes the tensor as its residual operand (identity shortcut).
    merge = set()
    for n in nodes:
        for out in n.outputs:
            cons = consumers.get(id(out), [])
            if id(out) in output_ids or len(cons) != 2 or cons[0] is cons[1]:
                continue
            kinds = []
            for c in cons:
                role = plan.get(id(c))
                if role == "conv_fold_bias" and len(c.input_tensors) == 1:
                    kinds.append("conv")
                elif role in ("consume_add", "consume_add_relu"):
                    # the residual operand is the one that does not come from a deferred BatchNormalization
                    src = producers.get(id(out))
                    if src is not None and plan.get(id(src)) != "defer_bn":
                        kinds.append("add")
            if sorted(kinds) in (["conv", "conv"], ["add", "conv"]):
                merge.add(id(out))
    plan["merge_tensors"] = merge
    return plan


def run_pool_padded(layer, x, pairs):
    from keras_b200 import ops
    from keras_b200.kernels import dispatch

    out = dispatch.max_pool2d(x, layer.pool_size, layer.strides, "valid", zero_pad=pairs)
    if out is not None:
        return out
    pads = [(0, 0), tuple(pairs[0]), tuple(pairs[1]), (0, 0)]
    return layer(ops.pad(x, pads))


def run_conv_nobias(layer, x, pairs=None, want_stats=False):
    """The convolution of ``layer`` without its bias add (autocast applied as ``Layer.__call__`` would).

    ``pairs``: symmetric zero padding of a folded ZeroPadding2D, applied by the convolution itself.
    Returns ``(y, stats)``; ``stats`` holds the per-channel partial sums of ``y`` left by the convolution kernel's
    epilogue when ``want_stats`` is set and that kernel ran (else ``None``)."""
    from keras_b200 import ops
    from keras_b200.core.variables import AutocastScope
    from keras_b200.kernels import conv as kconv

    td = layer._compute_torch_dtype()
    with AutocastScope(layer.compute_dtype):
        if layer.rank == 2 and layer.groups == 1 and type(layer).convolution_op is BaseConvOp():
            padding = layer.padding if pairs is None else tuple(lo for lo, _ in pairs)
            w = layer.kernel.value
            xin = x
            if xin.dtype != td and xin.dtype.is_floating_point and not (xin.dtype == torch.float32 and w.shape[-2] % 8):
                xin = xin.to(td)  # an fp32 input with few channels is cast inside the patch kernel
            out = kconv.conv(xin, w, layer.strides, padding, layer.data_format, layer.dilation_rate, grad_target=layer.kernel, want_stats=want_stats)
            if out is not None:
                return out if want_stats else (out, None)
        if x.dtype != td and x.dtype.is_floating_point:
            x = x.to(td)
        if pairs is None:
            return layer.convolution_op(x, layer.kernel), None
        return ops.conv(x, layer.kernel, strides=list(layer.strides), padding=tuple(lo for lo, _ in pairs),
                        dilation_rate=layer.dilation_rate, data_format=layer.data_format), None


def BaseConvOp():
    from keras_b200.layers.convolutional.base_conv import BaseConv

    return BaseConv.convolution_op


def applicable(x):
    return isinstance(x, torch.Tensor) and x.is_cuda


def run_bn(layer, x, training, residual=None, relu=False, pre_bias=None, stats=None):
    """Execute a (possibly fused) BatchNormalization outside of ``Layer.__call__``."""
    from keras_b200.kernels import dispatch

    train = bool(training) and layer.trainable
    bias_value = pre_bias._value if pre_bias is not None else None
    out = dispatch.batch_norm(layer, x, train, residual=residual, relu=relu, pre_bias=bias_value, conv_stats=stats)
    if out is not None:
        if pre_bias is not None and train:
            # A bias in front of a batch normalization in training mode is removed with the batch mean: its gradient is exactly
            # zero.  The fused kernel never materialises it, so the variable is marked: gradient storage reports a zero
            # gradient for it (the optimizer then treats it as the reference does, weight decay included) instead of none.
            pre_bias._gradient_is_zero_when_absent = True
        return out
    if pre_bias is not None:
        x = x + pre_bias.value.to(x.dtype)
    out = layer(x, training=training)
    if residual is not None:
        out = out + residual
    if relu:
        out = torch.relu(out)
    return out
