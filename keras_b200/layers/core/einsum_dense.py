"""``EinsumDense``: a dense layer over an einsum equation.

Behaviour of keras/src/layers/core/einsum_dense.py: kernel/bias shapes are derived from the
equation (:1700-1900), VarianceScaling initialisers receive explicit input/output axes
(:165-199), LoRA, int8 and float8 modes.  Equations that are a plain contraction of trailing
input axes with leading kernel axes lower to one GEMM without permute copies.
"""

import re
import string

import torch

from keras_b200 import activations, constraints, initializers, ops, quantizers, regularizers
from keras_b200.core.export_registry import keras_export
from keras_b200.kernels import dispatch
from keras_b200.layers.core.calibrated_kernel import CalibratedKernel
from keras_b200.layers.layer import Layer


def analyze_einsum(equation, bias_axes, input_shape, output_shape):
    """→ (kernel_shape, bias_shape, full_output_shape, kernel_input_axes, kernel_output_axes)."""
    eq = equation.replace("...", "0")
    left_elided = False
    m = re.fullmatch(r"([a-zA-Z]+),([a-zA-Z]+)->([a-zA-Z]+)", eq)
    if not m:
        m = re.fullmatch(r"0([a-zA-Z]+),([a-zA-Z]+)->0([a-zA-Z]+)", eq)
        left_elided = bool(m)
    if not m:
        m = re.fullmatch(r"([a-zA-Z]{2,})0,([a-zA-Z]+)->([a-zA-Z]+)0", eq)
    if not m:
        raise ValueError(
            f"Invalid einsum equation '{equation}'. Equations must be in the form [X],[Y]->[Z], "
            "...[X],[Y]->...[Z], or [X]...,[Y]->[Z]...."
        )
    in_spec, w_spec, out_spec = m.group(1), m.group(2), m.group(3)
    elided = len(input_shape) - len(in_spec)
    full_out = [input_shape[0]] + ([output_shape] if isinstance(output_shape, int) else list(output_shape))
    if elided > 0 and left_elided:
        for i in range(1, elided):
            full_out.insert(1, input_shape[i])
    elif elided > 0:
        full_out.extend(input_shape[len(input_shape) - elided:])
    if left_elided:
        in_pos = {c: (i + elided) - len(input_shape) for i, c in enumerate(in_spec)}
        out_pos = {c: i + elided for i, c in enumerate(out_spec)}
    else:
        in_pos = {c: i for i, c in enumerate(in_spec)}
        out_pos = {c: i for i, c in enumerate(out_spec)}
    for c in in_spec:
        if c in out_pos:
            o = full_out[out_pos[c]]
            if o is not None and o != input_shape[in_pos[c]]:
                raise ValueError(
                    f"Input shape and output shape do not match at shared dimension '{c}'. Input shape is "
                    f"{input_shape[in_pos[c]]}, and output shape is {o}."
                )
    for c in out_spec:
        if c not in in_spec and c not in w_spec:
            raise ValueError(
                f"Dimension '{c}' was specified in the output '{out_spec}' but has no corresponding dim in the "
                f"input spec '{in_spec}' or weight spec '{out_spec}'"
            )
    kernel_shape, in_axes, out_axes = [], [], []
    for i, c in enumerate(w_spec):
        if c in out_pos:
            kernel_shape.append(full_out[out_pos[c]])
            out_axes.append(i)
        elif c in in_pos:
            kernel_shape.append(input_shape[in_pos[c]])
            in_axes.append(i)
        else:
            raise ValueError(
                f"Weight dimension '{c}' did not have a match in either the input spec '{in_spec}' or the output "
                f"spec '{out_spec}'. For this layer, the weight must be fully specified."
            )
    bias_shape = None
    if bias_axes is not None:
        shift = elided if left_elided else 0
        sizes = {c: full_out[i + shift] for i, c in enumerate(out_spec)}
        for c in bias_axes:
            if c not in out_spec:
                raise ValueError(f"Bias dimension '{c}' was requested, but is not part of the output spec '{out_spec}'")
        first = min(out_spec.find(c) for c in bias_axes)
        bias_shape = [sizes[c] if c in bias_axes else 1 for c in out_spec[first:]]
        if not left_elided:
            bias_shape.extend([1] * elided)
    return kernel_shape, bias_shape, full_out, in_axes, out_axes


def _gemm_plan(equation):
    """Detect ``<batch...><k...>,<k...><n...>-><batch...><n...>``: one GEMM, no permutes."""
    eq = equation.replace("...", "")
    m = re.fullmatch(r"([a-zA-Z]+),([a-zA-Z]+)->([a-zA-Z]+)", eq)
    if not m:
        return None
    a, w, o = m.groups()
    k = [c for c in w if c in a and c not in o]
    n = [c for c in w if c not in a]
    if not k or not n or w != "".join(k) + "".join(n):
        return None
    if not a.endswith("".join(k)):
        return None
    batch = a[: len(a) - len(k)]
    if o != batch + "".join(n):
        return None
    if any(c in w for c in batch):
        return None
    return len(k), len(n)


def scale_alignment(equation, input_rank):
    """Where each axis of the layer's output comes from in the kernel: a list over output axes of the kernel axis with the same
    label, or ``None``.  A quantised kernel's scale is stored with the output's rank (size 1 where the kernel has no such axis)
    so that it broadcasts against the product; files written by keras/src/layers/core/einsum_dense.py:1449-1491 have that
    shape."""
    eq = equation.replace("...", "0")
    left = right = 0
    m = re.fullmatch(r"([a-zA-Z]+),([a-zA-Z]+)->([a-zA-Z]+)", eq)
    if m is None:
        m = re.fullmatch(r"0([a-zA-Z]+),([a-zA-Z]+)->0([a-zA-Z]+)", eq)
        if m is not None:
            left = input_rank - len(m.group(1))
        else:
            m = re.fullmatch(r"([a-zA-Z]{2,})0,([a-zA-Z]+)->([a-zA-Z]+)0", eq)
            if m is None:
                raise ValueError(f"Invalid einsum equation '{equation}'.")
            right = input_rank - len(m.group(1))
    w_spec, out_spec = m.group(2), m.group(3)
    return [None] * left + [w_spec.index(c) if c in w_spec else None for c in out_spec] + [None] * right


def input_alignment(equation, input_rank):
    """``(contracted input axes, per output axis the input axis with the same label or None, equation of the input
    gradient)`` with the ellipsis written out."""
    eq = equation.replace("...", "0")
    m = re.fullmatch(r"([a-zA-Z]+),([a-zA-Z]+)->([a-zA-Z]+)", eq)
    in_spec = w_spec = out_spec = None
    if m is not None:
        in_spec, w_spec, out_spec = m.groups()
    else:
        m = re.fullmatch(r"0([a-zA-Z]+),([a-zA-Z]+)->0([a-zA-Z]+)", eq)
        side = "left"
        if m is None:
            m = re.fullmatch(r"([a-zA-Z]{2,})0,([a-zA-Z]+)->([a-zA-Z]+)0", eq)
            side = "right"
        if m is None:
            raise ValueError(f"Invalid einsum equation '{equation}'.")
        in_spec, w_spec, out_spec = m.groups()
        spare = [c for c in "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ" if c not in in_spec + w_spec + out_spec]
        extra = "".join(spare[: input_rank - len(in_spec)])
        in_spec, out_spec = (extra + in_spec, extra + out_spec) if side == "left" else (in_spec + extra, out_spec + extra)
    contracted = [i for i, c in enumerate(in_spec) if c not in out_spec]
    from_output = [in_spec.index(c) if c in in_spec else None for c in out_spec]
    return contracted, from_output, f"{out_spec},{w_spec}->{in_spec}"


class _Int8Einsum(torch.autograd.Function):
    """einsum of activations quantised at call time (abs-max over the contracted axes) with an int8 kernel, de-scaled; the
    gradient reaches the activations through the de-quantised kernel (keras/src/layers/core/einsum_dense.py:1055-1085)."""

    @staticmethod
    def forward(ctx, inputs, kernel, scale_for_output, scale_for_kernel, equation, contracted, from_output, grad_equation, quantizer):
        q, in_scale = quantizer(inputs, axis=tuple(contracted))
        kept = [a for a in from_output if a is not None]
        rest = [a for a in range(in_scale.ndim) if a not in kept]
        aligned = in_scale.permute(kept + rest).reshape([1 if a is None else inputs.shape[a] for a in from_output])
        if inputs.is_cuda:
            acc = torch.einsum(equation, q.float(), kernel.float())
        else:
            acc = torch.einsum(equation, q.to(torch.int32), kernel.to(torch.int32))
        ctx.save_for_backward(kernel, scale_for_kernel)
        ctx.grad_equation, ctx.compute = grad_equation, inputs.dtype
        return (acc.to(inputs.dtype) / (aligned * scale_for_output.to(inputs.dtype))).to(inputs.dtype)

    @staticmethod
    def backward(ctx, upstream):
        kernel, scale_for_kernel = ctx.saved_tensors
        float_kernel = kernel.to(ctx.compute) / scale_for_kernel.to(ctx.compute)
        return torch.einsum(ctx.grad_equation, upstream, float_kernel), None, None, None, None, None, None, None, None


@keras_export("keras.layers.EinsumDense")
class EinsumDense(CalibratedKernel, Layer):
    def __init__(self, equation, output_shape, activation=None, bias_axes=None, kernel_initializer="glorot_uniform",
                 bias_initializer="zeros", kernel_regularizer=None, bias_regularizer=None, kernel_constraint=None,
                 bias_constraint=None, lora_rank=None, lora_alpha=None, gptq_unpacked_column_size=None,
                 quantization_config=None, **kwargs):
        super().__init__(**kwargs)
        self.equation = equation
        self.partial_output_shape = (output_shape,) if isinstance(output_shape, int) else tuple(output_shape)
        self.bias_axes = bias_axes
        self.activation = activations.get(activation)
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.lora_rank = lora_rank
        self.lora_alpha = lora_alpha if lora_alpha is not None else lora_rank
        self.lora_enabled = False
        self.quantization_config = quantization_config
        self._is_quantized = False
        self._gemm = _gemm_plan(equation)

    def build(self, input_shape):
        kshape, bshape, full_out, in_axes, out_axes = analyze_einsum(self.equation, self.bias_axes, input_shape, self.partial_output_shape)
        self._kernel_shape = tuple(kshape)
        self.full_output_shape = tuple(full_out)
        self._kernel_in_axes, self._kernel_out_axes = in_axes, out_axes
        self._scale_from_output = scale_alignment(self.equation, len(input_shape))
        if self.quantization_mode:
            self.quantized_build(self._kernel_shape, mode=self.quantization_mode)
        if self.quantization_mode not in ("int8", "gptq", "awq"):
            init = self.kernel_initializer
            if isinstance(init, initializers.VarianceScaling):
                base = init

                def init(shape, dtype=None, _b=base):
                    return _b(shape, dtype=dtype, input_axes=in_axes, output_axes=out_axes)

            self._kernel = self.add_weight(name="kernel", shape=self._kernel_shape, initializer=init, regularizer=self.kernel_regularizer,
                                           constraint=self.kernel_constraint, dtype=self.dtype, trainable=True)
        if bshape is not None:
            self.bias = self.add_weight(name="bias", shape=tuple(bshape), initializer=self.bias_initializer, regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint, dtype=self.dtype, trainable=True)
        else:
            self.bias = None
        self.built = True
        if self.lora_rank:
            self.enable_lora(self.lora_rank, lora_alpha=self.lora_alpha)

    @property
    def kernel(self):
        if not self.built:
            raise AttributeError("You must build the layer before accessing `kernel`.")
        if self._calibrated:
            return self._calibrated_matrix().reshape(self._kernel_shape)
        if self.lora_enabled:
            return ops.add(self._kernel.value, (self.lora_alpha / self.lora_rank) * ops.matmul(self.lora_kernel_a.value, self.lora_kernel_b.value))
        return self._kernel

    def compute_output_shape(self, _):
        return self.full_output_shape

    def _contract(self, inputs, kernel, bias=None):
        """einsum(equation, inputs, kernel) lowered to a single GEMM when the equation allows.

        With ``bias`` given, returns ``(output, bias_applied)``: a bias spanning the trailing output dimensions is added
        in the GEMM epilogue."""
        plan = self._gemm
        if plan is not None and isinstance(inputs, torch.Tensor):
            nk, nn = plan
            kv = kernel.value if hasattr(kernel, "value") else kernel
            kdim = 1
            for d in kv.shape[:nk]:
                kdim *= d
            lead = inputs.shape[: inputs.ndim - nk]
            x2 = inputs.reshape(tuple(lead) + (kdim,))
            out_dims = tuple(kv.shape[nk:])
            from keras_b200.kernels import dispatch

            # the Variable itself goes to the GEMM front end, which can then accumulate the weight gradient in place
            source = kernel if hasattr(kernel, "_value") else kv
            bflat = None
            if bias is not None:
                bv = bias.value if hasattr(bias, "value") else bias
                if tuple(bv.shape) == out_dims:
                    bflat = bv.reshape(-1)
            if bias is None or bflat is not None:
                fused = dispatch.dense(x2, source, bflat, None, kernel_shape=(kdim, -1))
                if fused is not None:
                    out = fused[0].reshape(tuple(lead) + out_dims)
                    return out if bias is None else (out, True)
            out = ops.matmul(x2, kv.reshape(kdim, -1)).reshape(tuple(lead) + out_dims)
            return out if bias is None else (out, False)
        out = ops.einsum(self.equation, inputs, kernel)
        return out if bias is None else (out, False)

    def call(self, inputs, training=None):
        if getattr(self._kernel, "_shard_slices", None) is not None:
            from keras_b200.parallel import tensor_parallel

            out = tensor_parallel.einsum_dense(self, inputs)
            if out is not None:
                return out
        if self.bias is not None:
            x, applied = self._contract(inputs, self.kernel, self.bias)
            if not applied:
                x = ops.add(x, self.bias)
        else:
            x = self._contract(inputs, self.kernel)
        if self.activation is not None and self.activation is not activations.linear:
            x = self.activation(x)
        return x

    def enable_lora(self, rank, lora_alpha=None, a_initializer="he_uniform", b_initializer="zeros"):
        if self.kernel_constraint:
            raise ValueError("Lora is incompatible with kernel constraints. In order to enable lora on this layer, remove the `kernel_constraint` argument.")
        if not self.built:
            raise ValueError("Cannot enable lora on a layer that isn't yet built.")
        if self.lora_enabled:
            raise ValueError("lora is already enabled. This can only be done once per layer.")
        self._tracker_unlock()
        self.lora_kernel_a = self.add_weight(name="lora_kernel_a", shape=self._kernel_shape[:-1] + (rank,), initializer=initializers.get(a_initializer), regularizer=self.kernel_regularizer)
        self.lora_kernel_b = self.add_weight(name="lora_kernel_b", shape=(rank, self._kernel_shape[-1]), initializer=initializers.get(b_initializer), regularizer=self.kernel_regularizer)
        self._kernel.trainable = False
        self._lock_state()
        self._invalidate()
        self.lora_enabled = True
        self.lora_rank = rank
        self.lora_alpha = lora_alpha if lora_alpha is not None else rank

    # -- persistence ---------------------------------------------------------------------
    @property
    def variable_serialization_spec(self):
        return {
            None: ["kernel", "bias"],
            "int8": ["kernel", "bias", "kernel_scale"],
            "float8": ["kernel", "bias", "inputs_scale", "inputs_amax_history", "kernel_scale", "kernel_amax_history",
                       "outputs_grad_scale", "outputs_grad_amax_history"],
            **CalibratedKernel.SPEC,
        }

    def _saved_names(self):
        mode = self.quantization_mode if self._is_quantized else None
        if mode not in self.variable_serialization_spec:
            raise self._quantization_mode_error(mode)
        return [n for n in self.variable_serialization_spec[mode] if not (n == "bias" and self.bias is None)]

    def save_own_variables(self, store):
        if not self.built:
            return
        mode = self.quantization_mode if self._is_quantized else None
        if mode in ("gptq", "awq"):
            return self._calibrated_save(store, mode)
        kernel, scale = self._kernel, getattr(self, "kernel_scale", None)
        if self.lora_enabled:
            delta = (self.lora_alpha / self.lora_rank) * torch.matmul(self.lora_kernel_a._value, self.lora_kernel_b._value)
            if mode == "int8":
                full = self._kernel._value.to(torch.float32) / self._scale_for_kernel(self.kernel_scale._value) + delta
                kernel, scale = quantizers.abs_max_quantize(full, axis=self._kernel_in_axes, to_numpy=False)
                scale = self._scale_to_storage(scale)
            else:
                kernel = self._kernel._value + delta.to(self._kernel._value.dtype)
        for i, name in enumerate(self._saved_names()):
            if name == "kernel":
                store[str(i)] = kernel
            elif name == "kernel_scale" and mode == "int8":
                store[str(i)] = scale
            else:
                store[str(i)] = getattr(self, name)

    def load_own_variables(self, store):
        if not self.built:
            return
        if self._is_quantized and self.quantization_mode in ("gptq", "awq"):
            return self._calibrated_load(store, self.quantization_mode)
        names = self._saved_names()
        if len(store.keys()) != len(names):
            raise ValueError(f"Layer '{self.name}' expected {len(names)} variables, but received {len(store.keys())} variables during loading. Expected: {names}")
        for i, name in enumerate(names):
            target = self._kernel if name == "kernel" else getattr(self, name)
            value = store[str(i)]
            if name == "kernel_scale" and tuple(value.shape) != tuple(target.shape):
                value = torch.as_tensor(value).reshape(tuple(target.shape))
            target.assign(value)
        if self.lora_enabled:
            self.lora_kernel_a.assign(torch.zeros_like(self.lora_kernel_a._value))
            self.lora_kernel_b.assign(torch.zeros_like(self.lora_kernel_b._value))

    def get_config(self):
        cfg = {
            "output_shape": self.partial_output_shape, "equation": self.equation, "activation": activations.serialize(self.activation),
            "bias_axes": self.bias_axes, "kernel_initializer": initializers.serialize(self.kernel_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer), "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer), "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint), "bias_constraint": constraints.serialize(self.bias_constraint),
        }
        if self.lora_rank:
            cfg["lora_rank"] = self.lora_rank
            cfg["lora_alpha"] = self.lora_alpha
        return {**super().get_config(), **cfg}

    # -- quantization --------------------------------------------------------------------
    def _scale_storage_shape(self, kernel_shape):
        return tuple(1 if a is None else kernel_shape[a] for a in self._scale_from_output)

    def _scale_to_storage(self, scale):
        """Scale shaped like the kernel (1 on the contracted axes) -> output-aligned storage."""
        kept = [a for a in self._scale_from_output if a is not None]
        rest = [a for a in range(scale.ndim) if a not in kept]
        return scale.permute(kept + rest).reshape(self._scale_storage_shape(self._kernel_shape))

    def _scale_for_kernel(self, stored):
        """Output-aligned storage -> a tensor that broadcasts against the kernel."""
        kept = [a for a in self._scale_from_output if a is not None]
        t = stored.reshape([self._kernel_shape[a] for a in kept])
        t = t.permute([kept.index(a) for a in sorted(kept)])
        return t.reshape([d if i in kept else 1 for i, d in enumerate(self._kernel_shape)])

    def quantized_build(self, kernel_shape, mode, config=None):
        if mode == "int8":
            self._kernel = self.add_weight(name="kernel", shape=kernel_shape, initializer="zeros", dtype="int8", trainable=False)
            self.kernel_scale = self.add_weight(name="kernel_scale", shape=self._scale_storage_shape(kernel_shape), initializer="ones", trainable=False)
        elif mode == "float8":
            quantizers.float8_build(self)
        elif mode in ("gptq", "awq"):
            rows, columns = self.calibrated_matrix_shape(kernel_shape)
            self._calibrated_build(rows, columns, mode, config if config is not None else self.quantization_config)
        else:
            raise self._quantization_mode_error(mode)
        self._is_quantized = True

    @staticmethod
    def calibrated_matrix_shape(kernel_shape):
        """``(input features, output features)`` of a 2-D or 3-D projection kernel.  A 3-D kernel is an attention projection:
        ``[d_model, heads, head_dim]`` (query/key/value) when its largest axis comes first, else ``[heads, head_dim, d_model]``
        (output); the same rule as keras/src/layers/core/einsum_dense.py:669-690."""
        shape = list(kernel_shape)
        if len(shape) == 2:
            return shape[0], shape[1]
        if len(shape) == 3:
            if shape.index(max(shape)) == 0:
                return shape[0], shape[1] * shape[2]
            return shape[0] * shape[1], shape[2]
        raise ValueError(f"Calibrated quantization supports 2-D and 3-D kernels, got shape {tuple(kernel_shape)}.")

    def _calibrated_call(self, inputs):
        if self._calibrated:
            kernel = self._calibrated_matrix(inputs.dtype).reshape(self._kernel_shape)
        else:
            kernel = self._kernel.value
        return self._finish(self._contract(inputs, kernel), inputs)

    def _gptq_call(self, inputs, training=None):
        return self._calibrated_call(inputs)

    def _awq_call(self, inputs, training=None):
        return self._calibrated_call(inputs)

    def _finish(self, x, inputs):
        if self.lora_enabled:
            lora = ops.einsum(self.equation, inputs, ops.matmul(self.lora_kernel_a, self.lora_kernel_b))
            x = ops.add(x, (self.lora_alpha / self.lora_rank) * lora)
        if self.bias is not None:
            x = ops.add(x, ops.cast(self.bias, x.dtype))
        if self.activation is not None:
            x = self.activation(x)
        return x

    def _int8_call(self, inputs, training=None):
        plan = self._gemm
        kv = self._kernel.value
        if plan is not None and isinstance(inputs, torch.Tensor) and inputs.dtype in (torch.float32, torch.bfloat16, torch.float16):
            # The contraction is one GEMM over the flattened input axes: activations are quantised per row over those axes
            # at run time and the product runs on int8 operands (keras/src/layers/core/einsum_dense.py:1071-1085).
            nk = plan[0]
            kdim = 1
            for d in kv.shape[:nk]:
                kdim *= d
            lead = inputs.shape[: inputs.ndim - nk]
            quantizer = getattr(self, "inputs_quantizer", None)
            if quantizer is None:
                quantizer = self.inputs_quantizer = quantizers.AbsMaxQuantizer(axis=-1)
            x2 = inputs.reshape(tuple(lead) + (kdim,))
            flat_bias = self.bias is None or tuple(self.bias.shape) == tuple(kv.shape[nk:])
            if inputs.is_cuda and not self.lora_enabled and flat_bias:
                from keras_b200.kernels import dispatch

                act = self.activation
                fused = dispatch.int8_dense(x2, kv.reshape(kdim, -1), self.kernel_scale.value.reshape(-1), quantizer,
                                            self.bias._value if self.bias is not None else None, getattr(act, "__name__", None))
                if fused is not None:
                    out, act_done = fused
                    out = out.reshape(tuple(lead) + tuple(kv.shape[nk:]))
                    return out if act_done or act is None else act(out)
            out = quantizers.int8_dense_forward(x2, kv.reshape(kdim, -1), self.kernel_scale.value.reshape(-1), quantizer)
            return self._finish(out.reshape(tuple(lead) + tuple(kv.shape[nk:])), inputs)
        if isinstance(inputs, torch.Tensor) and inputs.dtype in (torch.float32, torch.bfloat16, torch.float16):
            # any other equation: the same arithmetic through einsum on the integer codes
            quantizer = getattr(self, "inputs_quantizer", None)
            if quantizer is None:
                quantizer = self.inputs_quantizer = quantizers.AbsMaxQuantizer(axis=-1)
            contracted, from_output, grad_equation = input_alignment(self.equation, inputs.ndim)
            stored = self.kernel_scale.value
            out = _Int8Einsum.apply(inputs, kv, stored, self._scale_for_kernel(stored), self.equation, contracted, from_output, grad_equation, quantizer)
            return self._finish(out, inputs)
        # symbolic inputs: de-quantise the kernel and contract in the compute dtype
        kernel = kv.to(inputs.dtype) / self._scale_for_kernel(self.kernel_scale.value).to(inputs.dtype)
        return self._finish(self._contract(inputs, kernel.detach()), inputs)

    def _float8_call(self, inputs, training=None):
        if self.lora_enabled:
            raise NotImplementedError("Currently, `_float8_call` doesn't support LoRA")
        plan = self._gemm
        kv = self._kernel.value
        if plan is not None:
            nk = plan[0]
            kdim = 1
            for d in kv.shape[:nk]:
                kdim *= d
            lead = inputs.shape[: inputs.ndim - nk]
            x2 = inputs.reshape(tuple(lead) + (kdim,))
            # a bias that spans exactly the kernel's output axes is one vector of the flattened width: the GEMM adds it
            flat_bias = self.bias is not None and tuple(self.bias.shape) == tuple(kv.shape[nk:])
            if flat_bias:
                out, bias_added = quantizers.float8_matmul(self, x2, kv.reshape(kdim, -1), None, training, bias=self.bias)
                out = out.reshape(tuple(lead) + tuple(kv.shape[nk:]))
                if bias_added:
                    return out if self.activation is None else self.activation(out)
            else:
                out = quantizers.float8_matmul(self, x2, kv.reshape(kdim, -1), None, training)
                out = out.reshape(tuple(lead) + tuple(kv.shape[nk:]))
        else:
            out = quantizers.float8_matmul(self, inputs, kv, self.equation, training)
        return self._finish(out, inputs)

    def quantize(self, mode=None, type_check=True, config=None):
        if type_check and type(self) is not EinsumDense:
            raise self._not_implemented_error(self.quantize)
        self.quantization_config = config
        kernel_shape = tuple(self._kernel.shape)
        if mode == "int8":
            q, scale = quantizers.abs_max_quantize(self._kernel._value, axis=tuple(self._kernel_in_axes), to_numpy=False)
            self._untrack_variable(self._kernel)
            del self._kernel
            self.quantized_build(kernel_shape, mode)
            self._kernel.assign(q)
            self.kernel_scale.assign(self._scale_to_storage(scale))
        elif mode == "float8":
            self.quantized_build(kernel_shape, mode)
        elif mode in ("gptq", "awq"):
            if self.lora_enabled:
                raise NotImplementedError(f"lora is not currently supported with {mode.upper()} quantization.")
            self.quantized_build(kernel_shape, mode, config)  # the float kernel stays until calibration replaces it
            mode = config.dtype_policy_string()
        else:
            raise self._quantization_mode_error(mode)
        quantizers.set_quantized_policy(self, mode)
