"""``TernaryDense``: a dense layer whose kernel acts as {-1, 0, +1} times one scale.

Training keeps a latent float kernel; the forward pass uses its ternarised copy and the backward pass hands the
gradient of that copy to the latent kernel unchanged (straight-through estimator).  ``quantize("ternary")`` drops the
latent kernel and stores five ternary digits per byte plus the scale (about 1.6 bits per weight).  Public behaviour
and the on-disk variable order follow keras/src/layers/core/ternary_dense.py.
"""

import torch

from keras_b200 import activations, constraints, initializers, ops, quantizers, regularizers
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer

_DIGITS_PER_BYTE = 5     # 3^5 = 243 <= 256
_ALL_ZERO_BYTE = 121     # the byte whose five balanced-ternary digits are all 0


class _Ternarise(torch.autograd.Function):
    """w -> sign(w) * [|w| > cut]; the gradient passes through as if the function were the identity."""

    @staticmethod
    def forward(ctx, w, cut):
        return torch.sign(w) * (w.abs() > cut).to(w.dtype)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


@keras_export("keras.layers.TernaryDense")
class TernaryDense(Layer):
    """``threshold=None``: weights below half the mean magnitude become 0 and the output is rescaled by the mean magnitude;
    a number: that fixed cut and no rescaling."""

    def __init__(self, units, threshold=None, activation=None, use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros",
                 kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None, kernel_constraint=None, bias_constraint=None, **kwargs):
        if not isinstance(units, int) or units <= 0:
            raise ValueError(f"Received an invalid value for `units`, expected a positive integer. Received: units={units}")
        if threshold is not None:
            if not isinstance(threshold, (int, float)):
                raise ValueError(f"Received an invalid value for `threshold`, expected a float or None. Received: threshold={threshold}")
            if threshold < 0:
                raise ValueError(f"Received an invalid value for `threshold`, expected a non-negative float or None. Received: threshold={threshold}")
        super().__init__(activity_regularizer=activity_regularizer, **kwargs)
        self.units, self.threshold, self.use_bias = units, threshold, use_bias
        self.activation = activations.get(activation)
        self.kernel_initializer, self.bias_initializer = initializers.get(kernel_initializer), initializers.get(bias_initializer)
        self.kernel_regularizer, self.bias_regularizer = regularizers.get(kernel_regularizer), regularizers.get(bias_regularizer)
        self.kernel_constraint, self.bias_constraint = constraints.get(kernel_constraint), constraints.get(bias_constraint)
        self.input_spec = InputSpec(min_ndim=2)
        self.supports_masking = True

    # -- state ---------------------------------------------------------------------------
    def build(self, input_shape):
        fan_in = input_shape[-1]
        if self.quantization_mode:
            self.quantized_build((fan_in, self.units), mode=self.quantization_mode)
        else:
            self.kernel = self.add_weight(name="kernel", shape=(fan_in, self.units), initializer=self.kernel_initializer,
                                          regularizer=self.kernel_regularizer, constraint=self.kernel_constraint)
        self.bias = None
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.units,), initializer=self.bias_initializer, regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint)
        self.input_spec = InputSpec(min_ndim=2, axes={-1: fan_in})
        self.built = True

    def quantized_build(self, kernel_shape, mode):
        if mode != "ternary":
            raise self._quantization_mode_error(mode)
        fan_in, units = kernel_shape
        packed_rows = -(-fan_in // _DIGITS_PER_BYTE)
        self._packed_kernel = self.add_weight(name="kernel", shape=(packed_rows, units), initializer=initializers.Constant(_ALL_ZERO_BYTE),
                                              dtype="uint8", trainable=False)
        self.kernel_scale = self.add_weight(name="kernel_scale", shape=(), initializer="ones", trainable=False)
        self._orig_input_dim = fan_in
        self._is_quantized = True

    # -- forward -------------------------------------------------------------------------
    def _scale_and_cut(self, latent):
        """(output scale or None, magnitude cut) for the latent kernel."""
        if self.threshold is not None:
            return None, self.threshold
        mean_magnitude = latent.abs().mean()
        return mean_magnitude, 0.5 * mean_magnitude.detach()

    def _ternary_kernel(self):
        latent = ops.convert_to_tensor(self.kernel)
        _, cut = self._scale_and_cut(latent)
        return _Ternarise.apply(latent, cut)

    def _finish(self, x):
        if self.bias is not None:
            x = ops.add(x, self.bias)
        return x if self.activation is None else self.activation(x)

    def call(self, inputs):
        latent = ops.convert_to_tensor(self.kernel)
        scale, cut = self._scale_and_cut(latent)
        x = ops.matmul(inputs, _Ternarise.apply(latent, cut))
        if scale is not None:
            x = ops.multiply(x, scale)
        return self._finish(x)

    def quantized_call(self, *args, **kwargs):
        if self.quantization_mode != "ternary":
            raise self._quantization_mode_error(self.quantization_mode)
        return self._ternary_call(*args, **kwargs)

    def _ternary_call(self, inputs):
        digits = quantizers.unpack_ternary(self._packed_kernel, self._orig_input_dim, axis=0)
        x = ops.matmul(inputs, ops.cast(digits, self.compute_dtype))
        return self._finish(ops.multiply(x, ops.cast(self.kernel_scale, self.compute_dtype)))

    # -- conversion ----------------------------------------------------------------------
    def quantize(self, mode="ternary", type_check=True, config=None):
        if type_check and type(self) is not TernaryDense:
            raise self._not_implemented_error(self.quantize)
        if mode != "ternary":
            raise self._quantization_mode_error(mode)
        latent = ops.convert_to_tensor(self.kernel)
        scale, cut = self._scale_and_cut(latent)
        digits = ops.convert_to_numpy(_Ternarise.apply(latent, cut))
        packed, _, _ = quantizers.pack_ternary(digits, axis=0)
        shape = tuple(self.kernel.shape)
        self._tracker_unlock()
        self._untrack_variable(self.kernel)
        del self.kernel
        self.quantized_build(shape, mode=mode)
        self._lock_state()
        self._packed_kernel.assign(packed)
        self.kernel_scale.assign(1.0 if scale is None else float(ops.convert_to_numpy(scale)))
        if self.dtype_policy.quantization_mode is None:
            from keras_b200 import dtype_policies

            self.dtype_policy = dtype_policies.get(f"ternary_from_{self.dtype_policy.name}")

    # -- persistence ---------------------------------------------------------------------
    @property
    def variable_serialization_spec(self):
        return {None: ["kernel", "bias"], "ternary": ["kernel", "bias", "kernel_scale"]}

    def _stored_variables(self):
        """Variables in on-disk order for the current mode (an absent bias takes no slot)."""
        mode = self.quantization_mode
        if mode not in self.variable_serialization_spec:
            raise self._quantization_mode_error(mode)
        by_name = {"kernel": self._packed_kernel if mode == "ternary" else self.kernel, "bias": self.bias,
                   "kernel_scale": getattr(self, "kernel_scale", None)}
        return [by_name[name] for name in self.variable_serialization_spec[mode] if not (name == "bias" and self.bias is None)]

    def save_own_variables(self, store):
        if self.built:
            for slot, variable in enumerate(self._stored_variables()):
                store[str(slot)] = variable

    def load_own_variables(self, store):
        if self.built:
            for slot, variable in enumerate(self._stored_variables()):
                variable.assign(store[str(slot)])

    def compute_output_shape(self, input_shape):
        return tuple(input_shape[:-1]) + (self.units,)

    def get_config(self):
        config = super().get_config()
        config.update(units=self.units, threshold=self.threshold, activation=activations.serialize(self.activation), use_bias=self.use_bias,
                      kernel_initializer=initializers.serialize(self.kernel_initializer), bias_initializer=initializers.serialize(self.bias_initializer),
                      kernel_regularizer=regularizers.serialize(self.kernel_regularizer), bias_regularizer=regularizers.serialize(self.bias_regularizer),
                      activity_regularizer=regularizers.serialize(self.activity_regularizer),
                      kernel_constraint=constraints.serialize(self.kernel_constraint), bias_constraint=constraints.serialize(self.bias_constraint))
        return config
