"""``TernaryDense``: dense layer trained with {-1, 0, +1} weights through a straight-through estimator and
stored at ~1.6 bits/weight after ``quantize("ternary")`` (keras/src/layers/core/ternary_dense.py)."""

from keras_b200 import activations, constraints, initializers, ops, quantizers, regularizers
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.TernaryDense")
class TernaryDense(Layer):
    def __init__(self, units, threshold=None, activation=None, use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros",
                 kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None, kernel_constraint=None, bias_constraint=None, **kwargs):
        if not isinstance(units, int) or units <= 0:
            raise ValueError(f"Received an invalid value for `units`, expected a positive integer. Received: units={units}")
        if threshold is not None and not isinstance(threshold, (int, float)):
            raise ValueError(f"Received an invalid value for `threshold`, expected a float or None. Received: threshold={threshold}")
        if threshold is not None and threshold < 0:
            raise ValueError(f"Received an invalid value for `threshold`, expected a non-negative float or None. Received: threshold={threshold}")
        super().__init__(activity_regularizer=activity_regularizer, **kwargs)
        self.units, self.threshold = units, threshold
        self.activation = activations.get(activation)
        self.use_bias = use_bias
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.input_spec = InputSpec(min_ndim=2)
        self.supports_masking = True

    def build(self, input_shape):
        input_dim = input_shape[-1]
        kernel_shape = (input_dim, self.units)
        if self.quantization_mode:
            self.quantized_build(kernel_shape, mode=self.quantization_mode)
        else:
            self.kernel = self.add_weight(name="kernel", shape=kernel_shape, initializer=self.kernel_initializer,
                                          regularizer=self.kernel_regularizer, constraint=self.kernel_constraint)
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.units,), initializer=self.bias_initializer, regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint)
        else:
            self.bias = None
        self.input_spec = InputSpec(min_ndim=2, axes={-1: input_dim})
        self.built = True

    def _ternary_kernel(self):
        k = ops.convert_to_tensor(self.kernel)
        abs_k = ops.abs(k)
        t = 0.5 * ops.mean(abs_k) if self.threshold is None else self.threshold
        k_ternary = ops.sign(k) * ops.cast(abs_k > t, dtype=k.dtype)
        return k + ops.stop_gradient(k_ternary - k)  # straight-through estimator

    def call(self, inputs):
        x = ops.matmul(inputs, self._ternary_kernel())
        if self.threshold is None:
            x = ops.multiply(x, ops.mean(ops.abs(self.kernel)))
        if self.bias is not None:
            x = ops.add(x, self.bias)
        if self.activation is not None:
            x = self.activation(x)
        return x

    def quantized_build(self, kernel_shape, mode):
        if mode != "ternary":
            raise self._quantization_mode_error(mode)
        input_dim, units = kernel_shape
        self._packed_kernel = self.add_weight(name="kernel", shape=((input_dim + 4) // 5, units), initializer=initializers.Constant(121),
                                              dtype="uint8", trainable=False)
        self.kernel_scale = self.add_weight(name="kernel_scale", shape=(), initializer="ones", trainable=False)
        self._orig_input_dim = input_dim
        self._is_quantized = True

    def quantized_call(self, *args, **kwargs):
        if self.quantization_mode != "ternary":
            raise self._quantization_mode_error(self.quantization_mode)
        return self._ternary_call(*args, **kwargs)

    def _ternary_call(self, inputs):
        k = quantizers.unpack_ternary(self._packed_kernel, self._orig_input_dim, axis=0)
        x = ops.matmul(inputs, ops.cast(k, self.compute_dtype))
        x = ops.multiply(x, ops.cast(self.kernel_scale, self.compute_dtype))
        if self.bias is not None:
            x = ops.add(x, self.bias)
        if self.activation is not None:
            x = self.activation(x)
        return x

    def quantize(self, mode="ternary", type_check=True, config=None):
        if type_check and type(self) is not TernaryDense:
            raise self._not_implemented_error(self.quantize)
        if mode != "ternary":
            raise self._quantization_mode_error(mode)
        kernel_shape = tuple(self.kernel.shape)
        kernel_ternary = ops.convert_to_numpy(self._ternary_kernel())
        beta = float(ops.convert_to_numpy(ops.mean(ops.abs(self.kernel)))) if self.threshold is None else 1.0
        packed, _, _ = quantizers.pack_ternary(kernel_ternary, axis=0)
        self._tracker_unlock()
        self._untrack_variable(self.kernel)
        del self.kernel
        self.quantized_build(kernel_shape, mode=mode)
        self._lock_state()
        self._packed_kernel.assign(packed)
        self.kernel_scale.assign(beta)
        if self.dtype_policy.quantization_mode is None:
            from keras_b200 import dtype_policies

            self.dtype_policy = dtype_policies.get(f"ternary_from_{self.dtype_policy.name}")

    @property
    def variable_serialization_spec(self):
        return {None: ["kernel", "bias"], "ternary": ["kernel", "bias", "kernel_scale"]}

    def _serialization_targets(self, mode):
        return {"kernel": self._packed_kernel if mode == "ternary" else self.kernel, "bias": self.bias,
                "kernel_scale": getattr(self, "kernel_scale", None)}

    def save_own_variables(self, store):
        if not self.built:
            return
        mode = self.quantization_mode
        if mode not in self.variable_serialization_spec:
            raise self._quantization_mode_error(mode)
        targets = self._serialization_targets(mode)
        idx = 0
        for name in self.variable_serialization_spec[mode]:
            if name == "bias" and self.bias is None:
                continue
            store[str(idx)] = targets[name]
            idx += 1

    def load_own_variables(self, store):
        if not self.built:
            return
        mode = self.quantization_mode
        if mode not in self.variable_serialization_spec:
            raise self._quantization_mode_error(mode)
        targets = self._serialization_targets(mode)
        idx = 0
        for name in self.variable_serialization_spec[mode]:
            if name == "bias" and self.bias is None:
                continue
            targets[name].assign(store[str(idx)])
            idx += 1

    def compute_output_shape(self, input_shape):
        out = list(input_shape)
        out[-1] = self.units
        return tuple(out)

    def get_config(self):
        return {**super().get_config(), "units": self.units, "threshold": self.threshold, "activation": activations.serialize(self.activation),
                "use_bias": self.use_bias, "kernel_initializer": initializers.serialize(self.kernel_initializer),
                "bias_initializer": initializers.serialize(self.bias_initializer),
                "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
                "bias_regularizer": regularizers.serialize(self.bias_regularizer),
                "activity_regularizer": regularizers.serialize(self.activity_regularizer),
                "kernel_constraint": constraints.serialize(self.kernel_constraint), "bias_constraint": constraints.serialize(self.bias_constraint)}
