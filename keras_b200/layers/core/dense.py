"""``Dense``: ``activation(inputs @ kernel + bias)`` with LoRA and quantized variants.

Behaviour of keras/src/layers/core/dense.py: variables ``kernel (in, units)`` and ``bias
(units,)``; LoRA (:251-312); quantization modes and on-disk variable order (:486-541); int8 path
(:938-986); float8 path with delayed scaling and six fp32 bookkeeping variables (:895-936,
1097-1186).  On a B200 the matmul + bias + activation run as one tcgen05 GEMM with a fused
epilogue (``keras_b200.kernels``).
"""

import torch

from keras_b200 import activations, constraints, initializers, ops, quantizers, regularizers
from keras_b200.core.export_registry import keras_export
from keras_b200.core.variables import Variable
from keras_b200.kernels import dispatch
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.core.calibrated_kernel import CalibratedKernel
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.Dense")
class Dense(CalibratedKernel, Layer):
    def __init__(self, units, activation=None, use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros",
                 kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None, kernel_constraint=None,
                 bias_constraint=None, lora_rank=None, lora_alpha=None, quantization_config=None, **kwargs):
        if not isinstance(units, int) or units <= 0:
            raise ValueError(f"Received an invalid value for `units`, expected a positive integer. Received: units={units}")
        super().__init__(activity_regularizer=activity_regularizer, **kwargs)
        self.units = units
        self.activation = activations.get(activation)
        self.use_bias = use_bias
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
        self.input_spec = InputSpec(min_ndim=2)
        self.supports_masking = True
        self._is_quantized = False

    def build(self, input_shape):
        kernel_shape = (input_shape[-1], self.units)
        if self.quantization_mode:
            self.quantized_build(kernel_shape, mode=self.quantization_mode)
        if self.quantization_mode not in ("int8", "int4", "gptq", "awq"):
            self._kernel = self.add_weight(name="kernel", shape=kernel_shape, initializer=self.kernel_initializer,
                                           regularizer=self.kernel_regularizer, constraint=self.kernel_constraint)
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.units,), initializer=self.bias_initializer,
                                        regularizer=self.bias_regularizer, constraint=self.bias_constraint)
        else:
            self.bias = None
        self.input_spec = InputSpec(min_ndim=2, axes={-1: input_shape[-1]})
        self.built = True
        if self.lora_rank:
            self.enable_lora(self.lora_rank, lora_alpha=self.lora_alpha)

    @property
    def kernel(self):
        if not self.built:
            raise AttributeError("You must build the layer before accessing `kernel`.")
        if self._calibrated:
            return self._calibrated_matrix()
        k = self._kernel
        if self._is_quantized and self.quantization_mode == "int4":
            k = quantizers.unpack_int4(k.value, self._orig_input_dim)
        if self.lora_enabled:
            base = k.value if isinstance(k, Variable) else k
            return ops.add(base, (self.lora_alpha / self.lora_rank) * ops.matmul(self.lora_kernel_a.value, self.lora_kernel_b.value))
        return k

    def call(self, inputs, training=None):
        if getattr(getattr(self, "_kernel", None), "_shard_slices", None) is not None:
            from keras_b200.parallel import tensor_parallel

            out = tensor_parallel.dense(self, inputs)
            if out is not None:
                return out
        kernel = self.kernel
        act = self.activation
        fused = dispatch.dense(inputs, kernel, self.bias, getattr(act, "__name__", None))
        if fused is not None:
            out, act_done = fused
            if not act_done and act is not None and act is not activations.linear:
                out = act(out)
            return out
        x = ops.matmul(inputs, kernel)
        if self.bias is not None:
            x = ops.add(x, self.bias)
        if act is not None and act is not activations.linear:
            x = act(x)
        return x

    def compute_output_shape(self, input_shape):
        out = list(input_shape)
        out[-1] = self.units
        return tuple(out)

    # -- LoRA ----------------------------------------------------------------------------
    def enable_lora(self, rank, lora_alpha=None, a_initializer="he_uniform", b_initializer="zeros"):
        if self.kernel_constraint:
            raise ValueError("Lora is incompatible with kernel constraints. In order to enable lora on this layer, remove the `kernel_constraint` argument.")
        if not self.built:
            raise ValueError("Cannot enable lora on a layer that isn't yet built.")
        if self.lora_enabled:
            raise ValueError("lora is already enabled. This can only be done once per layer.")
        self._tracker_unlock()
        in_dim = self._orig_input_dim if (self.quantization_mode == "int4" and self._is_quantized) else self._kernel.shape[0]
        self.lora_kernel_a = self.add_weight(name="lora_kernel_a", shape=(in_dim, rank), initializer=initializers.get(a_initializer), regularizer=self.kernel_regularizer)
        self.lora_kernel_b = self.add_weight(name="lora_kernel_b", shape=(rank, self.units), initializer=initializers.get(b_initializer), regularizer=self.kernel_regularizer)
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
            "int4": ["kernel", "bias", "kernel_scale"],
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
        if self._is_quantized and self.quantization_mode in ("gptq", "awq"):
            return self._calibrated_save(store, self.quantization_mode)
        kernel_value, merged_scale = self._get_kernel_with_merged_lora()
        mode = self.quantization_mode if self._is_quantized else None
        for i, name in enumerate(self._saved_names()):
            if name == "kernel":
                store[str(i)] = kernel_value
            elif name == "kernel_scale" and mode in ("int8", "int4"):
                store[str(i)] = merged_scale
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
            target.assign(store[str(i)])
        if self.lora_enabled:
            self.lora_kernel_a.assign(torch.zeros_like(self.lora_kernel_a._value))
            self.lora_kernel_b.assign(torch.zeros_like(self.lora_kernel_b._value))

    def _get_kernel_with_merged_lora(self):
        """(kernel value to save, kernel scale to save) with LoRA deltas folded in."""
        scale = getattr(self, "kernel_scale", None)
        if not self.lora_enabled:
            return self._kernel, scale
        delta = (self.lora_alpha / self.lora_rank) * torch.matmul(self.lora_kernel_a._value, self.lora_kernel_b._value)
        if self._is_quantized and self.quantization_mode == "int8":
            full = self._kernel._value.to(torch.float32) / self.kernel_scale._value + delta
            q, s = quantizers.abs_max_quantize(full, axis=0, to_numpy=False)
            return q, s.squeeze(0)
        if self._is_quantized and self.quantization_mode == "int4":
            unpacked = quantizers.unpack_int4(self._kernel._value, self._orig_input_dim)
            full = unpacked.to(torch.float32) / self.kernel_scale._value + delta
            q, s = quantizers.abs_max_quantize(full, axis=0, value_range=(-8, 7), dtype="int8", to_numpy=False)
            packed, _, _ = quantizers.pack_int4(q, axis=0)
            return packed, s.squeeze(0)
        return self._kernel._value + delta.to(self._kernel._value.dtype), scale

    def get_config(self):
        base = super().get_config()
        cfg = {
            "units": self.units,
            "activation": activations.serialize(self.activation),
            "use_bias": self.use_bias,
            "kernel_initializer": initializers.serialize(self.kernel_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer),
            "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint),
            "bias_constraint": constraints.serialize(self.bias_constraint),
        }
        if self.lora_rank:
            cfg["lora_rank"] = self.lora_rank
            cfg["lora_alpha"] = self.lora_alpha
        if self.quantization_config is not None:
            from keras_b200.saving import serialization_lib

            cfg["quantization_config"] = serialization_lib.serialize_keras_object(self.quantization_config)
        return {**base, **cfg}

    # -- quantization --------------------------------------------------------------------
    def quantized_build(self, kernel_shape, mode, config=None):
        if mode == "int8":
            self.inputs_quantizer = quantizers.AbsMaxQuantizer(axis=-1)
            self._kernel = self.add_weight(name="kernel", shape=kernel_shape, initializer="zeros", dtype="int8", trainable=False)
            self.kernel_scale = self.add_weight(name="kernel_scale", shape=(self.units,), initializer="ones", trainable=False)
        elif mode == "int4":
            self.inputs_quantizer = quantizers.AbsMaxQuantizer(axis=-1)
            in_dim, out_dim = kernel_shape
            self._kernel = self.add_weight(name="kernel", shape=((in_dim + 1) // 2, out_dim), initializer="zeros", dtype="int8", trainable=False)
            self.kernel_scale = self.add_weight(name="kernel_scale", shape=(self.units,), initializer="ones", trainable=False)
            self._orig_input_dim = in_dim
        elif mode == "float8":
            quantizers.float8_build(self)
        elif mode in ("gptq", "awq"):
            self._calibrated_build(kernel_shape[0], kernel_shape[1], mode, config if config is not None else self.quantization_config)
        else:
            raise self._quantization_mode_error(mode)
        self._is_quantized = True

    def _calibrated_call(self, inputs):
        kernel = self._calibrated_matrix(inputs.dtype) if self._calibrated else self._kernel.value
        return self._finish(ops.matmul(inputs, kernel), inputs)

    def _gptq_call(self, inputs, training=None):
        return self._calibrated_call(inputs)

    def _awq_call(self, inputs, training=None):
        return self._calibrated_call(inputs)

    def _finish(self, out, inputs):
        if self.lora_enabled:
            lora = ops.matmul(ops.matmul(inputs, self.lora_kernel_a), self.lora_kernel_b)
            out = ops.add(out, (self.lora_alpha / self.lora_rank) * lora)
        if self.bias is not None:
            out = ops.add(out, ops.cast(self.bias, out.dtype))
        if self.activation is not None:
            out = self.activation(out)
        return out

    def _int8_call(self, inputs, training=None):
        if not self.lora_enabled and isinstance(inputs, torch.Tensor) and inputs.is_cuda:
            # inference on the device: quantise the rows, then one GEMM whose epilogue de-scales, adds the bias and activates
            act = self.activation
            fused = dispatch.int8_dense(inputs, self._kernel.value, self.kernel_scale.value, self.inputs_quantizer,
                                        self.bias._value if self.bias is not None else None, getattr(act, "__name__", None))
            if fused is not None:
                out, act_done = fused
                return out if act_done or act is None or act is activations.linear else act(out)
        out = quantizers.int8_dense_forward(inputs, self._kernel.value, self.kernel_scale.value, self.inputs_quantizer)
        return self._finish(out, inputs)

    def _int4_call(self, inputs, training=None):
        unpacked = quantizers.unpack_int4(self._kernel.value, self._orig_input_dim)
        out = quantizers.int8_dense_forward(inputs, unpacked, self.kernel_scale.value, self.inputs_quantizer)
        return self._finish(out, inputs)

    def _float8_call(self, inputs, training=None):
        if self.lora_enabled:
            raise NotImplementedError("Currently, `_float8_call` doesn't support LoRA")
        if self.bias is None:
            return self._finish(quantizers.float8_matmul(self, inputs, self._kernel.value, None, training), inputs)
        out, bias_added = quantizers.float8_matmul(self, inputs, self._kernel.value, None, training, bias=self.bias)
        if not bias_added:
            return self._finish(out, inputs)
        return out if self.activation is None else self.activation(out)

    def quantize(self, mode=None, type_check=True, config=None):
        if type_check and type(self) is not Dense:
            raise self._not_implemented_error(self.quantize)
        self.quantization_config = config
        kernel_shape = tuple(self._kernel.shape)
        if mode in ("int8", "int4"):
            rng = (-127, 127) if mode == "int8" else (-8, 7)
            q, scale = quantizers.abs_max_quantize(self._kernel._value, axis=0, value_range=rng, dtype="int8", to_numpy=False)
            scale = scale.squeeze(0)
            if mode == "int4":
                q, _, _ = quantizers.pack_int4(q, axis=0)
            self._untrack_variable(self._kernel)
            del self._kernel
            self.quantized_build(kernel_shape, mode)
            self._kernel.assign(q)
            self.kernel_scale.assign(scale)
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
