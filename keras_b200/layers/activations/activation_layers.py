"""Activation layers (keras/src/layers/activations/*.py)."""

import torch

from keras_b200 import activations, constraints, initializers, ops, regularizers
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.Activation")
class Activation(Layer):
    def __init__(self, activation, **kwargs):
        super().__init__(**kwargs)
        self.supports_masking = True
        self.activation = activations.get(activation)
        self.built = True

    def call(self, inputs):
        return self.activation(inputs)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "activation": activations.serialize(self.activation)}


@keras_export("keras.layers.ReLU")
class ReLU(Layer):
    def __init__(self, max_value=None, negative_slope=0.0, threshold=0.0, **kwargs):
        super().__init__(**kwargs)
        if max_value is not None and max_value < 0.0:
            raise ValueError(f"max_value of a ReLU layer cannot be a negative value. Received: max_value={max_value}")
        if negative_slope is None or negative_slope < 0.0:
            raise ValueError(f"negative_slope of a ReLU layer cannot be a negative value. Received: negative_slope={negative_slope}")
        if threshold is None or threshold < 0.0:
            raise ValueError(f"threshold of a ReLU layer cannot be a negative value. Received: threshold={threshold}")
        self.max_value, self.negative_slope, self.threshold = max_value, negative_slope, threshold
        self.supports_masking = True
        self.built = True

    def call(self, inputs):
        return activations.relu(inputs, negative_slope=self.negative_slope, max_value=self.max_value, threshold=self.threshold)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "max_value": self.max_value, "negative_slope": self.negative_slope, "threshold": self.threshold}


@keras_export("keras.layers.LeakyReLU")
class LeakyReLU(Layer):
    def __init__(self, negative_slope=0.3, **kwargs):
        if "alpha" in kwargs:
            negative_slope = kwargs.pop("alpha")
        super().__init__(**kwargs)
        if negative_slope is None or negative_slope < 0:
            raise ValueError(f"The negative_slope value of a Leaky ReLU layer cannot be None or negative value. Expected a float. Received: negative_slope={negative_slope}")
        self.negative_slope = negative_slope
        self.supports_masking = True
        self.built = True

    def call(self, inputs):
        return activations.leaky_relu(inputs, negative_slope=self.negative_slope)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "negative_slope": self.negative_slope}


@keras_export("keras.layers.ELU")
class ELU(Layer):
    def __init__(self, alpha=1.0, **kwargs):
        super().__init__(**kwargs)
        self.alpha = alpha
        self.supports_masking = True
        self.built = True

    def call(self, inputs):
        return activations.elu(inputs, alpha=self.alpha)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "alpha": self.alpha}


@keras_export("keras.layers.PReLU")
class PReLU(Layer):
    def __init__(self, alpha_initializer="Zeros", alpha_regularizer=None, alpha_constraint=None, shared_axes=None, **kwargs):
        super().__init__(**kwargs)
        self.supports_masking = True
        self.alpha_initializer = initializers.get(alpha_initializer)
        self.alpha_regularizer = regularizers.get(alpha_regularizer)
        self.alpha_constraint = constraints.get(alpha_constraint)
        if shared_axes is None:
            self.shared_axes = None
        elif not isinstance(shared_axes, (list, tuple)):
            self.shared_axes = [shared_axes]
        else:
            self.shared_axes = list(shared_axes)

    def build(self, input_shape):
        param_shape = list(input_shape[1:])
        if self.shared_axes is not None:
            for i in self.shared_axes:
                param_shape[i - 1] = 1
        self.alpha = self.add_weight(shape=param_shape, name="alpha", initializer=self.alpha_initializer, regularizer=self.alpha_regularizer, constraint=self.alpha_constraint)
        axes = {}
        if self.shared_axes:
            for i in range(1, len(input_shape)):
                if i not in self.shared_axes:
                    axes[i] = input_shape[i]
        self.input_spec = InputSpec(ndim=len(input_shape), axes=axes)
        self.built = True

    def call(self, inputs):
        pos = activations.relu(inputs)
        neg = -self.alpha * activations.relu(-inputs)
        return pos + neg

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "alpha_initializer": initializers.serialize(self.alpha_initializer),
                "alpha_regularizer": regularizers.serialize(self.alpha_regularizer),
                "alpha_constraint": constraints.serialize(self.alpha_constraint), "shared_axes": self.shared_axes}


@keras_export("keras.layers.Softmax")
class Softmax(Layer):
    def __init__(self, axis=-1, **kwargs):
        super().__init__(**kwargs)
        self.axis = axis
        self.supports_masking = True
        self.built = True

    def call(self, inputs, mask=None):
        if mask is not None and isinstance(inputs, torch.Tensor) and inputs.is_cuda and isinstance(mask, torch.Tensor):
            fused = self._masked_on_device(inputs, mask)
            if fused is not None:
                return fused
        if mask is not None:
            # large negative instead of -inf so that fully masked rows do not produce NaN
            big = -3e4 if inputs.dtype == torch.float16 else -1e9
            inputs = inputs + (1.0 - ops.cast(mask, inputs.dtype)) * big
        if isinstance(self.axis, (tuple, list)):
            if len(self.axis) > 1:
                out = ops.softmax(inputs, axis=tuple(self.axis))
            else:
                out = activations.softmax(inputs, axis=self.axis[0])
        else:
            out = activations.softmax(inputs, axis=self.axis)
        if mask is not None:
            out = ops.multiply(out, ops.cast(mask, out.dtype))
        return out

    def _masked_on_device(self, inputs, mask):
        """Mask, softmax over the last axis and the final multiplication by the mask in one kernel plus one multiply."""
        from keras_b200.kernels import dispatch

        axis = self.axis[0] if isinstance(self.axis, (tuple, list)) and len(self.axis) == 1 else self.axis
        if not isinstance(axis, int) or axis % inputs.ndim != inputs.ndim - 1:
            return None
        keep = mask if mask.dtype == torch.bool else mask != 0
        try:
            keep = keep.expand(inputs.shape)
        except RuntimeError:
            return None
        out = dispatch.softmax(inputs, mask=keep, masked_add=-3e4 if inputs.dtype == torch.float16 else -1e9)
        if out is None:
            return None
        return out * keep.to(out.dtype)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "axis": self.axis}
