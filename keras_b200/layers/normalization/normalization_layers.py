"""Normalisation layers.

Behaviour: BatchNormalization keras/src/layers/normalization/batch_normalization.py:240-586
(variables gamma, beta, moving_mean, moving_variance, all ``autocast=False``; ≥fp32 compute;
masked moments; renorm), LayerNormalization layer_normalization.py:154-198, RMSNormalization
rms_normalization.py:50-76, GroupNormalization, UnitNormalization, SpectralNormalization.
"""

import torch

from keras_b200 import constraints, initializers, ops, regularizers
from keras_b200.core.dtypes import result_type
from keras_b200.core.export_registry import keras_export
from keras_b200.kernels import dispatch
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer
from keras_b200.layers.core.wrapper import Wrapper


@keras_export("keras.layers.BatchNormalization")
class BatchNormalization(Layer):
    def __init__(self, axis=-1, momentum=0.99, epsilon=1e-3, center=True, scale=True, beta_initializer="zeros", gamma_initializer="ones",
                 moving_mean_initializer="zeros", moving_variance_initializer="ones", beta_regularizer=None, gamma_regularizer=None,
                 beta_constraint=None, gamma_constraint=None, synchronized=False, renorm=False, renorm_clipping=None, renorm_momentum=0.99, **kwargs):
        super().__init__(**kwargs)
        self.axis = int(axis)
        self.synchronized = synchronized
        self.momentum = float(momentum)
        self.epsilon = float(epsilon)
        self.center, self.scale = center, scale
        self.beta_initializer = initializers.get(beta_initializer)
        self.gamma_initializer = initializers.get(gamma_initializer)
        self.moving_mean_initializer = initializers.get(moving_mean_initializer)
        self.moving_variance_initializer = initializers.get(moving_variance_initializer)
        self.beta_regularizer = regularizers.get(beta_regularizer)
        self.gamma_regularizer = regularizers.get(gamma_regularizer)
        self.beta_constraint = constraints.get(beta_constraint)
        self.gamma_constraint = constraints.get(gamma_constraint)
        self.supports_masking = True
        self.renorm = renorm
        if renorm:
            renorm_clipping = renorm_clipping or {}
            keys = ["rmax", "rmin", "dmax"]
            if set(renorm_clipping) - set(keys):
                raise ValueError(f"Received invalid keys for `renorm_clipping` argument: {renorm_clipping}. Supported values: {keys}.")
            rmax, rmin, dmax = renorm_clipping.get("rmax"), renorm_clipping.get("rmin"), renorm_clipping.get("dmax")
            if rmax is not None and rmin is not None and rmax < rmin:
                raise ValueError("rmax should be greater than rmin in the `renorm_clipping` argument. " f"Received: rmax={rmax}, rmin={rmin}.")
            if dmax is not None and dmax < 0:
                raise ValueError(f"dmax should be non-negative in the `renorm_clipping` argument. Received: dmax={dmax}.")
        self.renorm_clipping = renorm_clipping
        self.renorm_momentum = renorm_momentum
        self.gamma = self.beta = self.moving_mean = self.moving_variance = None
        self._reduction_axes = None

    def build(self, input_shape):
        shape = (input_shape[self.axis],)
        if self.scale:
            self.gamma = self.add_weight(shape=shape, name="gamma", initializer=self.gamma_initializer, regularizer=self.gamma_regularizer,
                                         constraint=self.gamma_constraint, trainable=True, autocast=False)
        if self.center:
            self.beta = self.add_weight(shape=shape, name="beta", initializer=self.beta_initializer, regularizer=self.beta_regularizer,
                                        constraint=self.beta_constraint, trainable=True, autocast=False)
        self.moving_mean = self.add_weight(shape=shape, name="moving_mean", initializer=self.moving_mean_initializer, trainable=False, autocast=False)
        self.moving_variance = self.add_weight(shape=shape, name="moving_variance", initializer=self.moving_variance_initializer, trainable=False, autocast=False)
        if self.renorm:
            self.renorm_mean = self.add_weight(shape=shape, name="renorm_mean", initializer=self.moving_mean_initializer, trainable=False, autocast=False)
            self.renorm_stddev = self.add_weight(shape=shape, name="renorm_stddev", initializer=initializers.get("ones"), trainable=False, autocast=False)
        self.input_spec = InputSpec(ndim=len(input_shape), axes={self.axis: input_shape[self.axis]})
        axes = list(range(len(input_shape)))
        del axes[self.axis]
        self._reduction_axes = axes
        self.built = True

    def compute_output_shape(self, input_shape):
        if isinstance(self.axis, int):
            axes = [self.axis]
        else:
            axes = self.axis
        for a in axes:
            if a >= len(input_shape) or a < -len(input_shape):
                raise ValueError(f"Axis {a} is out of bounds for input shape {input_shape}. Received: axis={self.axis}")
        return input_shape

    def call(self, inputs, training=None, mask=None):
        if mask is not None and len(mask.shape) != len(inputs.shape) - 1:
            raise ValueError(f"The mask provided should be one dimension less than the inputs. Received: mask.shape={tuple(mask.shape)}, inputs.shape={tuple(inputs.shape)}")
        input_dtype = inputs.dtype
        train = bool(training) and self.trainable
        if mask is None and not self.renorm and not self.synchronized:
            fused = dispatch.batch_norm(self, inputs, train)
            if fused is not None:
                return fused
        compute = torch.float32 if input_dtype in (torch.float16, torch.bfloat16) else input_dtype
        x = inputs.to(compute) if inputs.dtype != compute else inputs
        moving_mean = self.moving_mean.value.to(compute)
        moving_variance = self.moving_variance.value.to(compute)
        if train:
            mean, variance = self._moments(x, mask)
            if self.synchronized:
                from keras_b200.parallel import collectives

                mean, variance = collectives.sync_batch_moments(mean, variance, x, self._reduction_axes)
            if self.renorm:
                outputs, mean, variance = self._renorm_correction_and_moments(x, mean, variance, training)
                return outputs.to(input_dtype)
            with torch.no_grad():
                self.moving_mean.assign(moving_mean * self.momentum + mean.detach() * (1.0 - self.momentum))
                self.moving_variance.assign(moving_variance * self.momentum + variance.detach() * (1.0 - self.momentum))
        else:
            mean, variance = moving_mean, moving_variance
        gamma = self.gamma.value.to(compute) if self.scale else None
        beta = self.beta.value.to(compute) if self.center else None
        out = ops.batch_normalization(x, mean, variance, axis=self.axis, offset=beta, scale=gamma, epsilon=self.epsilon)
        return out.to(input_dtype)

    def _moments(self, inputs, mask):
        if mask is None:
            return ops.moments(inputs, axes=self._reduction_axes, synchronized=False)
        mask_w = ops.cast(mask, inputs.dtype)
        mask_b = ops.broadcast_to(ops.expand_dims(mask_w, axis=-1), ops.shape(inputs))
        bshape = [1] * inputs.ndim
        bshape[self.axis] = inputs.shape[self.axis]
        wsum = ops.sum(mask_b, self._reduction_axes, keepdims=True)
        mean = ops.sum(inputs * mask_b, self._reduction_axes, keepdims=True) / wsum
        diff = inputs - mean
        var = ops.sum(diff * diff * mask_b, self._reduction_axes, keepdims=True) / wsum
        return ops.squeeze(mean, self._reduction_axes), ops.squeeze(var, self._reduction_axes)

    def _renorm_correction_and_moments(self, x, mean, variance, training):
        stddev = torch.sqrt(variance + self.epsilon)
        rs, rm = self.renorm_stddev.value.to(x.dtype), self.renorm_mean.value.to(x.dtype)
        r = (stddev / rs).detach()
        d = ((mean - rm) / rs).detach()
        clip = self.renorm_clipping or {}
        if clip.get("rmax") is not None or clip.get("rmin") is not None:
            r = torch.clip(r, clip.get("rmin"), clip.get("rmax"))
        if clip.get("dmax") is not None:
            d = torch.clip(d, -clip["dmax"], clip["dmax"])
        bshape = [1] * x.ndim
        bshape[self.axis] = x.shape[self.axis]
        xn = (x - mean.reshape(bshape)) / stddev.reshape(bshape)
        xn = xn * r.reshape(bshape) + d.reshape(bshape)
        if self.scale:
            xn = xn * self.gamma.value.to(x.dtype).reshape(bshape)
        if self.center:
            xn = xn + self.beta.value.to(x.dtype).reshape(bshape)
        with torch.no_grad():
            m = self.renorm_momentum
            self.renorm_mean.assign(rm * m + mean.detach() * (1 - m))
            self.renorm_stddev.assign(rs * m + stddev.detach() * (1 - m))
            self.moving_mean.assign(self.moving_mean.value.to(x.dtype) * self.momentum + mean.detach() * (1 - self.momentum))
            new_std = torch.sqrt(self.moving_variance.value.to(x.dtype) + self.epsilon) * self.momentum + stddev.detach() * (1 - self.momentum)
            self.moving_variance.assign(torch.relu(new_std * new_std - self.epsilon))
        return xn, mean, variance

    def get_config(self):
        base = super().get_config()
        cfg = {
            "axis": self.axis, "momentum": self.momentum, "epsilon": self.epsilon, "center": self.center, "scale": self.scale,
            "beta_initializer": initializers.serialize(self.beta_initializer), "gamma_initializer": initializers.serialize(self.gamma_initializer),
            "moving_mean_initializer": initializers.serialize(self.moving_mean_initializer),
            "moving_variance_initializer": initializers.serialize(self.moving_variance_initializer),
            "beta_regularizer": regularizers.serialize(self.beta_regularizer), "gamma_regularizer": regularizers.serialize(self.gamma_regularizer),
            "beta_constraint": constraints.serialize(self.beta_constraint), "gamma_constraint": constraints.serialize(self.gamma_constraint),
            "synchronized": self.synchronized, "renorm": self.renorm, "renorm_clipping": self.renorm_clipping, "renorm_momentum": self.renorm_momentum,
        }
        return {**base, **cfg}


@keras_export("keras.layers.LayerNormalization")
class LayerNormalization(Layer):
    def __init__(self, axis=-1, epsilon=1e-3, center=True, scale=True, beta_initializer="zeros", gamma_initializer="ones",
                 beta_regularizer=None, gamma_regularizer=None, beta_constraint=None, gamma_constraint=None, **kwargs):
        rms_scaling = kwargs.pop("rms_scaling", False)
        super().__init__(**kwargs)
        if isinstance(axis, (list, tuple)):
            self.axis = list(axis)
        elif isinstance(axis, int):
            self.axis = axis
        else:
            raise TypeError(f"Expected an int or a list/tuple of ints for the argument 'axis', but received: {axis!r}")
        self.epsilon = epsilon
        self.center, self.scale, self.rms_scaling = center, scale, rms_scaling
        self.beta_initializer = initializers.get(beta_initializer)
        self.gamma_initializer = initializers.get(gamma_initializer)
        self.beta_regularizer = regularizers.get(beta_regularizer)
        self.gamma_regularizer = regularizers.get(gamma_regularizer)
        self.beta_constraint = constraints.get(beta_constraint)
        self.gamma_constraint = constraints.get(gamma_constraint)
        self.supports_masking = True
        self.autocast = False
        self.gamma = self.beta = None

    def build(self, input_shape):
        if isinstance(self.axis, list):
            shape = tuple(input_shape[d] for d in self.axis)
        else:
            shape = (input_shape[self.axis],)
            self.axis = [self.axis]
        if self.scale or self.rms_scaling:
            self.gamma = self.add_weight(name="gamma", shape=shape, initializer=self.gamma_initializer, regularizer=self.gamma_regularizer,
                                         constraint=self.gamma_constraint, trainable=True, autocast=False)
        if self.center and not self.rms_scaling:
            self.beta = self.add_weight(name="beta", shape=shape, initializer=self.beta_initializer, regularizer=self.beta_regularizer,
                                        constraint=self.beta_constraint, trainable=True, autocast=False)
        self.built = True

    def call(self, inputs):
        return ops.layer_normalization(inputs, self.gamma if (self.scale or self.rms_scaling) else None,
                                       self.beta if (self.center and not self.rms_scaling) else None,
                                       axis=self.axis, epsilon=self.epsilon, rms_scaling=self.rms_scaling)

    def compute_output_shape(self, input_shape):
        axes = [self.axis] if isinstance(self.axis, int) else self.axis
        for a in axes:
            if a >= len(input_shape) or a < -len(input_shape):
                raise ValueError(f"Axis {a} is out of bounds for input shape {input_shape}. Received: axis={self.axis}")
        return input_shape

    def get_config(self):
        cfg = {
            "axis": self.axis, "epsilon": self.epsilon, "center": self.center, "scale": self.scale, "rms_scaling": self.rms_scaling,
            "beta_initializer": initializers.serialize(self.beta_initializer), "gamma_initializer": initializers.serialize(self.gamma_initializer),
            "beta_regularizer": regularizers.serialize(self.beta_regularizer), "gamma_regularizer": regularizers.serialize(self.gamma_regularizer),
            "beta_constraint": constraints.serialize(self.beta_constraint), "gamma_constraint": constraints.serialize(self.gamma_constraint),
        }
        return {**super().get_config(), **cfg}


@keras_export("keras.layers.RMSNormalization")
class RMSNormalization(Layer):
    def __init__(self, axis=-1, epsilon=1e-6, **kwargs):
        super().__init__(**kwargs)
        self.axis = axis
        self.epsilon = epsilon

    def build(self, input_shape):
        if isinstance(self.axis, (list, tuple)):
            shape = tuple(input_shape[d] for d in self.axis)
        else:
            shape = (input_shape[self.axis],)
            self.axis = [self.axis]
        self.scale = self.add_weight(name="scale", shape=shape, initializer="ones")
        self.built = True

    def call(self, x):
        return ops.rms_normalization(x, scale=self.scale, axis=self.axis, epsilon=self.epsilon)

    def compute_output_shape(self, input_shape):
        axes = [self.axis] if isinstance(self.axis, int) else self.axis
        for a in axes:
            if a >= len(input_shape) or a < -len(input_shape):
                raise ValueError(f"Axis {a} is out of bounds for input shape {input_shape}. Received: axis={self.axis}")
        return input_shape

    def get_config(self):
        return {**super().get_config(), "axis": self.axis, "epsilon": self.epsilon}


@keras_export("keras.layers.GroupNormalization")
class GroupNormalization(Layer):
    def __init__(self, groups=32, axis=-1, epsilon=1e-3, center=True, scale=True, beta_initializer="zeros", gamma_initializer="ones",
                 beta_regularizer=None, gamma_regularizer=None, beta_constraint=None, gamma_constraint=None, **kwargs):
        super().__init__(**kwargs)
        self.supports_masking = True
        self.groups, self.axis, self.epsilon, self.center, self.scale = groups, axis, epsilon, center, scale
        self.beta_initializer = initializers.get(beta_initializer)
        self.gamma_initializer = initializers.get(gamma_initializer)
        self.beta_regularizer = regularizers.get(beta_regularizer)
        self.gamma_regularizer = regularizers.get(gamma_regularizer)
        self.beta_constraint = constraints.get(beta_constraint)
        self.gamma_constraint = constraints.get(gamma_constraint)
        self.gamma = self.beta = None

    def build(self, input_shape):
        dim = input_shape[self.axis]
        if dim is None:
            raise ValueError(f"Axis {self.axis} of input tensor should have a defined dimension but the layer received an input with shape {input_shape}.")
        if self.groups == -1:
            self.groups = dim
        if dim < self.groups:
            raise ValueError(f"Number of groups ({self.groups}) cannot be more than the number of channels ({dim}).")
        if dim % self.groups != 0:
            raise ValueError(f"Number of groups ({self.groups}) must be a multiple of the number of channels ({dim}).")
        self.input_spec = InputSpec(ndim=len(input_shape), axes={self.axis: dim})
        if self.scale:
            self.gamma = self.add_weight(shape=(dim,), name="gamma", initializer=self.gamma_initializer, regularizer=self.gamma_regularizer, constraint=self.gamma_constraint)
        if self.center:
            self.beta = self.add_weight(shape=(dim,), name="beta", initializer=self.beta_initializer, regularizer=self.beta_regularizer, constraint=self.beta_constraint)
        self.built = True

    def call(self, inputs):
        x = inputs
        axis = self.axis % x.ndim
        shape = list(x.shape)
        gshape = shape[:axis] + [self.groups, shape[axis] // self.groups] + shape[axis + 1:]
        ori = x.dtype
        xg = x.reshape(gshape)
        xg = xg.float() if ori in (torch.float16, torch.bfloat16) else xg
        red = [i for i in range(1, len(gshape)) if i != axis]
        mean = xg.mean(dim=red, keepdim=True)
        var = xg.var(dim=red, keepdim=True, correction=0)
        xn = ((xg - mean) * torch.rsqrt(var + self.epsilon)).reshape(shape)
        bshape = [1] * len(shape)
        bshape[axis] = shape[axis]
        if self.scale:
            xn = xn * self.gamma.value.to(xn.dtype).reshape(bshape)
        if self.center:
            xn = xn + self.beta.value.to(xn.dtype).reshape(bshape)
        return xn.to(ori)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        cfg = {
            "groups": self.groups, "axis": self.axis, "epsilon": self.epsilon, "center": self.center, "scale": self.scale,
            "beta_initializer": initializers.serialize(self.beta_initializer), "gamma_initializer": initializers.serialize(self.gamma_initializer),
            "beta_regularizer": regularizers.serialize(self.beta_regularizer), "gamma_regularizer": regularizers.serialize(self.gamma_regularizer),
            "beta_constraint": constraints.serialize(self.beta_constraint), "gamma_constraint": constraints.serialize(self.gamma_constraint),
        }
        return {**super().get_config(), **cfg}


@keras_export("keras.layers.UnitNormalization")
class UnitNormalization(Layer):
    def __init__(self, axis=-1, **kwargs):
        super().__init__(**kwargs)
        if isinstance(axis, (list, tuple)):
            self.axis = list(axis)
        elif isinstance(axis, int):
            self.axis = axis
        else:
            raise TypeError(f"Invalid value for `axis` argument: expected an int or a list/tuple of ints. Received: axis={axis}")
        self.supports_masking = True
        self.built = True

    def call(self, inputs):
        return ops.normalize(inputs, axis=self.axis, order=2, epsilon=1e-12)

    def compute_output_shape(self, input_shape):
        axes = [self.axis] if isinstance(self.axis, int) else self.axis
        for a in axes:
            if a >= len(input_shape) or a < -len(input_shape):
                raise ValueError(f"Axis {a} is out of bounds for input shape {input_shape}. Received: axis={self.axis}")
        return input_shape

    def get_config(self):
        return {**super().get_config(), "axis": self.axis}


@keras_export("keras.layers.SpectralNormalization")
class SpectralNormalization(Wrapper):
    def __init__(self, layer, power_iterations=1, **kwargs):
        super().__init__(layer, **kwargs)
        if power_iterations <= 0:
            raise ValueError(f"`power_iterations` should be greater than zero. Received: `power_iterations={power_iterations}`")
        self.power_iterations = power_iterations

    def build(self, input_shape):
        super().build(input_shape)
        self.input_spec = InputSpec(min_ndim=1, axes={-1: input_shape[-1]})
        if hasattr(self.layer, "kernel"):
            self.kernel = self.layer.kernel
        elif hasattr(self.layer, "embeddings"):
            self.kernel = self.layer.embeddings
        else:
            raise ValueError(f"{type(self.layer).__name__} object has no attribute 'kernel' nor 'embeddings'")
        self.kernel_shape = tuple(self.kernel.shape)
        self.vector_u = self.add_weight(shape=(1, self.kernel_shape[-1]), initializer=initializers.TruncatedNormal(stddev=0.02), trainable=False,
                                        name="vector_u", dtype=self.kernel.dtype)

    def call(self, inputs, training=False):
        if training:
            new_u, new_kernel = self.normalized_weights()
            with torch.no_grad():
                self.vector_u.assign(new_u)
                self.kernel.assign(new_kernel)
        out = self.layer(inputs)
        return ops.cast(out, inputs.dtype)

    def compute_output_shape(self, input_shape):
        return self.layer.compute_output_shape(input_shape)

    def normalized_weights(self):
        w = self.kernel.value_unautocast().reshape(-1, self.kernel_shape[-1]).detach()
        u = self.vector_u.value_unautocast().detach()
        for _ in range(self.power_iterations):
            v = torch.nn.functional.normalize(u @ w.t(), dim=None, eps=1e-12)
            u = torch.nn.functional.normalize(v @ w, dim=None, eps=1e-12)
        sigma = v @ w @ u.t()
        kernel = (self.kernel.value_unautocast().detach() / sigma).reshape(self.kernel_shape)
        return u, kernel

    def get_config(self):
        return {**super().get_config(), "power_iterations": self.power_iterations}
