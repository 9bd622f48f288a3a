"""``Sum`` / ``Mean`` / ``MeanMetricWrapper`` (keras/src/metrics/reduction_metrics.py)."""

import torch

from keras_b200 import initializers, losses
from keras_b200.core.dtypes import to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.losses.loss import squeeze_or_expand_to_same_rank
from keras_b200.metrics.metric import Metric


def reduce_to_samplewise_values(values, sample_weight, reduce_fn, dtype):
    td = to_torch_dtype(dtype)
    values = convert_to_tensor(values, dtype=td)
    mask = getattr(values, "_keras_mask", None)
    if sample_weight is not None:
        sample_weight = convert_to_tensor(sample_weight, dtype=td)
        if mask is not None:
            sample_weight = losses.loss.apply_mask(sample_weight, mask, dtype=td, reduction="sum")
        values, sample_weight = squeeze_or_expand_to_same_rank(values, sample_weight)
        weight_ndim, values_ndim = sample_weight.ndim, values.ndim
        if values_ndim > weight_ndim:
            values = reduce_fn(values, dim=list(range(weight_ndim, values_ndim)))
        sample_weight = torch.broadcast_to(sample_weight, values.shape) if sample_weight.shape != values.shape and sample_weight.ndim == values.ndim else sample_weight
        values = values * sample_weight
        if weight_ndim > 1:
            sample_weight = reduce_fn(sample_weight, dim=list(range(1, weight_ndim)))
    values_ndim = values.ndim
    if values_ndim > 1:
        values = reduce_fn(values, dim=list(range(1, values_ndim)))
    return values, sample_weight


@keras_export("keras.metrics.Sum")
class Sum(Metric):
    def __init__(self, name="sum", dtype=None):
        super().__init__(name=name, dtype=dtype)
        self.total = self.add_variable(shape=(), initializer=initializers.Zeros(), dtype=self.dtype, name="total")

    def update_state(self, values, sample_weight=None):
        values, _ = reduce_to_samplewise_values(values, sample_weight, reduce_fn=torch.sum, dtype=self.dtype)
        self.total.assign_add(torch.sum(values))

    def reset_state(self):
        self.total.assign(0)

    def result(self):
        return self.total.value.to(to_torch_dtype(self.dtype))


@keras_export("keras.metrics.Mean")
class Mean(Metric):
    def __init__(self, name="mean", dtype=None):
        super().__init__(name=name, dtype=dtype)
        self.total = self.add_variable(shape=(), initializer=initializers.Zeros(), dtype=self.dtype, name="total")
        self.count = self.add_variable(shape=(), initializer=initializers.Zeros(), dtype=self.dtype, name="count")

    def update_state(self, values, sample_weight=None):
        if type(values) is torch.Tensor and values.ndim == 0 and isinstance(sample_weight, (int, float)):
            # fast path used by the loss tracker: scalar loss weighted by the batch size
            with torch.no_grad():
                v = values.detach().to(self.total._torch_dtype)
                self.total._value.add_(v * sample_weight)
                self.count._value.add_(sample_weight)
            return
        values, sample_weight = reduce_to_samplewise_values(values, sample_weight, reduce_fn=torch.mean, dtype=self.dtype)
        self.total.assign_add(torch.sum(values))
        if sample_weight is not None:
            num_samples = torch.sum(sample_weight)
        elif values.ndim >= 1:
            num_samples = values.shape[0]
        else:
            num_samples = 1
        if not isinstance(num_samples, torch.Tensor):
            num_samples = torch.full((), num_samples, dtype=self.count._torch_dtype, device=self.count._value.device)  # a fill: no host copy
        self.count.assign_add(num_samples)

    def reset_state(self):
        self.total.assign(0)
        self.count.assign(0)

    def result(self):
        total, count = self.total.value, self.count.value
        return torch.where(count == 0, torch.zeros_like(total), total / torch.where(count == 0, torch.ones_like(count), count))


@keras_export("keras.metrics.MeanMetricWrapper")
class MeanMetricWrapper(Mean):
    def __init__(self, fn, name=None, dtype=None, **kwargs):
        super().__init__(name=name, dtype=dtype)
        self._fn = fn
        self._fn_kwargs = kwargs
        if self._fn in losses.ALL_OBJECTS or (hasattr(self._fn, "__class__") and self._fn.__class__ in losses.ALL_OBJECTS):
            self._direction = "down"

    def update_state(self, y_true, y_pred, sample_weight=None):
        mask = getattr(y_pred, "_keras_mask", None)
        values = self._fn(y_true, y_pred, **self._fn_kwargs)
        if mask is not None:
            # masked entries weigh nothing, with or without sample weights (keras/src/metrics/reduction_metrics.py:201-206)
            weights = convert_to_tensor(sample_weight) if sample_weight is not None else None
            sample_weight = losses.loss.apply_mask(weights, convert_to_tensor(mask), dtype=to_torch_dtype(self.dtype), reduction="sum")
        return super().update_state(values, sample_weight=sample_weight)

    def get_config(self):
        from keras_b200.saving import serialization_lib

        base = super().get_config()
        config = {"fn": serialization_lib.serialize_keras_object(self._fn)}
        config.update(serialization_lib.serialize_keras_object(self._fn_kwargs))
        return {**base, **config}

    @classmethod
    def from_config(cls, config):
        from keras_b200.saving import serialization_lib

        if "fn" in config:
            config = serialization_lib.deserialize_keras_object(config)
        return cls(**config)
