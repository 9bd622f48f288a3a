"""Accuracy, regression, probabilistic and hinge metrics (keras/src/metrics/*_metrics.py)."""

import torch

from keras_b200 import initializers, ops
from keras_b200.core.dtypes import to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.losses import losses as L
from keras_b200.losses.loss import squeeze_or_expand_to_same_rank
from keras_b200.metrics.metric import Metric
from keras_b200.metrics.reduction_metrics import Mean, MeanMetricWrapper, reduce_to_samplewise_values


def accuracy(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
    return (y_true == y_pred).to(torch.float32)


@keras_export("keras.metrics.binary_accuracy")
def binary_accuracy(y_true, y_pred, threshold=0.5):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
    y_pred = (y_pred > threshold).to(y_true.dtype)
    return (y_true == y_pred).to(torch.float32)


@keras_export("keras.metrics.categorical_accuracy")
def categorical_accuracy(y_true, y_pred):
    y_true = torch.argmax(convert_to_tensor(y_true), dim=-1)
    y_pred = convert_to_tensor(y_pred)
    reshape = False
    y_true_org_shape = y_true.shape
    if y_true.ndim == y_pred.ndim and y_true.ndim > 0 and y_true.shape[-1] == 1:
        y_true = y_true.squeeze(-1)
        reshape = True
    y_pred_idx = torch.argmax(y_pred, dim=-1)
    matches = (y_true == y_pred_idx).to(torch.float32)
    if reshape:
        matches = matches.reshape(y_true_org_shape)
    return matches


@keras_export("keras.metrics.sparse_categorical_accuracy")
def sparse_categorical_accuracy(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true)
    reshape = False
    y_true_org_shape = y_true.shape
    if y_true.ndim == y_pred.ndim and y_true.ndim > 0 and y_true.shape[-1] == 1:
        y_true = y_true.squeeze(-1)
        reshape = True
    y_pred_idx = torch.argmax(y_pred, dim=-1)
    matches = (y_true.to(y_pred_idx.dtype) == y_pred_idx).to(torch.float32) if not y_true.dtype.is_floating_point else (y_true == y_pred_idx.to(y_true.dtype)).to(torch.float32)
    if reshape:
        matches = matches.reshape(y_true_org_shape)
    if matches.ndim > 1 and matches.shape[-1] == 1:
        matches = matches.squeeze(-1)
    return matches


@keras_export("keras.metrics.top_k_categorical_accuracy")
def top_k_categorical_accuracy(y_true, y_pred, k=5):
    y_pred = convert_to_tensor(y_pred)
    y_true = torch.argmax(convert_to_tensor(y_true), dim=-1)
    return _in_top_k(y_true, y_pred, k)


@keras_export("keras.metrics.sparse_top_k_categorical_accuracy")
def sparse_top_k_categorical_accuracy(y_true, y_pred, k=5, from_sorted_ids=False):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true)
    if y_true.ndim == y_pred.ndim and y_true.shape[-1] == 1:
        y_true = y_true.squeeze(-1)
    if from_sorted_ids:
        return torch.any(y_true.unsqueeze(-1).to(y_pred.dtype) == y_pred[..., :k], dim=-1).to(torch.float32)
    return _in_top_k(y_true.long(), y_pred, k)


def _in_top_k(y_true, y_pred, k):
    shape = y_true.shape
    yp = y_pred.reshape(-1, y_pred.shape[-1])
    yt = y_true.reshape(-1).long()
    return ops.in_top_k(yt, yp, k).to(torch.float32).reshape(shape)


def _wrap(name, fn, exports, arg_defaults, default_name, direction="up", leading=()):
    """Metric class averaging ``fn`` over samples.  Positional constructor arguments are ``leading`` (for example ``k``
    of the top-k accuracies), then ``name`` and ``dtype``, then the remaining entries of ``arg_defaults``."""
    arg_names = list(arg_defaults)
    positional = list(leading) + ["name", "dtype"] + [a for a in arg_names if a not in leading]

    def __init__(self, *args, **kwargs):
        if len(args) > len(positional):
            raise TypeError(f"{name}() takes at most {len(positional)} positional arguments but {len(args)} were given")
        for key, value in zip(positional, args):
            if key in kwargs:
                raise TypeError(f"{name}() got multiple values for argument '{key}'")
            kwargs[key] = value
        metric_name = kwargs.pop("name", default_name)
        dtype = kwargs.pop("dtype", None)
        vals = dict(arg_defaults)
        for k in list(kwargs):
            if k in vals:
                vals[k] = kwargs.pop(k)
        if kwargs:
            raise TypeError(f"Unexpected keyword arguments: {kwargs}")
        MeanMetricWrapper.__init__(self, fn, name=metric_name, dtype=dtype, **vals)
        for k, v in vals.items():
            setattr(self, k, v)
        self._direction = direction

    def get_config(self):
        cfg = {"name": self.name, "dtype": self.dtype}
        cfg.update({k: getattr(self, k) for k in arg_names})
        return cfg

    cls = type(name, (MeanMetricWrapper,), {"__init__": __init__, "get_config": get_config})
    cls.__module__ = __name__
    cls.from_config = classmethod(lambda c, config: c(**config))
    return keras_export(exports)(cls)


Accuracy = _wrap("Accuracy", accuracy, "keras.metrics.Accuracy", {}, "accuracy")
BinaryAccuracy = _wrap("BinaryAccuracy", binary_accuracy, "keras.metrics.BinaryAccuracy", {"threshold": 0.5}, "binary_accuracy")
CategoricalAccuracy = _wrap("CategoricalAccuracy", categorical_accuracy, "keras.metrics.CategoricalAccuracy", {}, "categorical_accuracy")
SparseCategoricalAccuracy = _wrap("SparseCategoricalAccuracy", sparse_categorical_accuracy, "keras.metrics.SparseCategoricalAccuracy", {}, "sparse_categorical_accuracy")
TopKCategoricalAccuracy = _wrap("TopKCategoricalAccuracy", top_k_categorical_accuracy, "keras.metrics.TopKCategoricalAccuracy", {"k": 5}, "top_k_categorical_accuracy", leading=("k",))
SparseTopKCategoricalAccuracy = _wrap("SparseTopKCategoricalAccuracy", sparse_top_k_categorical_accuracy, "keras.metrics.SparseTopKCategoricalAccuracy", {"k": 5, "from_sorted_ids": False}, "sparse_top_k_categorical_accuracy", leading=("k",))

MeanSquaredError = _wrap("MeanSquaredError", L.mean_squared_error, "keras.metrics.MeanSquaredError", {}, "mean_squared_error", "down")
MeanAbsoluteError = _wrap("MeanAbsoluteError", L.mean_absolute_error, "keras.metrics.MeanAbsoluteError", {}, "mean_absolute_error", "down")
MeanAbsolutePercentageError = _wrap("MeanAbsolutePercentageError", L.mean_absolute_percentage_error, "keras.metrics.MeanAbsolutePercentageError", {}, "mean_absolute_percentage_error", "down")
MeanSquaredLogarithmicError = _wrap("MeanSquaredLogarithmicError", L.mean_squared_logarithmic_error, "keras.metrics.MeanSquaredLogarithmicError", {}, "mean_squared_logarithmic_error", "down")
LogCoshError = _wrap("LogCoshError", L.log_cosh, "keras.metrics.LogCoshError", {}, "logcosh", "down")
KLDivergence = _wrap("KLDivergence", L.kl_divergence, "keras.metrics.KLDivergence", {}, "kl_divergence", "down")
Poisson = _wrap("Poisson", L.poisson, "keras.metrics.Poisson", {}, "poisson", "down")
BinaryCrossentropy = _wrap("BinaryCrossentropy", L.binary_crossentropy, "keras.metrics.BinaryCrossentropy", {"from_logits": False, "label_smoothing": 0}, "binary_crossentropy", "down")
CategoricalCrossentropy = _wrap("CategoricalCrossentropy", L.categorical_crossentropy, "keras.metrics.CategoricalCrossentropy", {"from_logits": False, "label_smoothing": 0, "axis": -1}, "categorical_crossentropy", "down")
SparseCategoricalCrossentropy = _wrap("SparseCategoricalCrossentropy", L.sparse_categorical_crossentropy, "keras.metrics.SparseCategoricalCrossentropy", {"from_logits": False, "axis": -1}, "sparse_categorical_crossentropy", "down")
Hinge = _wrap("Hinge", L.hinge, "keras.metrics.Hinge", {}, "hinge", "down")
SquaredHinge = _wrap("SquaredHinge", L.squared_hinge, "keras.metrics.SquaredHinge", {}, "squared_hinge", "down")
CategoricalHinge = _wrap("CategoricalHinge", L.categorical_hinge, "keras.metrics.CategoricalHinge", {}, "categorical_hinge", "down")


@keras_export("keras.metrics.RootMeanSquaredError")
class RootMeanSquaredError(Mean):
    def __init__(self, name="root_mean_squared_error", dtype=None):
        super().__init__(name, dtype=dtype)
        self._direction = "down"

    def update_state(self, y_true, y_pred, sample_weight=None):
        y_true = convert_to_tensor(y_true, dtype=self.dtype)
        y_pred = convert_to_tensor(y_pred, dtype=self.dtype)
        y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
        return super().update_state(torch.square(y_pred - y_true), sample_weight=sample_weight)

    def result(self):
        return torch.sqrt(super().result())


@keras_export("keras.metrics.CosineSimilarity")
class CosineSimilarity(MeanMetricWrapper):
    def __init__(self, name="cosine_similarity", dtype=None, axis=-1):
        super().__init__(_cosine_similarity, name, dtype=dtype, axis=axis)
        self._direction = "up"

    def get_config(self):
        return {"name": self.name, "dtype": self.dtype}


def _cosine_similarity(y_true, y_pred, axis=-1):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
    return torch.sum(ops.normalize(y_pred, axis=axis) * ops.normalize(y_true, axis=axis), dim=axis)


@keras_export("keras.metrics.R2Score")
class R2Score(Metric):
    def __init__(self, class_aggregation="uniform_average", num_regressors=0, name="r2_score", dtype=None):
        super().__init__(name=name, dtype=dtype)
        self._direction = "up"
        valid = (None, "uniform_average", "variance_weighted_average")
        if class_aggregation not in valid:
            raise ValueError(f"Invalid value for argument `class_aggregation`. Expected one of {valid}. Received: class_aggregation={class_aggregation}")
        if num_regressors < 0:
            raise ValueError(f"Invalid value for argument `num_regressors`. Expected a value >= 0. Received: num_regressors={num_regressors}")
        self.class_aggregation = class_aggregation
        self.num_regressors = num_regressors
        self.num_samples = self.add_variable(shape=(), initializer=initializers.Zeros(), name="num_samples")
        self._built = False

    def _build(self, y_true_shape, y_pred_shape):
        if len(y_pred_shape) != 2 or len(y_true_shape) != 2:
            raise ValueError(f"R2Score expects 2D inputs with shape (batch_size, output_dim). Received input shapes: y_pred.shape={y_pred_shape} and y_true.shape={y_true_shape}.")
        if y_pred_shape[-1] is None or y_true_shape[-1] is None:
            raise ValueError(f"R2Score expects 2D inputs with shape (batch_size, output_dim), with output_dim fully defined (not None). Received input shapes: y_pred.shape={y_pred_shape} and y_true.shape={y_true_shape}.")
        n = y_pred_shape[-1]
        self.squared_sum = self.add_variable(name="squared_sum", shape=[n], initializer=initializers.Zeros())
        self.sum = self.add_variable(name="sum", shape=[n], initializer=initializers.Zeros())
        self.total_mse = self.add_variable(name="residual", shape=[n], initializer=initializers.Zeros())
        self.count = self.add_variable(name="count", shape=[n], initializer=initializers.Zeros())
        self._built = True

    def update_state(self, y_true, y_pred, sample_weight=None):
        y_true = convert_to_tensor(y_true, dtype=self.dtype)
        y_pred = convert_to_tensor(y_pred, dtype=self.dtype)
        y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
        if not self._built:
            self._build(tuple(y_true.shape), tuple(y_pred.shape))
        if sample_weight is None:
            sample_weight = 1
        sample_weight = convert_to_tensor(sample_weight, dtype=self.dtype)
        if sample_weight.ndim == 1:
            sample_weight = sample_weight.unsqueeze(1)
        sample_weight = torch.broadcast_to(sample_weight, y_true.shape)
        weighted_y_true = y_true * sample_weight
        self.sum.assign(self.sum.value + torch.sum(weighted_y_true, dim=0))
        self.squared_sum.assign(self.squared_sum.value + torch.sum(y_true * weighted_y_true, dim=0))
        self.total_mse.assign(self.total_mse.value + torch.sum((y_true - y_pred) ** 2 * sample_weight, dim=0))
        self.count.assign(self.count.value + torch.sum(sample_weight, dim=0))
        self.num_samples.assign(self.num_samples.value + y_true.shape[0])

    def result(self):
        mean = self.sum.value / self.count.value
        total = self.squared_sum.value - self.sum.value * mean
        raw_scores = 1 - (self.total_mse.value / total)
        raw_scores = torch.where(torch.isinf(raw_scores), torch.zeros_like(raw_scores), raw_scores)
        if self.class_aggregation == "uniform_average":
            r2 = torch.mean(raw_scores)
        elif self.class_aggregation == "variance_weighted_average":
            r2 = torch.sum(total * raw_scores) / torch.sum(total)
        else:
            r2 = raw_scores
        if self.num_regressors != 0:
            n = self.num_samples.value.to(torch.float32)
            if self.num_regressors > float(n) - 1:
                import warnings

                warnings.warn("More independent predictors than datapoints in adjusted R2 score. Falling back to standard R2 score.", stacklevel=2)
            elif self.num_regressors == float(n) - 1:
                import warnings

                warnings.warn("Division by zero in Adjusted R2 score. Falling back to standard R2 score.", stacklevel=2)
            else:
                p = float(self.num_regressors)
                r2 = 1 - (1 - r2) * (n - 1) / (n - p - 1)
        return r2

    def reset_state(self):
        for v in self.variables:
            v.assign(torch.zeros(tuple(v.shape), dtype=v._torch_dtype))

    def get_config(self):
        return {"name": self.name, "dtype": self.dtype, "class_aggregation": self.class_aggregation, "num_regressors": self.num_regressors}
