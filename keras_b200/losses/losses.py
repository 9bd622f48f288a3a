"""Loss functions and classes (``keras.losses``; keras/src/losses/losses.py)."""

import math
import warnings

import torch

from keras_b200 import ops, tree
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.losses.loss import Loss, squeeze_or_expand_to_same_rank

_EPS = config.epsilon


def _pair(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    return squeeze_or_expand_to_same_rank(y_true, y_pred)


class LossFunctionWrapper(Loss):
    def __init__(self, fn, reduction="sum_over_batch_size", name=None, dtype=None, **kwargs):
        super().__init__(name=name, reduction=reduction, dtype=dtype)
        self.fn = fn
        self._fn_kwargs = kwargs

    def _accepts_low_precision(self, y_pred):
        # the fused softmax cross-entropy kernel reads bf16 logits and accumulates in float32
        import torch

        if self.fn is not sparse_categorical_crossentropy or not isinstance(y_pred, torch.Tensor) or y_pred.dtype != torch.bfloat16:
            return False
        kw = self._fn_kwargs
        if not kw.get("from_logits") or kw.get("ignore_class") is not None or kw.get("axis", -1) not in (-1, y_pred.ndim - 1):
            return False
        from keras_b200.kernels import dispatch

        return self.dtype == "float32" and dispatch.enabled(y_pred) and y_pred.shape[-1] >= 64

    def call(self, y_true, y_pred):
        y_true_y_pred = tree.map_structure(squeeze_or_expand_to_same_rank, y_true, y_pred)
        y_true = tree.map_structure_up_to(y_true, lambda x: x[0], y_true_y_pred)
        y_pred = tree.map_structure_up_to(y_pred, lambda x: x[1], y_true_y_pred)
        return self.fn(y_true, y_pred, **self._fn_kwargs)

    def get_config(self):
        from keras_b200.saving import serialization_lib

        cfg = super().get_config()
        cfg.update({"fn": serialization_lib.serialize_keras_object(self.fn)})
        cfg.update(serialization_lib.serialize_keras_object(self._fn_kwargs))
        return cfg

    @classmethod
    def from_config(cls, config):
        from keras_b200.saving import serialization_lib

        if "fn" in config:
            config = serialization_lib.deserialize_keras_object(config)
        return cls(**config)

    def __repr__(self):
        return f"<LossFunctionWrapper({self.fn}, kwargs={self._fn_kwargs})>"


# --- functions -----------------------------------------------------------------------------

@keras_export(["keras.metrics.mean_squared_error", "keras.losses.mean_squared_error", "keras.losses.mse", "keras.losses.MSE", "keras.metrics.mse", "keras.metrics.MSE"])
def mean_squared_error(y_true, y_pred):
    y_true, y_pred = _pair(y_true, y_pred)
    return torch.mean(torch.square(y_true - y_pred), dim=-1)


@keras_export(["keras.metrics.mean_absolute_error", "keras.losses.mean_absolute_error", "keras.losses.mae", "keras.losses.MAE", "keras.metrics.mae", "keras.metrics.MAE"])
def mean_absolute_error(y_true, y_pred):
    y_true, y_pred = _pair(y_true, y_pred)
    return torch.mean(torch.abs(y_true - y_pred), dim=-1)


@keras_export(["keras.metrics.mean_absolute_percentage_error", "keras.losses.mean_absolute_percentage_error", "keras.losses.mape", "keras.losses.MAPE", "keras.metrics.mape", "keras.metrics.MAPE"])
def mean_absolute_percentage_error(y_true, y_pred):
    y_true, y_pred = _pair(y_true, y_pred)
    diff = torch.abs((y_true - y_pred) / torch.clamp(torch.abs(y_true), min=_EPS()))
    return 100.0 * torch.mean(diff, dim=-1)


@keras_export(["keras.metrics.mean_squared_logarithmic_error", "keras.losses.mean_squared_logarithmic_error", "keras.losses.msle", "keras.losses.MSLE", "keras.metrics.msle", "keras.metrics.MSLE"])
def mean_squared_logarithmic_error(y_true, y_pred):
    y_true, y_pred = _pair(y_true, y_pred)
    a = torch.log(torch.clamp(y_pred, min=_EPS()) + 1.0)
    b = torch.log(torch.clamp(y_true, min=_EPS()) + 1.0)
    return torch.mean(torch.square(a - b), dim=-1)


@keras_export("keras.losses.cosine_similarity")
def cosine_similarity(y_true, y_pred, axis=-1):
    y_true, y_pred = _pair(y_true, y_pred)
    return -torch.sum(ops.normalize(y_pred, axis=axis) * ops.normalize(y_true, axis=axis), dim=axis)


@keras_export(["keras.losses.huber", "keras.metrics.huber"])
def huber(y_true, y_pred, delta=1.0):
    y_true, y_pred = _pair(y_true, y_pred)
    error = y_pred - y_true
    abs_error = torch.abs(error)
    half = 0.5
    return torch.mean(torch.where(abs_error <= delta, half * torch.square(error), delta * abs_error - half * delta * delta), dim=-1)


@keras_export(["keras.losses.log_cosh", "keras.metrics.log_cosh", "keras.losses.logcosh", "keras.metrics.logcosh"])
def log_cosh(y_true, y_pred):
    y_true, y_pred = _pair(y_true, y_pred)
    x = y_pred - y_true
    return torch.mean(x + torch.nn.functional.softplus(-2.0 * x) - math.log(2.0), dim=-1)


@keras_export(["keras.metrics.hinge", "keras.losses.hinge"])
def hinge(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true = convert_binary_labels_to_hinge(y_true)
    return torch.mean(torch.clamp(1.0 - y_true * y_pred, min=0.0), dim=-1)


@keras_export(["keras.metrics.squared_hinge", "keras.losses.squared_hinge"])
def squared_hinge(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_binary_labels_to_hinge(convert_to_tensor(y_true).to(y_pred.dtype))
    return torch.mean(torch.square(torch.clamp(1.0 - y_true * y_pred, min=0.0)), dim=-1)


@keras_export(["keras.metrics.categorical_hinge", "keras.losses.categorical_hinge"])
def categorical_hinge(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    pos = torch.sum(y_true * y_pred, dim=-1)
    neg = torch.amax((1.0 - y_true) * y_pred, dim=-1)
    return torch.clamp(neg - pos + 1.0, min=0.0)


def convert_binary_labels_to_hinge(y_true):
    are_zeros = y_true == 0
    are_ones = y_true == 1
    is_binary = torch.all(are_zeros | are_ones)
    return torch.where(is_binary, 2.0 * y_true - 1.0, y_true)


@keras_export(["keras.metrics.kl_divergence", "keras.losses.kl_divergence", "keras.losses.kld", "keras.losses.KLD", "keras.metrics.kld", "keras.metrics.KLD"])
def kl_divergence(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true = torch.clip(y_true, _EPS(), 1)
    y_pred = torch.clip(y_pred, _EPS(), 1)
    return torch.sum(y_true * torch.log(y_true / y_pred), dim=-1)


@keras_export(["keras.metrics.poisson", "keras.losses.poisson"])
def poisson(y_true, y_pred):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    return torch.mean(y_pred - y_true * torch.log(y_pred + _EPS()), dim=-1)


@keras_export(["keras.metrics.categorical_crossentropy", "keras.losses.categorical_crossentropy"])
def categorical_crossentropy(y_true, y_pred, from_logits=False, label_smoothing=0.0, axis=-1):
    if isinstance(axis, bool):
        raise ValueError(f"`axis` must be of type `int`. Received: axis={axis} of type {type(axis)}")
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    if y_pred.shape[-1] == 1:
        warnings.warn(
            "In loss categorical_crossentropy, expected y_pred.shape to be (batch_size, num_classes) with num_classes > 1. "
            f"Received: y_pred.shape={tuple(y_pred.shape)}. Consider using 'binary_crossentropy' if you only have 2 classes.",
            SyntaxWarning, stacklevel=2,
        )
    if label_smoothing:
        num_classes = y_true.shape[-1]
        y_true = y_true * (1.0 - label_smoothing) + (label_smoothing / num_classes)
    return ops.categorical_crossentropy(y_true, y_pred, from_logits=from_logits, axis=axis)


@keras_export(["keras.metrics.categorical_focal_crossentropy", "keras.losses.categorical_focal_crossentropy"])
def categorical_focal_crossentropy(y_true, y_pred, alpha=0.25, gamma=2.0, from_logits=False, label_smoothing=0.0, axis=-1):
    if isinstance(axis, bool):
        raise ValueError(f"`axis` must be of type `int`. Received: axis={axis} of type {type(axis)}")
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    if label_smoothing:
        y_true = y_true * (1.0 - label_smoothing) + (label_smoothing / y_true.shape[-1])
    if from_logits:
        y_pred = torch.softmax(y_pred, dim=axis)
    output = y_pred / torch.sum(y_pred, dim=axis, keepdim=True)
    output = torch.clip(output, _EPS(), 1.0 - _EPS())
    cce = -y_true * torch.log(output)
    modulating = torch.pow(1.0 - output, gamma)
    return torch.sum(alpha * modulating * cce, dim=axis)


@keras_export(["keras.metrics.sparse_categorical_crossentropy", "keras.losses.sparse_categorical_crossentropy"])
def sparse_categorical_crossentropy(y_true, y_pred, from_logits=False, ignore_class=None, axis=-1):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true)
    if len(y_true.shape) == len(y_pred.shape) and y_true.shape[-1] == 1:
        y_true = y_true.squeeze(-1)
    if ignore_class is not None:
        res_shape = y_pred.shape[:-1]
        valid_mask = y_true != ignore_class
        y_true = y_true * valid_mask.to(y_true.dtype)
        y_pred = y_pred * valid_mask.unsqueeze(-1).to(y_pred.dtype)
    res = ops.sparse_categorical_crossentropy(y_true, y_pred, from_logits=from_logits, axis=axis)
    if ignore_class is not None:
        valid_mask = valid_mask.reshape(res_shape)
        res = torch.where(valid_mask, res, torch.zeros_like(res))
        try:
            res._keras_mask = valid_mask
        except AttributeError:
            pass
    return res


@keras_export(["keras.metrics.binary_crossentropy", "keras.losses.binary_crossentropy"])
def binary_crossentropy(y_true, y_pred, from_logits=False, label_smoothing=0.0, axis=-1):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    if label_smoothing:
        y_true = y_true * (1.0 - label_smoothing) + 0.5 * label_smoothing
    return torch.mean(ops.binary_crossentropy(y_true, y_pred, from_logits=from_logits), dim=axis)


@keras_export(["keras.metrics.binary_focal_crossentropy", "keras.losses.binary_focal_crossentropy"])
def binary_focal_crossentropy(y_true, y_pred, apply_class_balancing=False, alpha=0.25, gamma=2.0, from_logits=False, label_smoothing=0.0, axis=-1):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    if label_smoothing:
        y_true = y_true * (1.0 - label_smoothing) + 0.5 * label_smoothing
    if from_logits:
        y_pred = torch.sigmoid(y_pred)
    bce = ops.binary_crossentropy(y_true, y_pred, from_logits=False)
    p_t = y_true * y_pred + (1 - y_true) * (1 - y_pred)
    focal_factor = torch.pow(1.0 - p_t, gamma)
    focal_bce = focal_factor * bce
    if apply_class_balancing:
        weight = y_true * alpha + (1 - y_true) * (1 - alpha)
        focal_bce = weight * focal_bce
    return torch.mean(focal_bce, dim=axis)


@keras_export("keras.losses.ctc")
def ctc(y_true, y_pred):
    y_true = convert_to_tensor(y_true)
    y_pred = convert_to_tensor(y_pred)
    if len(y_true.shape) != 2:
        raise ValueError(f"Targets `y_true` are expected to be a tensor of shape `(batch_size, max_length)` in integer format. Received: y_true.shape={tuple(y_true.shape)}")
    if len(y_pred.shape) != 3:
        raise ValueError(f"Logits `y_pred` are expected to be a tensor of shape `(batch_size, max_length, num_classes)`. Received: y_pred.shape={tuple(y_pred.shape)}")
    mask_index = 0
    batch_length = y_pred.shape[0]
    input_length = torch.full((batch_length,), y_pred.shape[1], dtype=torch.int32, device=y_pred.device)
    label_length = torch.sum(y_true != mask_index, dim=-1).to(torch.int32)
    return ops.ctc_loss(y_true, y_pred, label_length, input_length, mask_index=mask_index)


@keras_export("keras.losses.dice")
def dice(y_true, y_pred, axis=None):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    inputs, targets = y_true, y_pred
    if axis is None:
        intersection = torch.sum(inputs * targets)
        denom = torch.sum(y_true) + torch.sum(y_pred)
    else:
        intersection = torch.sum(inputs * targets, dim=axis)
        denom = torch.sum(y_true, dim=axis) + torch.sum(y_pred, dim=axis)
    d = (2.0 * intersection + _EPS()) / (denom + _EPS())
    return 1 - d


@keras_export("keras.losses.tversky")
def tversky(y_true, y_pred, alpha=0.5, beta=0.5, axis=None):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    kw = {} if axis is None else {"dim": axis}
    intersection = torch.sum(y_true * y_pred, **kw)
    fp = torch.sum((1 - y_true) * y_pred, **kw)
    fn = torch.sum(y_true * (1 - y_pred), **kw)
    t = (intersection + _EPS()) / (intersection + alpha * fp + beta * fn + _EPS())
    return 1 - t


@keras_export("keras.losses.circle")
def circle(y_true, y_pred, ref_labels=None, ref_embeddings=None, remove_diagonal=True, gamma=80, margin=0.4):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(torch.int32)
    ref_embeddings = y_pred if ref_embeddings is None else convert_to_tensor(ref_embeddings)
    ref_labels = y_true if ref_labels is None else convert_to_tensor(ref_labels).to(torch.int32)
    optim_pos, optim_neg = margin, 1 + margin
    delta_pos, delta_neg = margin, 1 - margin
    pairwise_cosine_distances = 1 - torch.matmul(y_pred, ref_embeddings.t())
    pairwise_cosine_distances = torch.clamp(pairwise_cosine_distances, min=0.0)
    y_true2 = y_true.reshape(-1, 1)
    ref2 = ref_labels.reshape(1, -1)
    positive_mask = y_true2 == ref2
    negative_mask = ~positive_mask
    if remove_diagonal:
        positive_mask = positive_mask & ~torch.eye(positive_mask.shape[0], positive_mask.shape[1], dtype=torch.bool, device=y_pred.device)
    pos_weights = optim_pos + pairwise_cosine_distances
    pos_weights = pos_weights * positive_mask.to(y_pred.dtype)
    pos_weights = torch.clamp(pos_weights, min=0.0)
    neg_weights = optim_neg - pairwise_cosine_distances
    neg_weights = neg_weights * negative_mask.to(y_pred.dtype)
    neg_weights = torch.clamp(neg_weights, min=0.0)
    pos_dists = delta_pos - pairwise_cosine_distances
    neg_dists = delta_neg - pairwise_cosine_distances
    pos_wdists = -1 * gamma * pos_weights * pos_dists
    neg_wdists = gamma * neg_weights * neg_dists
    ninf = -1e9
    p_loss = torch.logsumexp(torch.where(positive_mask, pos_wdists, torch.full_like(pos_wdists, ninf)), dim=1)
    n_loss = torch.logsumexp(torch.where(negative_mask, neg_wdists, torch.full_like(neg_wdists, ninf)), dim=1)
    out = torch.nn.functional.softplus(p_loss + n_loss)
    out._keras_mask = out > 0  # anchors without a positive or without a negative do not count in the reduction
    return out


@keras_export("keras.losses.categorical_generalized_cross_entropy")
def categorical_generalized_cross_entropy(y_true, y_pred, q):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).long()
    if y_true.ndim == y_pred.ndim and y_true.shape[-1] == 1:
        y_true = y_true.squeeze(-1)
    p = torch.gather(y_pred, -1, y_true.unsqueeze(-1)).squeeze(-1)
    return (1 - torch.pow(p, q)) / q


# --- classes -------------------------------------------------------------------------------

def _wrapper_class(name, fn, exports, arg_defaults, default_name, doc=None, reduction_default="sum_over_batch_size"):
    arg_names = list(arg_defaults)

    def __init__(self, *args, reduction=reduction_default, name=default_name, dtype=None, **kwargs):
        vals = dict(arg_defaults)
        for n, v in zip(arg_names, args):
            vals[n] = v
        for k in list(kwargs):
            if k in vals:
                vals[k] = kwargs.pop(k)
        if kwargs:
            raise TypeError(f"Unexpected keyword arguments: {kwargs}")
        LossFunctionWrapper.__init__(self, fn, name=name, reduction=reduction, dtype=dtype, **vals)
        for k, v in vals.items():
            setattr(self, k, v)

    def get_config(self):
        cfg = Loss.get_config(self)
        cfg.update({k: getattr(self, k) for k in arg_names})
        return cfg

    cls = type(name, (LossFunctionWrapper,), {"__init__": __init__, "get_config": get_config, "__doc__": doc})
    cls.__module__ = __name__
    cls.from_config = classmethod(lambda c, config: c(**config))
    return keras_export(exports)(cls)


MeanSquaredError = _wrapper_class("MeanSquaredError", mean_squared_error, "keras.losses.MeanSquaredError", {}, "mean_squared_error")
MeanAbsoluteError = _wrapper_class("MeanAbsoluteError", mean_absolute_error, "keras.losses.MeanAbsoluteError", {}, "mean_absolute_error")
MeanAbsolutePercentageError = _wrapper_class("MeanAbsolutePercentageError", mean_absolute_percentage_error, "keras.losses.MeanAbsolutePercentageError", {}, "mean_absolute_percentage_error")
MeanSquaredLogarithmicError = _wrapper_class("MeanSquaredLogarithmicError", mean_squared_logarithmic_error, "keras.losses.MeanSquaredLogarithmicError", {}, "mean_squared_logarithmic_error")
CosineSimilarity = _wrapper_class("CosineSimilarity", cosine_similarity, "keras.losses.CosineSimilarity", {"axis": -1}, "cosine_similarity")
Huber = _wrapper_class("Huber", huber, "keras.losses.Huber", {"delta": 1.0}, "huber_loss")
LogCosh = _wrapper_class("LogCosh", log_cosh, "keras.losses.LogCosh", {}, "log_cosh")
Hinge = _wrapper_class("Hinge", hinge, "keras.losses.Hinge", {}, "hinge")
SquaredHinge = _wrapper_class("SquaredHinge", squared_hinge, "keras.losses.SquaredHinge", {}, "squared_hinge")
CategoricalHinge = _wrapper_class("CategoricalHinge", categorical_hinge, "keras.losses.CategoricalHinge", {}, "categorical_hinge")
KLDivergence = _wrapper_class("KLDivergence", kl_divergence, "keras.losses.KLDivergence", {}, "kl_divergence")
Poisson = _wrapper_class("Poisson", poisson, "keras.losses.Poisson", {}, "poisson")
BinaryCrossentropy = _wrapper_class("BinaryCrossentropy", binary_crossentropy, "keras.losses.BinaryCrossentropy", {"from_logits": False, "label_smoothing": 0.0, "axis": -1}, "binary_crossentropy")
BinaryFocalCrossentropy = _wrapper_class("BinaryFocalCrossentropy", binary_focal_crossentropy, "keras.losses.BinaryFocalCrossentropy", {"apply_class_balancing": False, "alpha": 0.25, "gamma": 2.0, "from_logits": False, "label_smoothing": 0.0, "axis": -1}, "binary_focal_crossentropy")
CategoricalCrossentropy = _wrapper_class("CategoricalCrossentropy", categorical_crossentropy, "keras.losses.CategoricalCrossentropy", {"from_logits": False, "label_smoothing": 0.0, "axis": -1}, "categorical_crossentropy")
CategoricalFocalCrossentropy = _wrapper_class("CategoricalFocalCrossentropy", categorical_focal_crossentropy, "keras.losses.CategoricalFocalCrossentropy", {"alpha": 0.25, "gamma": 2.0, "from_logits": False, "label_smoothing": 0.0, "axis": -1}, "categorical_focal_crossentropy")
SparseCategoricalCrossentropy = _wrapper_class("SparseCategoricalCrossentropy", sparse_categorical_crossentropy, "keras.losses.SparseCategoricalCrossentropy", {"from_logits": False, "ignore_class": None, "axis": -1}, "sparse_categorical_crossentropy")
CTC = _wrapper_class("CTC", ctc, "keras.losses.CTC", {}, "ctc")
Dice = _wrapper_class("Dice", dice, "keras.losses.Dice", {"axis": None}, "dice")
Tversky = _wrapper_class("Tversky", tversky, "keras.losses.Tversky", {"alpha": 0.5, "beta": 0.5, "axis": None}, "tversky")
Circle = _wrapper_class("Circle", circle, "keras.losses.Circle", {"gamma": 80.0, "margin": 0.4, "remove_diagonal": True}, "circle")
CategoricalGeneralizedCrossEntropy = _wrapper_class("CategoricalGeneralizedCrossEntropy", categorical_generalized_cross_entropy, "keras.losses.CategoricalGeneralizedCrossEntropy", {"q": 0.5}, "categorical_generalized_cross_entropy")
