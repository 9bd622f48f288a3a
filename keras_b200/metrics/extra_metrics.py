"""IoU family, F-scores and correlation metrics (keras/src/metrics/iou_metrics.py,
f_score_metrics.py, correlation_metrics.py)."""

import torch

from keras_b200 import initializers
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.losses.loss import squeeze_or_expand_to_same_rank
from keras_b200.metrics.metric import Metric
from keras_b200.metrics.reduction_metrics import MeanMetricWrapper


def _div_no_nan(a, b):
    return torch.where(b == 0, torch.zeros_like(a), a / torch.where(b == 0, torch.ones_like(b), b))


class _IoUBase(Metric):
    def __init__(self, num_classes, name=None, dtype=None, ignore_class=None, sparse_y_true=True, sparse_y_pred=True, axis=-1):
        super().__init__(name=name, dtype=dtype or "float32")
        self._direction = "up"
        self.num_classes = num_classes
        self.ignore_class = ignore_class
        self.sparse_y_true, self.sparse_y_pred, self.axis = sparse_y_true, sparse_y_pred, axis
        self.total_cm = self.add_variable(name="total_confusion_matrix", shape=(num_classes, num_classes), initializer=initializers.Zeros(), dtype=self.dtype)

    def update_state(self, y_true, y_pred, sample_weight=None):
        y_true, y_pred = convert_to_tensor(y_true), convert_to_tensor(y_pred)
        if not self.sparse_y_true:
            y_true = torch.argmax(y_true, dim=self.axis)
        if not self.sparse_y_pred:
            y_pred = torch.argmax(y_pred, dim=self.axis)
        y_true = y_true.reshape(-1).long()
        y_pred = y_pred.reshape(-1).long()
        if sample_weight is None:
            w = torch.ones_like(y_true, dtype=self.total_cm._torch_dtype)
        else:
            w = convert_to_tensor(sample_weight).to(self.total_cm._torch_dtype)
            w = torch.broadcast_to(w.reshape(-1) if w.numel() == y_true.numel() else w.reshape(-1, 1).expand(-1, y_true.numel() // max(w.numel(), 1)).reshape(-1), y_true.shape)
        if self.ignore_class is not None:
            valid = y_true != self.ignore_class
            y_true, y_pred, w = y_true[valid], y_pred[valid], w[valid]
        valid = (y_true >= 0) & (y_true < self.num_classes) & (y_pred >= 0) & (y_pred < self.num_classes)
        y_true, y_pred, w = y_true[valid], y_pred[valid], w[valid]
        cm = torch.zeros((self.num_classes * self.num_classes,), dtype=self.total_cm._torch_dtype, device=y_true.device)
        cm.index_add_(0, y_true * self.num_classes + y_pred, w)
        self.total_cm.assign(self.total_cm.value + cm.reshape(self.num_classes, self.num_classes).to(self.total_cm.value.device))

    def reset_state(self):
        self.total_cm.assign(torch.zeros((self.num_classes, self.num_classes)))


@keras_export("keras.metrics.IoU")
class IoU(_IoUBase):
    def __init__(self, num_classes, target_class_ids, name=None, dtype=None, ignore_class=None, sparse_y_true=True, sparse_y_pred=True, axis=-1):
        super().__init__(name=name, num_classes=num_classes, ignore_class=ignore_class, sparse_y_true=sparse_y_true, sparse_y_pred=sparse_y_pred, axis=axis, dtype=dtype)
        if max(target_class_ids) >= num_classes:
            raise ValueError(f"Target class id {max(target_class_ids)} is out of range, which is [{0}, {num_classes}).")
        self.target_class_ids = list(target_class_ids)

    def result(self):
        cm = self.total_cm.value
        sum_over_row = torch.sum(cm, dim=0)
        sum_over_col = torch.sum(cm, dim=1)
        tp = torch.diagonal(cm)
        denom = sum_over_row + sum_over_col - tp
        ids = torch.as_tensor(self.target_class_ids, device=cm.device)
        tp, denom = tp[ids], denom[ids]
        num_valid = torch.sum((denom != 0).to(cm.dtype))
        iou = _div_no_nan(tp, denom)
        return _div_no_nan(torch.sum(iou), num_valid)

    def get_config(self):
        return {"num_classes": self.num_classes, "target_class_ids": self.target_class_ids, "name": self.name, "dtype": self._dtype,
                "ignore_class": self.ignore_class, "sparse_y_true": self.sparse_y_true, "sparse_y_pred": self.sparse_y_pred, "axis": self.axis}


@keras_export("keras.metrics.BinaryIoU")
class BinaryIoU(IoU):
    def __init__(self, target_class_ids=(0, 1), threshold=0.5, name=None, dtype=None):
        super().__init__(num_classes=2, target_class_ids=target_class_ids, name=name, dtype=dtype)
        self.threshold = threshold

    def update_state(self, y_true, y_pred, sample_weight=None):
        y_pred = (convert_to_tensor(y_pred).float() >= self.threshold).to(torch.int64)
        return super().update_state(y_true, y_pred, sample_weight)

    def get_config(self):
        return {"target_class_ids": self.target_class_ids, "threshold": self.threshold, "name": self.name, "dtype": self._dtype}


@keras_export("keras.metrics.MeanIoU")
class MeanIoU(IoU):
    def __init__(self, num_classes, name=None, dtype=None, ignore_class=None, sparse_y_true=True, sparse_y_pred=True, axis=-1):
        target_class_ids = list(range(num_classes))
        super().__init__(name=name, num_classes=num_classes, target_class_ids=target_class_ids, axis=axis, dtype=dtype,
                         ignore_class=ignore_class, sparse_y_true=sparse_y_true, sparse_y_pred=sparse_y_pred)

    def get_config(self):
        return {"num_classes": self.num_classes, "name": self.name, "dtype": self._dtype, "ignore_class": self.ignore_class,
                "sparse_y_true": self.sparse_y_true, "sparse_y_pred": self.sparse_y_pred, "axis": self.axis}


@keras_export("keras.metrics.OneHotIoU")
class OneHotIoU(IoU):
    def __init__(self, num_classes, target_class_ids, name=None, dtype=None, ignore_class=None, sparse_y_pred=False, axis=-1):
        super().__init__(num_classes=num_classes, target_class_ids=target_class_ids, name=name, dtype=dtype, ignore_class=ignore_class,
                         sparse_y_true=False, sparse_y_pred=sparse_y_pred, axis=axis)

    def get_config(self):
        return {"num_classes": self.num_classes, "target_class_ids": self.target_class_ids, "name": self.name, "dtype": self._dtype,
                "ignore_class": self.ignore_class, "sparse_y_pred": self.sparse_y_pred, "axis": self.axis}


@keras_export("keras.metrics.OneHotMeanIoU")
class OneHotMeanIoU(MeanIoU):
    def __init__(self, num_classes, name=None, dtype=None, ignore_class=None, sparse_y_pred=False, axis=-1):
        super().__init__(num_classes=num_classes, axis=axis, name=name, dtype=dtype, ignore_class=ignore_class, sparse_y_true=False, sparse_y_pred=sparse_y_pred)

    def get_config(self):
        return {"num_classes": self.num_classes, "name": self.name, "dtype": self._dtype, "ignore_class": self.ignore_class,
                "sparse_y_pred": self.sparse_y_pred, "axis": self.axis}


@keras_export("keras.metrics.FBetaScore")
class FBetaScore(Metric):
    def __init__(self, average=None, beta=1.0, threshold=None, name="fbeta_score", dtype=None):
        super().__init__(name=name, dtype=dtype)
        self._direction = "up"
        if average not in (None, "micro", "macro", "weighted"):
            raise ValueError(f"Invalid `average` argument value. Expected one of: {{None, 'micro', 'macro', 'weighted'}}. Received: average={average}")
        if not isinstance(beta, float):
            raise ValueError(f"Invalid `beta` argument value. It should be a Python float. Received: beta={beta} of type '{type(beta)}'")
        if beta <= 0.0:
            raise ValueError(f"Invalid `beta` argument value. It should be > 0. Received: beta={beta}")
        if threshold is not None:
            if not isinstance(threshold, float):
                raise ValueError(f"Invalid `threshold` argument value. It should be a Python float. Received: threshold={threshold} of type '{type(threshold)}'")
            if threshold > 1.0 or threshold <= 0.0:
                raise ValueError(f"Invalid `threshold` argument value. It should verify 0 < threshold <= 1. Received: threshold={threshold}")
        self.average, self.beta, self.threshold = average, beta, threshold
        self.axis = None if average == "micro" else 0
        self._built = False

    def _build(self, y_true_shape, y_pred_shape):
        if len(y_pred_shape) != 2 or len(y_true_shape) != 2:
            raise ValueError(f"FBetaScore expects 2D inputs with shape (batch_size, output_dim). Received input shapes: y_pred.shape={y_pred_shape} and y_true.shape={y_true_shape}.")
        if y_pred_shape[-1] is None or y_true_shape[-1] is None:
            raise ValueError(f"FBetaScore expects 2D inputs with shape (batch_size, output_dim), with output_dim fully defined (not None). Received input shapes: y_pred.shape={y_pred_shape} and y_true.shape={y_true_shape}.")
        num_classes = y_pred_shape[-1]
        init_shape = () if self.average == "micro" else (num_classes,)
        for n in ("true_positives", "false_positives", "false_negatives", "intermediate_weights"):
            setattr(self, n, self.add_variable(name=n, shape=init_shape, initializer=initializers.Zeros(), dtype=self.dtype))
        self._built = True

    def update_state(self, y_true, y_pred, sample_weight=None):
        y_true = convert_to_tensor(y_true, dtype=self.dtype)
        y_pred = convert_to_tensor(y_pred, dtype=self.dtype)
        if not self._built:
            self._build(tuple(y_true.shape), tuple(y_pred.shape))
        if self.threshold is None:
            threshold = torch.amax(y_pred, dim=-1, keepdim=True)
            y_pred = torch.logical_and(y_pred >= threshold, torch.abs(y_pred) > 1e-9)
        else:
            y_pred = y_pred > self.threshold
        y_pred = y_pred.to(y_true.dtype)
        if sample_weight is not None:
            sample_weight = convert_to_tensor(sample_weight, dtype=self.dtype)

        def _weighted_sum(val, sw):
            if sw is not None:
                val = val * sw.unsqueeze(1) if sw.ndim == 1 else val * sw
            return torch.sum(val, dim=self.axis) if self.axis is not None else torch.sum(val)

        self.true_positives.assign(self.true_positives.value + _weighted_sum(y_pred * y_true, sample_weight))
        self.false_positives.assign(self.false_positives.value + _weighted_sum(y_pred * (1 - y_true), sample_weight))
        self.false_negatives.assign(self.false_negatives.value + _weighted_sum((1 - y_pred) * y_true, sample_weight))
        self.intermediate_weights.assign(self.intermediate_weights.value + _weighted_sum(y_true, sample_weight))

    def result(self):
        eps = config.epsilon()
        precision = self.true_positives.value / (self.true_positives.value + self.false_positives.value + eps)
        recall = self.true_positives.value / (self.true_positives.value + self.false_negatives.value + eps)
        precision = torch.where((self.true_positives.value + self.false_positives.value) == 0, torch.zeros_like(precision), precision) if False else precision
        mul = precision * recall
        add = (self.beta ** 2) * precision + recall
        mean = mul / (add + eps)
        f1 = mean * (1 + self.beta ** 2)
        if self.average == "weighted":
            weights = self.intermediate_weights.value / (torch.sum(self.intermediate_weights.value) + eps)
            f1 = torch.sum(f1 * weights)
        elif self.average is not None:
            f1 = torch.mean(f1)
        return f1

    def reset_state(self):
        for v in self.variables:
            v.assign(torch.zeros(tuple(v.shape), dtype=v._torch_dtype))

    def get_config(self):
        return {"name": self.name, "dtype": self.dtype, "average": self.average, "beta": self.beta, "threshold": self.threshold}


@keras_export("keras.metrics.F1Score")
class F1Score(FBetaScore):
    def __init__(self, average=None, threshold=None, name="f1_score", dtype=None):
        super().__init__(average=average, beta=1.0, threshold=threshold, name=name, dtype=dtype)

    def get_config(self):
        cfg = super().get_config()
        del cfg["beta"]
        return cfg


@keras_export("keras.metrics.pearson_correlation")
def pearson_correlation(y_true, y_pred, axis=-1):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
    yt = y_true - torch.mean(y_true, dim=axis, keepdim=True)
    yp = y_pred - torch.mean(y_pred, dim=axis, keepdim=True)
    yt = yt / torch.clamp(torch.linalg.vector_norm(yt, dim=axis, keepdim=True), min=1e-12)
    yp = yp / torch.clamp(torch.linalg.vector_norm(yp, dim=axis, keepdim=True), min=1e-12)
    return torch.sum(yt * yp, dim=axis)


@keras_export("keras.metrics.concordance_correlation")
def concordance_correlation(y_true, y_pred, axis=-1):
    y_pred = convert_to_tensor(y_pred)
    y_true = convert_to_tensor(y_true).to(y_pred.dtype)
    y_true, y_pred = squeeze_or_expand_to_same_rank(y_true, y_pred)
    mt, mp = torch.mean(y_true, dim=axis, keepdim=True), torch.mean(y_pred, dim=axis, keepdim=True)
    vt = torch.var(y_true - mt, dim=axis, keepdim=True, correction=0)
    vp = torch.var(y_pred - mp, dim=axis, keepdim=True, correction=0)
    cov = torch.mean((y_true - mt) * (y_pred - mp), dim=axis)
    return (2 * cov) / (vt.squeeze(axis) + vp.squeeze(axis) + torch.square(mt - mp).squeeze(axis) + config.epsilon())


@keras_export("keras.metrics.PearsonCorrelation")
class PearsonCorrelation(MeanMetricWrapper):
    def __init__(self, name="pearson_correlation", dtype=None, axis=-1):
        super().__init__(fn=pearson_correlation, name=name, dtype=dtype, axis=axis)
        self.axis = axis
        self._direction = "up"

    def get_config(self):
        return {"name": self.name, "dtype": self.dtype, "axis": self.axis}


@keras_export("keras.metrics.ConcordanceCorrelation")
class ConcordanceCorrelation(MeanMetricWrapper):
    def __init__(self, name="concordance_correlation", dtype=None, axis=-1):
        super().__init__(fn=concordance_correlation, name=name, dtype=dtype, axis=axis)
        self.axis = axis
        self._direction = "up"

    def get_config(self):
        return {"name": self.name, "dtype": self.dtype, "axis": self.axis}
