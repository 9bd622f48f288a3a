"""Confusion-matrix metrics (keras/src/metrics/confusion_metrics.py, metrics_utils.py):
TP/FP/TN/FN, Precision, Recall, the sensitivity/specificity family and AUC."""

import numpy as np
import torch

from keras_b200 import activations, initializers, ops
from keras_b200.core import config
from keras_b200.core.dtypes import to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.losses.loss import squeeze_or_expand_to_same_rank
from keras_b200.metrics.metric import Metric

NEG_INF = -1e10
_TP, _FP, _TN, _FN = "tp", "fp", "tn", "fn"


def parse_init_thresholds(thresholds, default_threshold=0.5):
    if thresholds is not None:
        for t in (thresholds if isinstance(thresholds, (list, tuple)) else [thresholds]):
            if t is None or t < 0 or t > 1:
                raise ValueError(f"Invalid value for argument `thresholds`. Threshold values must be in [0, 1]. Received: thresholds={thresholds}")
    if thresholds is None:
        return [default_threshold]
    return list(thresholds) if isinstance(thresholds, (list, tuple)) else [thresholds]


def is_evenly_distributed_thresholds(thresholds):
    n = thresholds.shape[0]
    if n < 3:
        return False
    even = np.arange(n, dtype=np.float32) / (n - 1)
    return np.allclose(thresholds, even, atol=config.epsilon())


def update_confusion_matrix_variables(variables_to_update, y_true, y_pred, thresholds, top_k=None, class_id=None,
                                      sample_weight=None, multi_label=False, label_weights=None, thresholds_distributed_evenly=False):
    """Accumulate tp/fp/tn/fn counts at every threshold into the given variables."""
    if multi_label and label_weights is not None:
        raise ValueError("`label_weights` for multilabel data should be handled outside of `update_confusion_matrix_variables` when `multi_label` is True.")
    if not variables_to_update:
        return
    some = next(iter(variables_to_update.values()))
    vtd = some._torch_dtype
    y_pred = convert_to_tensor(y_pred).to(vtd)
    y_true = convert_to_tensor(y_true).to(vtd)
    if sample_weight is not None:
        sample_weight = convert_to_tensor(sample_weight).to(vtd)
    thr = convert_to_tensor(np.asarray(thresholds, dtype="float32")).to(vtd).to(y_pred.device)
    one_thresh = not multi_label or thr.ndim == 1
    y_pred, y_true = squeeze_or_expand_to_same_rank(y_pred, y_true)
    if sample_weight is not None:
        y_true, sample_weight = squeeze_or_expand_to_same_rank(y_true, sample_weight, expand_rank_1=False)
    if top_k is not None:
        vals, idx = torch.topk(y_pred, top_k, dim=-1)
        mask = torch.zeros_like(y_pred, dtype=torch.bool).scatter_(-1, idx, True)
        y_pred = torch.where(mask, y_pred, torch.full_like(y_pred, NEG_INF))
    if class_id is not None:
        y_true = y_true[..., class_id, None] if y_true.ndim > 1 else y_true
        y_pred = y_pred[..., class_id, None] if y_pred.ndim > 1 else y_pred
    num_thresholds = thr.shape[0] if thr.ndim else 1
    if multi_label:
        num_labels = y_pred.shape[-1] if y_pred.ndim > 1 else 1
        yp = y_pred.reshape(1, -1, num_labels)
        yt = y_true.reshape(1, -1, num_labels)
        th = thr.reshape(-1, 1, 1) if one_thresh else thr.reshape(num_thresholds, 1, -1)
    else:
        yp = y_pred.reshape(1, -1)
        yt = y_true.reshape(1, -1)
        th = thr.reshape(-1, 1)
    pred_pos = yp > th
    label_pos = torch.broadcast_to(yt.to(torch.bool), pred_pos.shape)
    if sample_weight is not None:
        sw = torch.broadcast_to(sample_weight, y_pred.shape) if sample_weight.ndim == y_pred.ndim or sample_weight.ndim == 0 else torch.broadcast_to(sample_weight.reshape(sample_weight.shape + (1,) * (y_pred.ndim - sample_weight.ndim)), y_pred.shape)
        w = sw.reshape(yp.shape).to(vtd)
    else:
        w = None
    if label_weights is not None and not multi_label:
        lw = torch.broadcast_to(convert_to_tensor(label_weights).to(vtd).to(y_pred.device).reshape(1, -1), y_pred.reshape(-1, y_pred.shape[-1]).shape).reshape(yp.shape)
        w = lw if w is None else w * lw

    def acc(var, label, pred):
        hit = (label & pred).to(vtd)
        if w is not None:
            hit = hit * w
        var.assign(var.value + torch.sum(hit, dim=1).reshape(var.shape))

    if _TP in variables_to_update:
        acc(variables_to_update[_TP], label_pos, pred_pos)
    if _FN in variables_to_update:
        acc(variables_to_update[_FN], label_pos, ~pred_pos)
    if _FP in variables_to_update:
        acc(variables_to_update[_FP], ~label_pos, pred_pos)
    if _TN in variables_to_update:
        acc(variables_to_update[_TN], ~label_pos, ~pred_pos)


class _ConfusionMatrixConditionCount(Metric):
    def __init__(self, confusion_matrix_cond, thresholds=None, name=None, dtype=None):
        super().__init__(name=name, dtype=dtype)
        self._confusion_matrix_cond = confusion_matrix_cond
        self.init_thresholds = thresholds
        self.thresholds = parse_init_thresholds(thresholds, default_threshold=0.5)
        self._thresholds_distributed_evenly = is_evenly_distributed_thresholds(np.asarray(self.thresholds, dtype="float32"))
        self.accumulator = self.add_variable(shape=(len(self.thresholds),), initializer=initializers.Zeros(), name="accumulator")

    def update_state(self, y_true, y_pred, sample_weight=None):
        return update_confusion_matrix_variables({self._confusion_matrix_cond: self.accumulator}, y_true, y_pred,
                                                 thresholds=self.thresholds, sample_weight=sample_weight)

    def result(self):
        if len(self.thresholds) == 1:
            return self.accumulator.value[0]
        return self.accumulator.value

    def get_config(self):
        return {**super().get_config(), "thresholds": self.init_thresholds}


def _cond_class(name, cond):
    def __init__(self, thresholds=None, name=None, dtype=None):
        _ConfusionMatrixConditionCount.__init__(self, confusion_matrix_cond=cond, thresholds=thresholds, name=name, dtype=dtype)

    cls = type(name, (_ConfusionMatrixConditionCount,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(f"keras.metrics.{name}")(cls)


FalsePositives = _cond_class("FalsePositives", _FP)
FalseNegatives = _cond_class("FalseNegatives", _FN)
TrueNegatives = _cond_class("TrueNegatives", _TN)
TruePositives = _cond_class("TruePositives", _TP)


def _div_no_nan(a, b):
    return torch.where(b == 0, torch.zeros_like(a), a / torch.where(b == 0, torch.ones_like(b), b))


@keras_export("keras.metrics.Precision")
class Precision(Metric):
    def __init__(self, thresholds=None, top_k=None, class_id=None, name=None, dtype=None):
        super().__init__(name=name, dtype=dtype)
        self._direction = "up"
        self.init_thresholds = thresholds
        self.top_k, self.class_id = top_k, class_id
        default_threshold = 0.5 if top_k is None else NEG_INF
        self.thresholds = parse_init_thresholds(thresholds, default_threshold=default_threshold)
        self._thresholds_distributed_evenly = is_evenly_distributed_thresholds(np.asarray(self.thresholds, dtype="float32"))
        self.true_positives = self.add_variable(shape=(len(self.thresholds),), initializer=initializers.Zeros(), name="true_positives")
        self.false_positives = self.add_variable(shape=(len(self.thresholds),), initializer=initializers.Zeros(), name="false_positives")

    def update_state(self, y_true, y_pred, sample_weight=None):
        update_confusion_matrix_variables({_TP: self.true_positives, _FP: self.false_positives}, y_true, y_pred,
                                          thresholds=self.thresholds, top_k=self.top_k, class_id=self.class_id, sample_weight=sample_weight)

    def result(self):
        r = _div_no_nan(self.true_positives.value, self.true_positives.value + self.false_positives.value)
        return r[0] if len(self.thresholds) == 1 else r

    def reset_state(self):
        n = len(self.thresholds)
        self.true_positives.assign(torch.zeros((n,)))
        self.false_positives.assign(torch.zeros((n,)))

    def get_config(self):
        return {**super().get_config(), "thresholds": self.init_thresholds, "top_k": self.top_k, "class_id": self.class_id}


@keras_export("keras.metrics.Recall")
class Recall(Metric):
    def __init__(self, thresholds=None, top_k=None, class_id=None, name=None, dtype=None):
        super().__init__(name=name, dtype=dtype)
        self._direction = "up"
        self.init_thresholds = thresholds
        self.top_k, self.class_id = top_k, class_id
        default_threshold = 0.5 if top_k is None else NEG_INF
        self.thresholds = parse_init_thresholds(thresholds, default_threshold=default_threshold)
        self.true_positives = self.add_variable(shape=(len(self.thresholds),), initializer=initializers.Zeros(), name="true_positives")
        self.false_negatives = self.add_variable(shape=(len(self.thresholds),), initializer=initializers.Zeros(), name="false_negatives")

    def update_state(self, y_true, y_pred, sample_weight=None):
        update_confusion_matrix_variables({_TP: self.true_positives, _FN: self.false_negatives}, y_true, y_pred,
                                          thresholds=self.thresholds, top_k=self.top_k, class_id=self.class_id, sample_weight=sample_weight)

    def result(self):
        r = _div_no_nan(self.true_positives.value, self.true_positives.value + self.false_negatives.value)
        return r[0] if len(self.thresholds) == 1 else r

    def reset_state(self):
        n = len(self.thresholds)
        self.true_positives.assign(torch.zeros((n,)))
        self.false_negatives.assign(torch.zeros((n,)))

    def get_config(self):
        return {**super().get_config(), "thresholds": self.init_thresholds, "top_k": self.top_k, "class_id": self.class_id}


class SensitivitySpecificityBase(Metric):
    def __init__(self, value, num_thresholds=200, class_id=None, name=None, dtype=None):
        super().__init__(name=name, dtype=dtype)
        self._direction = "up"
        if num_thresholds <= 0:
            raise ValueError(f"Argument `num_thresholds` must be an integer > 0. Received: num_thresholds={num_thresholds}")
        self.value = value
        self.class_id = class_id
        if num_thresholds == 1:
            self.thresholds = [0.5]
            self._thresholds_distributed_evenly = False
        else:
            thresholds = [(i + 1) * 1.0 / (num_thresholds - 1) for i in range(num_thresholds - 2)]
            self.thresholds = [0.0] + thresholds + [1.0]
            self._thresholds_distributed_evenly = True
        for n in ("true_positives", "false_positives", "true_negatives", "false_negatives"):
            setattr(self, n, self.add_variable(shape=(len(self.thresholds),), initializer=initializers.Zeros(), name=n))

    def update_state(self, y_true, y_pred, sample_weight=None):
        update_confusion_matrix_variables(
            {_TP: self.true_positives, _TN: self.true_negatives, _FP: self.false_positives, _FN: self.false_negatives},
            y_true, y_pred, thresholds=self.thresholds, class_id=self.class_id, sample_weight=sample_weight)

    def reset_state(self):
        n = len(self.thresholds)
        for v in (self.true_positives, self.false_positives, self.true_negatives, self.false_negatives):
            v.assign(torch.zeros((n,)))

    def _find_max_under_constraint(self, constrained, dependent, predicate):
        feasible = predicate(constrained, self.value)
        masked = torch.where(feasible, dependent, torch.full_like(dependent, -1.0))
        best = torch.amax(masked)
        return torch.where(torch.any(feasible), best, torch.zeros_like(best))

    def get_config(self):
        return {**super().get_config(), "class_id": self.class_id}


def _sens(self):
    return _div_no_nan(self.true_positives.value, self.true_positives.value + self.false_negatives.value)


def _spec(self):
    return _div_no_nan(self.true_negatives.value, self.true_negatives.value + self.false_positives.value)


def _prec(self):
    return _div_no_nan(self.true_positives.value, self.true_positives.value + self.false_positives.value)


def _ss_class(name, arg, constrained_fn, dependent_fn):
    def __init__(self, *args, num_thresholds=200, class_id=None, name=None, dtype=None, **kwargs):
        value = args[0] if args else kwargs.pop(arg)
        if value < 0 or value > 1:
            raise ValueError(f"Argument `{arg}` must be in the range [0, 1]. Received: {arg}={value}")
        setattr(self, arg, value)
        self.num_thresholds = num_thresholds
        SensitivitySpecificityBase.__init__(self, value, num_thresholds=num_thresholds, class_id=class_id, name=name, dtype=dtype)

    def result(self):
        return self._find_max_under_constraint(constrained_fn(self), dependent_fn(self), torch.greater_equal)

    def get_config(self):
        cfg = SensitivitySpecificityBase.get_config(self)
        cfg.update({"num_thresholds": self.num_thresholds, arg: getattr(self, arg)})
        return cfg

    cls = type(name, (SensitivitySpecificityBase,), {"__init__": __init__, "result": result, "get_config": get_config})
    cls.__module__ = __name__
    return keras_export(f"keras.metrics.{name}")(cls)


SensitivityAtSpecificity = _ss_class("SensitivityAtSpecificity", "specificity", _spec, _sens)
SpecificityAtSensitivity = _ss_class("SpecificityAtSensitivity", "sensitivity", _sens, _spec)
PrecisionAtRecall = _ss_class("PrecisionAtRecall", "recall", _sens, _prec)
RecallAtPrecision = _ss_class("RecallAtPrecision", "precision", _prec, _sens)


@keras_export("keras.metrics.AUC")
class AUC(Metric):
    def __init__(self, num_thresholds=200, curve="ROC", summation_method="interpolation", name=None, dtype=None, thresholds=None,
                 multi_label=False, num_labels=None, label_weights=None, from_logits=False):
        self._direction = "up"
        if curve not in ("ROC", "PR", "roc", "pr"):
            raise ValueError(f'Invalid `curve` argument value "{curve}". Expected one of: ["ROC", "PR"]')
        if summation_method not in ("interpolation", "majoring", "minoring"):
            raise ValueError(f'Invalid `summation_method` argument value "{summation_method}". Expected one of: ["interpolation", "majoring", "minoring"]')
        self._init_from_thresholds = thresholds is not None
        if thresholds is not None:
            self.num_thresholds = len(thresholds) + 2
            thresholds = sorted(thresholds)
            self._thresholds_distributed_evenly = is_evenly_distributed_thresholds(np.array([0.0] + thresholds + [1.0]))
        else:
            if num_thresholds <= 1:
                raise ValueError(f"Argument `num_thresholds` must be an integer > 1. Received: num_thresholds={num_thresholds}")
            self.num_thresholds = num_thresholds
            thresholds = [(i + 1) * 1.0 / (num_thresholds - 1) for i in range(num_thresholds - 2)]
            self._thresholds_distributed_evenly = True
        self._thresholds = np.array([0.0 - config.epsilon()] + thresholds + [1.0 + config.epsilon()])
        self.curve = curve.upper()
        self.summation_method = summation_method
        super().__init__(name=name, dtype=dtype)
        self.multi_label = multi_label
        self.num_labels = num_labels
        if label_weights is not None:
            label_weights = np.asarray(label_weights, dtype=self.dtype)
            if (label_weights < 0).any():
                raise ValueError("All values of `label_weights` must be non-negative.")
        self.label_weights = label_weights
        self._from_logits = from_logits
        self._built = False
        if self.multi_label:
            if num_labels:
                self._build((None, num_labels))
        else:
            if num_labels:
                raise ValueError("`num_labels` is needed only when `multi_label` is True.")
            self._build(None)

    @property
    def thresholds(self):
        return list(self._thresholds)

    def _build(self, shape):
        if self.multi_label:
            if len(shape) != 2:
                raise ValueError(f"`y_pred` must have rank 2 when `multi_label=True`. Found rank {len(shape)}. Full shape received for `y_pred`: {shape}")
            self._num_labels = shape[1]
            variable_shape = [self.num_thresholds, self._num_labels]
        else:
            variable_shape = [self.num_thresholds]
        self._build_input_shape = shape
        for n in ("true_positives", "false_positives", "true_negatives", "false_negatives"):
            setattr(self, n, self.add_variable(shape=variable_shape, initializer=initializers.Zeros(), name=n))
        self._built = True

    def update_state(self, y_true, y_pred, sample_weight=None):
        if not self._built:
            self._build(tuple(y_pred.shape))
        y_pred = convert_to_tensor(y_pred)
        if self._from_logits:
            y_pred = torch.sigmoid(y_pred.float())
        label_weights = None if self.multi_label else self.label_weights
        update_confusion_matrix_variables(
            {_TP: self.true_positives, _TN: self.true_negatives, _FP: self.false_positives, _FN: self.false_negatives},
            y_true, y_pred, self._thresholds, thresholds_distributed_evenly=self._thresholds_distributed_evenly,
            sample_weight=sample_weight, multi_label=self.multi_label, label_weights=label_weights)

    def interpolate_pr_auc(self):
        tp, fp, fn = self.true_positives.value, self.false_positives.value, self.false_negatives.value
        n = self.num_thresholds
        dtp = tp[: n - 1] - tp[1:]
        p = tp + fp
        dp = p[: n - 1] - p[1:]
        prec_slope = _div_no_nan(dtp, torch.clamp(dp, min=0))
        intercept = tp[1:] - prec_slope * p[1:]
        safe_p_ratio = torch.where((p[: n - 1] > 0) & (p[1:] > 0), _div_no_nan(p[: n - 1], torch.clamp(p[1:], min=0)), torch.ones_like(p[1:]))
        pr_auc_increment = _div_no_nan(prec_slope * (dtp + intercept * torch.log(safe_p_ratio)), torch.clamp(tp[1:] + fn[1:], min=0))
        if self.multi_label:
            by_label_auc = torch.sum(pr_auc_increment, dim=0)
            if self.label_weights is None:
                return torch.mean(by_label_auc)
            lw = convert_to_tensor(self.label_weights).to(by_label_auc.device)
            return _div_no_nan(torch.sum(by_label_auc * lw), torch.sum(lw))
        return torch.sum(pr_auc_increment)

    def result(self):
        if self.curve == "PR" and self.summation_method == "interpolation":
            return self.interpolate_pr_auc()
        tp, fp, tn, fn = self.true_positives.value, self.false_positives.value, self.true_negatives.value, self.false_negatives.value
        recall = _div_no_nan(tp, tp + fn)
        if self.curve == "ROC":
            x, y = _div_no_nan(fp, fp + tn), recall
        else:
            x, y = recall, _div_no_nan(tp, tp + fp)
        n = self.num_thresholds
        if self.summation_method == "interpolation":
            heights = (y[: n - 1] + y[1:]) / 2.0
        elif self.summation_method == "minoring":
            heights = torch.minimum(y[: n - 1], y[1:])
        else:
            heights = torch.maximum(y[: n - 1], y[1:])
        if self.multi_label:
            riemann = torch.sum((x[: n - 1] - x[1:]) * heights, dim=0)
            if self.label_weights is None:
                return torch.mean(riemann)
            lw = convert_to_tensor(self.label_weights).to(riemann.device)
            return _div_no_nan(torch.sum(riemann * lw), torch.sum(lw))
        return torch.sum((x[: n - 1] - x[1:]) * heights)

    def reset_state(self):
        if self._built:
            shape = (self.num_thresholds, self._num_labels) if self.multi_label else (self.num_thresholds,)
            for v in (self.true_positives, self.false_positives, self.true_negatives, self.false_negatives):
                v.assign(torch.zeros(shape))

    def get_config(self):
        label_weights = self.label_weights
        cfg = {"num_thresholds": self.num_thresholds, "curve": self.curve, "summation_method": self.summation_method,
               "multi_label": self.multi_label, "num_labels": self.num_labels,
               "label_weights": None if label_weights is None else label_weights.tolist(), "from_logits": self._from_logits}
        if self._init_from_thresholds:
            cfg["thresholds"] = self.thresholds[1:-1]
        return {**super().get_config(), **cfg}
