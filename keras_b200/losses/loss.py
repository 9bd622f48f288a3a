"""``Loss`` base class and the weighted reduction helpers.

Behaviour of keras/src/losses/loss.py:11-258: reductions ``sum_over_batch_size`` (default),
``sum``, ``mean``, ``mean_with_sample_weight``, ``none``; masks fold into sample weights.
"""

import torch

from keras_b200 import dtype_policies, tree
from keras_b200.core import config
from keras_b200.core.dtypes import to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import auto_name
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.ops.operation import KerasSaveable


@keras_export(["keras.Loss", "keras.losses.Loss"])
class Loss(KerasSaveable):
    def __init__(self, name=None, reduction="sum_over_batch_size", dtype=None):
        self.name = name or auto_name(self.__class__.__name__)
        self.reduction = standardize_reduction(reduction)
        self._dtype_policy = dtype_policies.get(dtype or config.floatx())
        self._dtype = self._dtype_policy.compute_dtype

    @property
    def dtype(self):
        return self._dtype

    def _accepts_low_precision(self, y_pred):
        """True when ``call`` computes in float32 from half-precision predictions by itself (no up-cast copy needed)."""
        return False

    def __call__(self, y_true, y_pred, sample_weight=None):
        in_mask = getattr(y_pred, "_keras_mask", None)
        td = to_torch_dtype(self.dtype)
        if not self._accepts_low_precision(y_pred):
            y_pred = tree.map_structure(lambda x: convert_to_tensor(x, dtype=td), y_pred)
        y_true = tree.map_structure(lambda x: _convert_true(x, td), y_true)
        losses = self.call(y_true, y_pred)
        out_mask = getattr(losses, "_keras_mask", None)
        if in_mask is not None and out_mask is not None:
            mask = in_mask & out_mask
        elif in_mask is not None:
            mask = in_mask
        elif out_mask is not None:
            mask = out_mask
        else:
            mask = None
        return reduce_weighted_values(losses, sample_weight=sample_weight, mask=mask, reduction=self.reduction, dtype=self.dtype)

    def call(self, y_true, y_pred):
        raise NotImplementedError

    def get_config(self):
        return {"name": self.name, "reduction": self.reduction}

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def _obj_type(self):
        return "Loss"


def _convert_true(x, td):
    t = convert_to_tensor(x)
    return t.to(td) if t.dtype != td else t


def standardize_reduction(reduction):
    allowed = {"sum_over_batch_size", "sum", None, "none", "mean", "mean_with_sample_weight"}
    if reduction not in allowed:
        raise ValueError(f"Invalid value for argument `reduction`. Expected one of {allowed}. Received: reduction={reduction}")
    return reduction


def squeeze_or_expand_to_same_rank(x1, x2, expand_rank_1=True):
    r1, r2 = x1.ndim, x2.ndim
    if r1 == r2:
        return x1, x2
    if r1 == r2 + 1:
        if x1.shape[-1] == 1:
            if r2 == 1 and expand_rank_1:
                x2 = x2.unsqueeze(-1)
            else:
                x1 = x1.squeeze(-1)
    if r2 == r1 + 1:
        if x2.shape[-1] == 1:
            if r1 == 1 and expand_rank_1:
                x1 = x1.unsqueeze(-1)
            else:
                x2 = x2.squeeze(-1)
    return x1, x2


def reduce_values(values, sample_weight=None, reduction="sum_over_batch_size"):
    if reduction is None or reduction == "none" or values.ndim == 0:
        return values
    loss = torch.sum(values)
    if reduction in ("sum_over_batch_size", "mean", "mean_with_sample_weight"):
        if reduction == "mean_with_sample_weight" and sample_weight is not None:
            divisor = torch.sum(sample_weight).to(loss.dtype)
        else:
            divisor = values.numel()
        if isinstance(divisor, torch.Tensor):
            loss = torch.where(divisor == 0, torch.zeros_like(loss), loss / torch.where(divisor == 0, torch.ones_like(divisor), divisor))
        else:
            loss = loss / divisor if divisor else torch.zeros_like(loss)
    return loss


def reduce_weighted_values(values, sample_weight=None, mask=None, reduction="sum_over_batch_size", dtype=None):
    reduction = standardize_reduction(reduction)
    td = to_torch_dtype(dtype) if dtype is not None else None
    values = convert_to_tensor(values, dtype=td)
    if sample_weight is not None:
        sample_weight = convert_to_tensor(sample_weight, dtype=td)
    if mask is not None:
        mask = convert_to_tensor(mask, dtype=td)
    sample_weight = apply_mask(sample_weight, mask, dtype=values.dtype, reduction=reduction)
    if sample_weight is not None:
        sample_weight = sample_weight.to(values.dtype)
        values, sample_weight = squeeze_or_expand_to_same_rank(values, sample_weight)
        values = values * sample_weight
    return reduce_values(values, sample_weight, reduction)


def apply_mask(sample_weight, mask, dtype, reduction):
    if mask is None:
        return sample_weight
    mask = mask.to(dtype)
    if reduction in ("mean", "sum_over_batch_size"):
        # valid entries weigh total/valid, so that the mean over all entries is the mean over the valid ones; no valid entry: 0
        valid = torch.sum(mask)
        weight = torch.where(valid == 0, torch.zeros_like(valid), float(mask.numel()) / valid)
        mask = torch.where(mask.to(torch.bool), weight, torch.zeros_like(weight))
    if sample_weight is not None:
        sample_weight = sample_weight.to(dtype)
        mask, sample_weight = squeeze_or_expand_to_same_rank(mask, sample_weight)
        return sample_weight * mask
    return mask
