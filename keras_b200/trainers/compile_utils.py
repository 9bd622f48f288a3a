"""Mapping of user-provided losses / metrics onto model outputs.

Behaviour of keras/src/trainers/compile_utils.py:15-853: ``"accuracy"`` / ``"crossentropy"``
resolve from shapes (:40-127); nested output structures; loss weights; per-output loss trackers.
"""

from collections import namedtuple

import torch

from keras_b200 import losses as losses_module
from keras_b200 import metrics as metrics_module
from keras_b200 import ops, tree
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.losses.loss import Loss


class MetricsList(metrics_module.Metric):
    def __init__(self, metrics, name="metrics_list", output_name=None):
        super().__init__(name=name)
        self.metrics = metrics
        self.output_name = output_name

    def update_state(self, y_true, y_pred, sample_weight=None):
        for m in self.metrics:
            m.update_state(y_true, y_pred, sample_weight=sample_weight)

    def reset_state(self):
        for m in self.metrics:
            m.reset_state()

    def get_result(self):
        return {m.name: m.result() for m in self.metrics}

    def get_config(self):
        raise NotImplementedError

    @classmethod
    def from_config(cls, config):
        raise NotImplementedError


def is_function_like(value):
    if value is None:
        return True
    if isinstance(value, str):
        return True
    if callable(value):
        return True
    return False


def is_binary_or_sparse_categorical(y_true, y_pred):
    y_t_rank = len(y_true.shape)
    y_p_rank = len(y_pred.shape)
    y_t_last_dim = y_true.shape[-1] if y_t_rank else None
    y_p_last_dim = y_pred.shape[-1] if y_p_rank else None
    is_binary = y_p_last_dim == 1
    is_sparse_categorical = y_t_rank < y_p_rank or (y_t_last_dim == 1 and y_p_last_dim > 1)
    return is_binary, is_sparse_categorical


def get_metric(identifier, y_true, y_pred):
    if identifier is None:
        return None
    if str(identifier).lower() not in ["accuracy", "acc"]:
        metric_obj = metrics_module.get(identifier)
    else:
        is_binary, is_sparse = is_binary_or_sparse_categorical(y_true, y_pred)
        if is_binary:
            metric_obj = metrics_module.BinaryAccuracy(name=str(identifier))
        elif is_sparse:
            metric_obj = metrics_module.SparseCategoricalAccuracy(name=str(identifier))
        else:
            metric_obj = metrics_module.CategoricalAccuracy(name=str(identifier))
    if isinstance(identifier, str):
        metric_name = identifier
    else:
        metric_name = getattr(metric_obj, "name", None) or getattr(metric_obj, "__name__", "metric")
    if not isinstance(metric_obj, metrics_module.Metric):
        metric_obj = metrics_module.MeanMetricWrapper(metric_obj)
    metric_obj.name = metric_name
    return metric_obj


def get_loss(identifier, y_true, y_pred):
    if identifier is None:
        return None
    if str(identifier).lower() not in ["crossentropy", "ce"]:
        loss_obj = losses_module.get(identifier)
    else:
        is_binary, is_sparse = is_binary_or_sparse_categorical(y_true, y_pred)
        if is_binary:
            loss_obj = losses_module.binary_crossentropy
        elif is_sparse:
            loss_obj = losses_module.sparse_categorical_crossentropy
        else:
            loss_obj = losses_module.categorical_crossentropy
    if not isinstance(loss_obj, Loss):
        if isinstance(identifier, str):
            loss_name = identifier
        else:
            loss_name = getattr(loss_obj, "__name__", None) or type(loss_obj).__name__
        loss_obj = losses_module.LossFunctionWrapper(loss_obj, name=loss_name)
    return loss_obj


class CompileMetrics(metrics_module.Metric):
    def __init__(self, metrics, weighted_metrics, name="compile_metric", output_names=None):
        super().__init__(name=name)
        if metrics and not isinstance(metrics, (list, tuple, dict)):
            raise ValueError(f"Expected `metrics` argument to be a list, tuple, or dict. Received instead: metrics={metrics} of type {type(metrics)}")
        if weighted_metrics and not isinstance(weighted_metrics, (list, tuple, dict)):
            raise ValueError(f"Expected `weighted_metrics` argument to be a list, tuple, or dict. Received instead: weighted_metrics={weighted_metrics} of type {type(weighted_metrics)}")
        self._user_metrics = metrics
        self._user_weighted_metrics = weighted_metrics
        self.built = False
        self.name = "compile_metrics"
        self.output_names = output_names

    @property
    def metrics(self):
        if not self.built:
            return []
        out = []
        for group in (self._flat_metrics, self._flat_weighted_metrics):
            for m in group:
                if isinstance(m, MetricsList):
                    out.extend(m.metrics)
                elif m is not None:
                    out.append(m)
        return out

    @property
    def variables(self):
        if not self.built:
            return []
        v = []
        for m in self.metrics:
            v.extend(m.variables)
        return v

    def build(self, y_true, y_pred):
        num_outputs = 1
        if self.output_names:
            output_names = self.output_names
        elif isinstance(y_pred, dict):
            output_names = sorted(list(y_pred.keys()))
        elif isinstance(y_pred, (list, tuple)):
            num_outputs = len(y_pred)
            if all(hasattr(x, "_keras_history") for x in y_pred):
                output_names = [x._keras_history.operation.name for x in y_pred]
            else:
                output_names = None
        else:
            output_names = None
        if output_names:
            num_outputs = len(output_names)
        y_pred = self._flatten_y(y_pred)
        y_true = self._flatten_y(y_true)
        self._flat_metrics = self._build_metrics_set(self._user_metrics, num_outputs, output_names, y_true, y_pred, argument_name="metrics")
        self._flat_weighted_metrics = self._build_metrics_set(self._user_weighted_metrics, num_outputs, output_names, y_true, y_pred, argument_name="weighted_metrics")
        self.built = True

    def _build_metrics_set(self, metrics, num_outputs, output_names, y_true, y_pred, argument_name):
        flat = []
        if isinstance(metrics, dict):
            for name in metrics.keys():
                if name not in (output_names or []):
                    raise ValueError(f"In the dict argument `{argument_name}`, key '{name}' does not correspond to any model output. Received:\n{argument_name}={metrics}")
        if num_outputs == 1:
            if not metrics:
                flat.append(None)
            else:
                if isinstance(metrics, dict):
                    metrics = tree.flatten(metrics)
                if not isinstance(metrics, list):
                    metrics = [metrics]
                if not all(is_function_like(m) for m in metrics):
                    raise ValueError(f"Expected all entries in the `{argument_name}` list to be metric objects. Received instead:\n{argument_name}={metrics}")
                flat.append(MetricsList([get_metric(m, y_true[0], y_pred[0]) for m in metrics if m is not None]))
        else:
            if isinstance(metrics, (list, tuple)):
                if len(metrics) != len(y_pred):
                    raise ValueError(f"For a model with multiple outputs, when providing the `{argument_name}` argument as a list, it should have as many entries as the model has outputs. Received:\n{argument_name}={metrics}\nof length {len(metrics)} whereas the model has {len(y_pred)} outputs.")
                for idx, (mls, yt, yp) in enumerate(zip(metrics, y_true, y_pred)):
                    if not isinstance(mls, list):
                        mls = [mls]
                    name = output_names[idx] if output_names else None
                    if not all(is_function_like(e) for e in mls):
                        raise ValueError(f"All entries in the sublists of the `{argument_name}` list should be metric objects. Found the following sublist with unknown types: {mls}")
                    flat.append(MetricsList([get_metric(m, yt, yp) for m in mls if m is not None], output_name=name))
            elif isinstance(metrics, dict):
                if output_names is None:
                    raise ValueError(f"Argument `{argument_name}` can only be provided as a dict when the model also returns a dict of outputs. Received {argument_name}={metrics}")
                for name in metrics.keys():
                    if not isinstance(metrics[name], list):
                        metrics[name] = [metrics[name]]
                    if not all(is_function_like(e) for e in metrics[name]):
                        raise ValueError(f"All entries in the sublists of the `{argument_name}` dict should be metric objects. At key '{name}', found the following sublist with unknown types: {metrics[name]}")
                for name, yt, yp in zip(output_names, y_true, y_pred):
                    if name in metrics:
                        flat.append(MetricsList([get_metric(m, yt, yp) for m in metrics[name] if m is not None], output_name=name))
                    else:
                        flat.append(None)
            else:
                flat = [None] * num_outputs
        return flat

    def _flatten_y(self, y):
        names = self.output_names
        if isinstance(y, dict) and names:
            out = []
            for n in names:
                if n in y:
                    out.append(y[n])
            return out
        return tree.flatten(y)

    def update_state(self, y_true, y_pred, sample_weight=None):
        if not self.built:
            self.build(y_true, y_pred)
        y_true = self._flatten_y(y_true)
        y_pred = self._flatten_y(y_pred)
        for m, yt, yp in zip(self._flat_metrics, y_true, y_pred):
            if m:
                m.update_state(yt, yp)
        if sample_weight is not None:
            sample_weight = self._flatten_y(sample_weight)
            if len(sample_weight) < len(y_true):
                sample_weight = sample_weight + [None] * (len(y_true) - len(sample_weight))
        else:
            sample_weight = [None] * len(y_true)
        for m, yt, yp, s in zip(self._flat_weighted_metrics, y_true, y_pred, sample_weight):
            if m:
                m.update_state(yt, yp, s)

    def reset_state(self):
        if not self.built:
            return
        for m in self._flat_metrics + self._flat_weighted_metrics:
            if m:
                m.reset_state()

    def result(self):
        if not self.built:
            raise ValueError("Cannot get result() since the metric has not yet been built.")
        results = {}
        unique_name_counters = {}
        for mls in self._flat_metrics:
            if not mls:
                continue
            for m in mls.metrics:
                name = m.name
                if mls.output_name:
                    name = f"{mls.output_name}_{name}"
                if name not in unique_name_counters:
                    results[name] = m.result()
                    unique_name_counters[name] = 1
                else:
                    index = unique_name_counters[name]
                    unique_name_counters[name] += 1
                    name = f"{name}_{index}"
                    results[name] = m.result()
        for mls in self._flat_weighted_metrics:
            if not mls:
                continue
            for m in mls.metrics:
                name = m.name
                if mls.output_name:
                    name = f"{mls.output_name}_{name}"
                if name not in unique_name_counters:
                    results[name] = m.result()
                    unique_name_counters[name] = 1
                else:
                    name = f"weighted_{m.name}"
                    if mls.output_name:
                        name = f"{mls.output_name}_{name}"
                    if name not in unique_name_counters:
                        unique_name_counters[name] = 1
                    else:
                        index = unique_name_counters[name]
                        unique_name_counters[name] += 1
                        name = f"{name}_{index}"
                    results[name] = m.result()
        return results

    def get_config(self):
        raise NotImplementedError

    @classmethod
    def from_config(cls, config):
        raise NotImplementedError


class CompileLoss(Loss):
    Loss_ = namedtuple("Loss", ["path", "loss", "loss_weights", "name"])

    def __init__(self, loss, loss_weights=None, reduction="sum_over_batch_size", output_names=None):
        if loss_weights and not isinstance(loss_weights, (list, tuple, dict, float)):
            raise ValueError(f"Expected `loss_weights` argument to be a float (single output case) or a list, tuple, or dict (multiple output case). Received instead: loss_weights={loss_weights} of type {type(loss_weights)}")
        self._user_loss = loss
        self._user_loss_weights = loss_weights
        self.built = False
        self.output_names = output_names
        super().__init__(name="compile_loss", reduction=reduction)
        self._metrics = []
        self._tracked_metrics = []
        self._flat_losses = None
        self._y_pred_build_structure = None
        self._y_true_build_structure = None

    @property
    def metrics(self):
        return self._metrics

    @property
    def variables(self):
        v = []
        for m in self.metrics:
            v.extend(m.variables)
        return v

    def _build_nested(self, y_true, y_pred, loss, output_names, current_path):
        flat_y_pred = tree.flatten(y_pred)
        if not tree.is_nested(loss):
            _loss = loss.loss if isinstance(loss, CompileLoss.Loss_) else loss
            if _loss is None:
                return
            if isinstance(y_pred, (list, tuple)) and not isinstance(y_true, (list, tuple)) and False:
                pass
            if tree.is_nested(y_pred) and len(flat_y_pred) > 1:
                # one loss for many outputs: apply to every output
                _loss_obj = _loss
                for i, (yt, yp) in enumerate(zip(tree.flatten(y_true), flat_y_pred)):
                    name = output_names[i] if output_names else None
                    self._flat_losses.append(CompileLoss.Loss_(current_path + (i,), get_loss(_loss_obj, yt, yp), None, name))
                return
            yt = tree.flatten(y_true)[0] if tree.is_nested(y_true) else y_true
            yp = flat_y_pred[0] if tree.is_nested(y_pred) else y_pred
            name = output_names[0] if output_names else None
            self._flat_losses.append(CompileLoss.Loss_(current_path, get_loss(_loss, yt, yp), None, name))
            return
        if isinstance(loss, dict):
            if isinstance(y_pred, dict):
                keys = list(y_pred.keys())
                for k in loss:
                    if k not in keys:
                        raise KeyError(f"The path: {current_path + (k,)} in the `loss` argument, can't be found in the model's output (`y_pred`).")
                for k in keys:
                    if k in loss:
                        self._build_nested(y_true[k], y_pred[k], loss[k], [k], current_path + (k,))
            else:
                # dict of losses keyed by output name, outputs are a list
                names = output_names or []
                for k in loss:
                    if k not in names:
                        raise KeyError(f"The path: {current_path + (k,)} in the `loss` argument, can't be found in the model's output (`y_pred`).")
                ypl = list(y_pred) if isinstance(y_pred, (list, tuple)) else [y_pred]
                ytl = list(y_true) if isinstance(y_true, (list, tuple)) else ([y_true[n] for n in names] if isinstance(y_true, dict) else [y_true])
                for i, n in enumerate(names):
                    if n in loss and loss[n] is not None:
                        self._flat_losses.append(CompileLoss.Loss_(current_path + (i,), get_loss(loss[n], ytl[i], ypl[i]), None, n))
            return
        if isinstance(loss, (list, tuple)):
            ypl = list(y_pred) if isinstance(y_pred, (list, tuple)) else ([y_pred[k] for k in (output_names or sorted(y_pred))] if isinstance(y_pred, dict) else [y_pred])
            ytl = list(y_true) if isinstance(y_true, (list, tuple)) else ([y_true[k] for k in (output_names or sorted(y_true))] if isinstance(y_true, dict) else [y_true])
            if len(loss) != len(ypl):
                raise ValueError(f"For a model with multiple outputs, when providing the `loss` argument as a list, it should have as many entries as the model has outputs. Received:\nloss={loss}\nof length {len(loss)} whereas the model has {len(ypl)} outputs.")
            for i, l in enumerate(loss):
                if l is None:
                    continue
                name = output_names[i] if output_names else None
                key = i if not isinstance(y_pred, dict) else (output_names or sorted(y_pred))[i]
                self._flat_losses.append(CompileLoss.Loss_(current_path + (key,), get_loss(l, ytl[i], ypl[i]), None, name))
            return
        raise TypeError(f"Unsupported type {type(loss)} in the `loss` configuration.")

    def build(self, y_true, y_pred):
        loss = self._user_loss
        loss_weights = self._user_loss_weights
        flat_output_names = self.output_names
        if self.output_names and isinstance(self._user_loss, dict) and not isinstance(y_pred, dict):
            pass
        if isinstance(y_pred, dict):
            flat_output_names = flat_output_names or sorted(y_pred.keys())
        self._flat_losses = []
        if isinstance(y_pred, dict) and isinstance(loss, dict):
            # keep dict order of outputs sorted by key (flatten order)
            pass
        self._build_nested(y_true, y_pred, loss, flat_output_names, ())
        # loss weights
        n = len(self._flat_losses)
        if loss_weights is None:
            weights = [None] * n
        elif isinstance(loss_weights, (int, float)):
            weights = [float(loss_weights)] * n
        elif isinstance(loss_weights, (list, tuple)):
            if len(loss_weights) != n:
                raise ValueError(f"When providing the `loss_weights` argument as a list, it should have as many entries as the model has outputs. Received: loss_weights={loss_weights} of length {len(loss_weights)} whereas the model has {n} outputs.")
            if not all(isinstance(e, (int, float)) or e is None for e in loss_weights):
                raise TypeError(f"For a model with multiple outputs, when providing the `loss_weights` argument as a list, each list entry should be a Python int, float (the weighting coefficient corresponding to the loss for that output). Received: loss_weights={loss_weights}")
            weights = list(loss_weights)
        elif isinstance(loss_weights, dict):
            names = [l.name if l.name is not None else (l.path[-1] if l.path else None) for l in self._flat_losses]
            for k in loss_weights:
                if k not in names:
                    raise ValueError(f"In the dict argument `loss_weights`, key '{k}' does not correspond to any model output. Received: loss_weights={loss_weights}")
                if not isinstance(loss_weights[k], (int, float)):
                    raise TypeError(f"For a model with multiple outputs, when providing the `loss_weights` argument as a dict, each dict entry should be a Python int, float (the weighting coefficient corresponding to the loss for that output). At entry '{k}', expected a int or float. Received: loss_weights={loss_weights}")
            weights = [loss_weights.get(nm) for nm in names]
        else:
            weights = [None] * n
        self._flat_losses = [CompileLoss.Loss_(l.path, l.loss, w, l.name) for l, w in zip(self._flat_losses, weights)]
        if len(self._flat_losses) > 1:
            for l in self._flat_losses:
                name = l.name
                if name is None and l.path:
                    name = "_".join(str(p) for p in l.path) if not isinstance(l.path[-1], str) else l.path[-1]
                    if not isinstance(l.path[-1], str):
                        name = None
                if name is not None:
                    self._tracked_metrics.append((l, metrics_module.Mean(name=f"{name}_loss")))
                    self._metrics.append(self._tracked_metrics[-1][1])
        self._y_pred_build_structure = tree.map_structure(lambda x: None, y_pred)
        self._y_true_build_structure = tree.map_structure(lambda x: None, y_true)
        self.built = True

    def __call__(self, y_true, y_pred, sample_weight=None):
        return self.call(y_true, y_pred, sample_weight)

    def call(self, y_true, y_pred, sample_weight=None):
        if not tree.is_nested(y_true) and not tree.is_nested(y_pred):
            if not self.built:
                self.build(y_true, y_pred)
            _, loss_fn, loss_weight, _ = self._flat_losses[0] if self._flat_losses else (None, None, None, None)
            if loss_fn is None:
                return None
            value = ops.cast(loss_fn(y_true, y_pred, sample_weight), dtype=self.dtype)
            if loss_weight is not None:
                value = ops.multiply(value, loss_weight)
            return value
        try:
            tree.assert_same_structure(y_pred, y_true, check_types=False)
        except ValueError:
            # align y_true to y_pred's structure
            flat_y_true = tree.flatten(y_true)
            try:
                y_true = tree.pack_sequence_as(y_pred, flat_y_true)
            except Exception:
                y_true_struct = tree.map_structure(lambda _: "*", y_true)
                y_pred_struct = tree.map_structure(lambda _: "*", y_pred)
                raise ValueError(
                    "y_true and y_pred have different structures.\n"
                    f"y_true: {y_true_struct}\ny_pred: {y_pred_struct}\n"
                )
        if not self.built:
            self.build(y_true, y_pred)
        try:
            tree.assert_same_structure(self._y_pred_build_structure, y_pred, check_types=False)
        except ValueError:
            y_pred = tree.pack_sequence_as(self._y_pred_build_structure, tree.flatten(y_pred))
        try:
            tree.assert_same_structure(self._y_true_build_structure, y_true, check_types=False)
        except ValueError:
            y_true = tree.pack_sequence_as(self._y_true_build_structure, tree.flatten(y_true))

        def resolve(struct, path):
            for p in path:
                struct = struct[p]
            return struct

        if sample_weight is not None and not tree.is_nested(sample_weight):
            sw_uniform = sample_weight
            sample_weight = None
        else:
            sw_uniform = None
        if sample_weight is not None:
            try:
                tree.assert_same_structure(sample_weight, y_pred, check_types=False)
            except ValueError:
                flat_sw = tree.flatten(sample_weight)
                if len(flat_sw) == len(tree.flatten(y_pred)):
                    sample_weight = tree.pack_sequence_as(y_pred, flat_sw)
                else:
                    sample_weight = None
                    sw_uniform = flat_sw[0] if flat_sw else None
        values = []
        track = {id(l): m for l, m in self._tracked_metrics}
        for entry in self._flat_losses:
            path, loss_fn, loss_weight, _ = entry
            yt = resolve(y_true, path)
            yp = resolve(y_pred, path)
            sw = resolve(sample_weight, path) if sample_weight is not None else sw_uniform
            if loss_fn is None:
                continue
            value = ops.cast(loss_fn(yt, yp, sw), dtype=self.dtype)
            m = track.get(id(entry))
            if m is not None:
                bs = tree.flatten(yp)[0].shape[0]
                m.update_state(value.detach() if isinstance(value, torch.Tensor) else value, sample_weight=bs)
            if loss_weight is not None:
                value = ops.multiply(value, loss_weight)
            values.append(value)
        if values:
            total = values[0]
            for v in values[1:]:
                total = total + v
            return total
        return None

    def get_config(self):
        raise NotImplementedError

    @classmethod
    def from_config(cls, config):
        raise NotImplementedError
