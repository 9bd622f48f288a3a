"""Callbacks (``keras.callbacks``; keras/src/callbacks/*.py)."""

import collections
import csv
import json
import os
import re
import shutil
import sys
import time
import warnings

import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils
from keras_b200.utils.progbar import Progbar


def _py(logs):
    from keras_b200.trainers.trainer import pythonify_logs

    return pythonify_logs(logs)


@keras_export("keras.callbacks.Callback")
class Callback:
    def __init__(self):
        self.params = None
        self._model = None

    def set_params(self, params):
        self.params = params

    def set_model(self, model):
        self._model = model

    @property
    def model(self):
        return self._model

    def on_batch_begin(self, batch, logs=None):
        pass

    def on_batch_end(self, batch, logs=None):
        pass

    def on_epoch_begin(self, epoch, logs=None):
        pass

    def on_epoch_end(self, epoch, logs=None):
        pass

    def on_train_batch_begin(self, batch, logs=None):
        self.on_batch_begin(batch, logs=logs)

    def on_train_batch_end(self, batch, logs=None):
        self.on_batch_end(batch, logs=logs)

    def on_test_batch_begin(self, batch, logs=None):
        pass

    def on_test_batch_end(self, batch, logs=None):
        pass

    def on_predict_batch_begin(self, batch, logs=None):
        pass

    def on_predict_batch_end(self, batch, logs=None):
        pass

    def on_train_begin(self, logs=None):
        pass

    def on_train_end(self, logs=None):
        pass

    def on_test_begin(self, logs=None):
        pass

    def on_test_end(self, logs=None):
        pass

    def on_predict_begin(self, logs=None):
        pass

    def on_predict_end(self, logs=None):
        pass


_BATCH_HOOKS = ("on_batch_begin", "on_batch_end", "on_train_batch_begin", "on_train_batch_end", "on_test_batch_begin",
                "on_test_batch_end", "on_predict_batch_begin", "on_predict_batch_end")


@keras_export("keras.callbacks.CallbackList")
class CallbackList(Callback):
    """Container that fans hooks out to callbacks.  Batch-level hooks are dispatched only to
    callbacks that override them, so an empty hook costs nothing in the step loop."""

    def __init__(self, callbacks=None, add_history=False, add_progbar=False, model=None, **params):
        self.callbacks = tree.flatten(callbacks) if callbacks else []
        self._in_begin_end_block_count = 0
        self._add_default_callbacks(add_history, add_progbar)
        self.set_model(model)
        self.set_params(params)
        self._overrides = {}
        for hook in _BATCH_HOOKS:
            self._overrides[hook] = [cb for cb in self.callbacks if _overrides(cb, hook)]

    def set_params(self, params):
        self.params = params
        if params:
            for cb in self.callbacks:
                cb.set_params(params)

    def _add_default_callbacks(self, add_history, add_progbar):
        self._progbar = None
        self._history = None
        for cb in self.callbacks:
            if isinstance(cb, ProgbarLogger):
                self._progbar = cb
            elif isinstance(cb, History):
                self._history = cb
        if self._history is None and add_history:
            self._history = History()
            self.callbacks.append(self._history)
        if self._progbar is None and add_progbar:
            self._progbar = ProgbarLogger()
            self.callbacks.append(self._progbar)

    def set_model(self, model):
        if not model:
            return
        Callback.set_model(self, model)
        if self._history:
            model.history = self._history
        for cb in self.callbacks:
            cb.set_model(model)

    def append(self, callback):
        self.callbacks.append(callback)
        for hook in _BATCH_HOOKS:
            if _overrides(callback, hook):
                self._overrides[hook].append(callback)

    def _batch(self, hook, batch, logs):
        for cb in self._overrides[hook]:
            getattr(cb, hook)(batch, logs=logs)

    def on_batch_begin(self, batch, logs=None):
        self._batch("on_batch_begin", batch, logs)

    def on_batch_end(self, batch, logs=None):
        self._batch("on_batch_end", batch, logs)

    def on_train_batch_begin(self, batch, logs=None):
        for cb in self._overrides["on_train_batch_begin"]:
            cb.on_train_batch_begin(batch, logs=logs)
        for cb in self._overrides["on_batch_begin"]:
            if cb not in self._overrides["on_train_batch_begin"]:
                cb.on_batch_begin(batch, logs=logs)

    def on_train_batch_end(self, batch, logs=None):
        for cb in self._overrides["on_train_batch_end"]:
            cb.on_train_batch_end(batch, logs=logs)
        for cb in self._overrides["on_batch_end"]:
            if cb not in self._overrides["on_train_batch_end"]:
                cb.on_batch_end(batch, logs=logs)

    def on_test_batch_begin(self, batch, logs=None):
        self._batch("on_test_batch_begin", batch, logs)

    def on_test_batch_end(self, batch, logs=None):
        self._batch("on_test_batch_end", batch, logs)

    def on_predict_batch_begin(self, batch, logs=None):
        self._batch("on_predict_batch_begin", batch, logs)

    def on_predict_batch_end(self, batch, logs=None):
        self._batch("on_predict_batch_end", batch, logs)

    def on_epoch_begin(self, epoch, logs=None):
        for cb in self.callbacks:
            cb.on_epoch_begin(epoch, logs)

    def on_epoch_end(self, epoch, logs=None):
        logs = _py(logs)
        for cb in self.callbacks:
            cb.on_epoch_end(epoch, logs)

    def on_train_begin(self, logs=None):
        for cb in self.callbacks:
            cb.on_train_begin(logs)

    def on_train_end(self, logs=None):
        logs = _py(logs)
        for cb in self.callbacks:
            cb.on_train_end(logs)

    def on_test_begin(self, logs=None):
        for cb in self.callbacks:
            cb.on_test_begin(logs)

    def on_test_end(self, logs=None):
        logs = _py(logs)
        for cb in self.callbacks:
            cb.on_test_end(logs)

    def on_predict_begin(self, logs=None):
        for cb in self.callbacks:
            cb.on_predict_begin(logs)

    def on_predict_end(self, logs=None):
        for cb in self.callbacks:
            cb.on_predict_end(logs)


def _overrides(cb, hook):
    fn = getattr(type(cb), hook, None)
    base = getattr(Callback, hook)
    if fn is None:
        return False
    if fn is not base:
        return True
    # the train-batch hooks forward to on_batch_*: count an override of those too
    if hook == "on_train_batch_begin":
        return getattr(type(cb), "on_batch_begin") is not Callback.on_batch_begin
    if hook == "on_train_batch_end":
        return getattr(type(cb), "on_batch_end") is not Callback.on_batch_end
    return False


@keras_export("keras.callbacks.History")
class History(Callback):
    def __init__(self):
        super().__init__()
        self.history = {}

    def on_train_begin(self, logs=None):
        self.epoch = []

    def on_epoch_end(self, epoch, logs=None):
        logs = logs or {}
        self.epoch.append(epoch)
        for k, v in logs.items():
            self.history.setdefault(k, []).append(v)
        self.model.history = self


@keras_export("keras.callbacks.ProgbarLogger")
class ProgbarLogger(Callback):
    """Prints metrics; reads device values at most every ``interval`` seconds, not every step."""

    def __init__(self):
        super().__init__()
        self.seen = 0
        self.progbar = None
        self.target = None
        self.verbose = 1
        self.epochs = 1
        self._called_in_fit = False
        self._last_print = 0.0

    def set_params(self, params):
        verbose = params["verbose"]
        if verbose == "auto":
            verbose = 1
        self.verbose = verbose
        self.epochs = params["epochs"]
        self.target = params["steps"]

    def on_train_begin(self, logs=None):
        self._called_in_fit = True

    def on_test_begin(self, logs=None):
        if not self._called_in_fit:
            self._reset_progbar()
            self._maybe_init_progbar()

    def on_predict_begin(self, logs=None):
        self._reset_progbar()
        self._maybe_init_progbar()

    def on_epoch_begin(self, epoch, logs=None):
        self._reset_progbar()
        self._maybe_init_progbar()
        if self.verbose and self.epochs > 1:
            io_utils.print_msg(f"Epoch {epoch + 1}/{self.epochs}")

    def on_train_batch_end(self, batch, logs=None):
        self._update_progbar(batch, logs)

    def on_test_batch_end(self, batch, logs=None):
        if not self._called_in_fit:
            self._update_progbar(batch, logs)

    def on_predict_batch_end(self, batch, logs=None):
        self._update_progbar(batch, None)

    def on_epoch_end(self, epoch, logs=None):
        self._finalize_progbar(logs)

    def on_test_end(self, logs=None):
        if not self._called_in_fit:
            self._finalize_progbar(logs)

    def on_predict_end(self, logs=None):
        self._finalize_progbar(logs)

    def _reset_progbar(self):
        self.seen = 0
        self.progbar = None

    def _maybe_init_progbar(self):
        if self.progbar is None:
            self.progbar = Progbar(target=self.target, verbose=self.verbose, unit_name="step")

    def _update_progbar(self, batch, logs=None):
        self._maybe_init_progbar()
        self.seen = batch + 1
        if self.verbose == 1:
            now = time.time()
            last = self.target is not None and self.seen >= self.target
            if now - self._last_print < 0.25 and not last:
                # skip: converting logs would synchronise with the device
                self.progbar._seen_so_far = self.seen
                return
            self._last_print = now
            logs = _py(logs or {})
            logs.pop("outputs", None)
            self.progbar.update(self.seen, list(logs.items()), finalize=False)

    def _finalize_progbar(self, logs):
        logs = _py(logs or {})
        if self.target is None:
            self.target = self.seen
            self.progbar.target = self.target
        self.progbar.update(self.target, list(logs.items()), finalize=True)


class MonitorCallback(Callback):
    """Base for callbacks that watch one metric (keras/src/callbacks/monitor_callback.py)."""

    def __init__(self, monitor="val_loss", mode="auto", baseline=None, min_delta=0):
        super().__init__()
        if mode not in ["auto", "min", "max"]:
            raise ValueError(f"{self.__class__.__name__} mode '{mode}' is unknown, fallback to auto mode.")
        self.monitor = monitor
        self.mode = mode
        self.best = baseline
        self.min_delta = abs(min_delta)
        self.monitor_op = None

    def _set_monitor_op(self):
        if self.mode == "min":
            self.monitor_op = np.less
        elif self.mode == "max":
            self.monitor_op = np.greater
        else:
            metric_name = self.monitor.removeprefix("val_")
            if metric_name == "loss":
                self.monitor_op = np.less
            if hasattr(self.model, "metrics"):
                all_metrics = []
                for m in self.model.metrics:
                    from keras_b200.trainers.compile_utils import CompileMetrics

                    if isinstance(m, CompileMetrics):
                        all_metrics.extend(m.metrics)
                    else:
                        all_metrics.append(m)
                for m in all_metrics:
                    if m.name == metric_name:
                        if hasattr(m, "_direction"):
                            self.monitor_op = np.greater if m._direction == "up" else np.less
        if self.monitor_op is None:
            if "acc" in self.monitor or "auc" in self.monitor or self.monitor.endswith("fmeasure"):
                self.monitor_op = np.greater
            else:
                raise ValueError(f"{self.__class__.__name__} callback received monitor={self.monitor}, but Keras isn't able to automatically determine whether that metric should be maximized or minimized. Pass `mode='max'` in order to monitor based on the highest metric value, or pass `mode='min'` in order to use the lowest value.")
        if self.monitor_op == np.less:
            self.min_delta *= -1

    def _is_improvement(self, monitor_value, reference_value):
        if reference_value is None:
            return True
        return self.monitor_op(monitor_value - self.min_delta, reference_value)


@keras_export("keras.callbacks.EarlyStopping")
class EarlyStopping(MonitorCallback):
    def __init__(self, monitor="val_loss", min_delta=0, patience=0, verbose=0, mode="auto", baseline=None, restore_best_weights=False, start_from_epoch=0):
        super().__init__(monitor, mode, min_delta=min_delta)
        self.patience = patience
        self.verbose = verbose
        self.baseline = baseline
        self.wait = 0
        self.stopped_epoch = 0
        self.restore_best_weights = restore_best_weights
        self.best_weights = None
        self.start_from_epoch = start_from_epoch

    def on_train_begin(self, logs=None):
        self.wait = 0
        self.stopped_epoch = 0
        self.best = None
        self.best_weights = None
        self.best_epoch = 0

    def on_epoch_end(self, epoch, logs=None):
        if self.monitor_op is None:
            self._set_monitor_op()
        current = self.get_monitor_value(logs)
        if current is None or epoch < self.start_from_epoch:
            return
        if self.restore_best_weights and self.best_weights is None:
            self.best_weights = self.model.get_weights()
            self.best_epoch = epoch
        self.wait += 1
        if self._is_improvement(current, self.best):
            self.best = current
            self.best_epoch = epoch
            if self.restore_best_weights:
                self.best_weights = self.model.get_weights()
            if self.baseline is None or self._is_improvement(current, self.baseline):
                self.wait = 0
            return
        if self.wait >= self.patience and epoch > 0:
            self.stopped_epoch = epoch
            self.model.stop_training = True

    def on_train_end(self, logs=None):
        if self.stopped_epoch > 0 and self.verbose > 0:
            io_utils.print_msg(f"Epoch {self.stopped_epoch + 1}: early stopping")
        if self.restore_best_weights and self.best_weights is not None:
            if self.verbose > 0:
                io_utils.print_msg(f"Restoring model weights from the end of the best epoch: {self.best_epoch + 1}.")
            self.model.set_weights(self.best_weights)

    def get_monitor_value(self, logs):
        logs = logs or {}
        monitor_value = logs.get(self.monitor)
        if monitor_value is None:
            warnings.warn(f"Early stopping conditioned on metric `{self.monitor}` which is not available. Available metrics are: {','.join(list(logs.keys()))}", stacklevel=2)
        return monitor_value


@keras_export("keras.callbacks.ModelCheckpoint")
class ModelCheckpoint(MonitorCallback):
    def __init__(self, filepath, monitor="val_loss", verbose=0, save_best_only=False, save_weights_only=False, mode="auto", save_freq="epoch", initial_value_threshold=None):
        super().__init__(monitor, mode, baseline=initial_value_threshold)
        self.verbose = verbose
        self.filepath = os.fspath(filepath)
        self.save_best_only = save_best_only
        self.save_weights_only = save_weights_only
        self.save_freq = save_freq
        self._batches_seen_since_last_saving = 0
        self._last_batch_seen = 0
        self._current_epoch = 0
        if self.save_freq != "epoch" and not isinstance(self.save_freq, int):
            raise ValueError(f"Unrecognized save_freq: {self.save_freq}. Expected save_freq are 'epoch' or integer values")
        if save_weights_only:
            if not self.filepath.endswith(".weights.h5"):
                raise ValueError(f"When using `save_weights_only=True` in `ModelCheckpoint`, the filepath provided must end in `.weights.h5` (Keras weights format). Received: filepath={self.filepath}")
        else:
            if not any(self.filepath.endswith(ext) for ext in (".keras", ".h5")):
                raise ValueError(f"The filepath provided must end in `.keras` (Keras model format). Received: filepath={self.filepath}")

    def on_train_batch_end(self, batch, logs=None):
        if self._should_save_on_batch(batch):
            self._save_model(epoch=self._current_epoch, batch=batch, logs=_py(logs))

    def on_epoch_begin(self, epoch, logs=None):
        self._current_epoch = epoch

    def on_epoch_end(self, epoch, logs=None):
        if self.monitor_op is None:
            try:
                self._set_monitor_op()
            except ValueError:
                if self.save_best_only:
                    raise
        if self.save_freq == "epoch":
            self._save_model(epoch=epoch, batch=None, logs=logs)

    def _should_save_on_batch(self, batch):
        if self.save_freq == "epoch":
            return False
        if batch <= self._last_batch_seen:
            add_batches = batch + 1
        else:
            add_batches = batch - self._last_batch_seen
        self._batches_seen_since_last_saving += add_batches
        self._last_batch_seen = batch
        if self._batches_seen_since_last_saving >= self.save_freq:
            self._batches_seen_since_last_saving = 0
            return True
        return False

    def _should_save_model(self, epoch, batch, logs, filepath):
        logs = logs or {}
        if self.save_best_only:
            current = logs.get(self.monitor)
            if current is None:
                warnings.warn(f"Can save best model only with {self.monitor} available.", stacklevel=2)
                return True
            if self.monitor_op is None:
                self._set_monitor_op()
            if self._is_improvement(current, self.best):
                if self.verbose > 0:
                    io_utils.print_msg(f"\nEpoch {epoch + 1}: {self.monitor} improved from {self.best} to {current:.5f}, saving model to {filepath}")
                self.best = current
                return True
            if self.verbose > 0:
                io_utils.print_msg(f"\nEpoch {epoch + 1}: {self.monitor} did not improve from {self.best}")
            return False
        if self.verbose > 0:
            io_utils.print_msg(f"\nEpoch {epoch + 1}: saving model to {filepath}")
        return True

    def _save_model(self, epoch, batch, logs):
        filepath = self._get_file_path(epoch, batch, logs)
        try:
            if self._should_save_model(epoch, batch, logs, filepath):
                dirname = os.path.dirname(filepath)
                if dirname and not os.path.exists(dirname):
                    os.makedirs(dirname, exist_ok=True)
                if _is_chief():
                    if self.save_weights_only:
                        self.model.save_weights(filepath, overwrite=True)
                    else:
                        self.model.save(filepath, overwrite=True)
        except IsADirectoryError:
            raise IOError(f"Please specify a non-directory filepath for ModelCheckpoint. Filepath used is an existing directory: {filepath}")
        except IOError as e:
            if "is a directory" in str(e.args[0]).lower():
                raise IOError(f"Please specify a non-directory filepath for ModelCheckpoint. Filepath used is an existing directory: f{filepath}")
            raise e

    def _get_file_path(self, epoch, batch, logs):
        try:
            if batch is None or "batch" in (logs or {}):
                return self.filepath.format(epoch=epoch + 1, **(logs or {}))
            return self.filepath.format(epoch=epoch + 1, batch=batch + 1, **(logs or {}))
        except KeyError as e:
            raise KeyError(f'Failed to format this callback filepath: "{self.filepath}". Reason: {e}')

    def _checkpoint_exists(self, filepath):
        return os.path.exists(filepath)


def _is_chief():
    """True on the process that writes checkpoints (rank 0 of the job)."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank() == 0
    except Exception:
        pass
    return True


@keras_export("keras.callbacks.BackupAndRestore")
class BackupAndRestore(Callback):
    def __init__(self, backup_dir, save_freq="epoch", double_checkpoint=False, delete_checkpoint=True):
        super().__init__()
        self.save_freq = save_freq
        self.double_checkpoint = double_checkpoint
        self.delete_checkpoint = delete_checkpoint
        self._batches_seen_since_last_saving = 0
        self._last_batch_seen = 0
        self._current_epoch = 0
        if not backup_dir:
            raise ValueError("Empty `backup_dir` argument passed")
        self.backup_dir = backup_dir
        self._weights_path = os.path.join(backup_dir, "latest.weights.h5")
        self._training_metadata_path = os.path.join(backup_dir, "training_metadata.json")
        self._prev_weights_path = self._weights_path + ".bkp"
        self._prev_training_metadata_path = self._training_metadata_path + ".bkp"
        if save_freq != "epoch" and not isinstance(save_freq, int):
            raise ValueError(f"Invalid value for argument `save_freq`. Received: save_freq={save_freq}. Expected either 'epoch' or an integer value.")

    def on_train_begin(self, logs=None):
        try:
            self._load_model()
        except OSError as e:
            if os.path.exists(self._prev_weights_path):
                if os.path.exists(self._weights_path):
                    os.remove(self._weights_path)
                os.rename(self._prev_weights_path, self._weights_path)
                if os.path.exists(self._prev_training_metadata_path):
                    os.rename(self._prev_training_metadata_path, self._training_metadata_path)
                self._load_model()
            else:
                raise e

    def _load_model(self):
        if not self.model.built:
            raise ValueError("To use the BackupAndRestore callback, you model must be built before you call `fit()`. " f"Model {self.model} is unbuilt. You can build it beforehand by calling it on a batch of data.")
        if os.path.exists(self._weights_path):
            if self.model.optimizer is not None and not self.model.optimizer.built:
                with torch.no_grad():
                    self.model.optimizer.build(self.model.trainable_variables)
            self.model.load_weights(self._weights_path)
        if os.path.exists(self._training_metadata_path):
            with open(self._training_metadata_path, "r") as f:
                training_metadata = json.loads(f.read())
            self.model._initial_epoch = training_metadata["epoch"]

    def on_epoch_end(self, epoch, logs=None):
        self._current_epoch = epoch + 1
        self._last_batch_seen = 0
        if self.save_freq == "epoch":
            self._save_model()

    def on_train_batch_end(self, batch, logs=None):
        if self._should_save_on_batch(batch):
            self._save_model()

    def _save_model(self):
        if not _is_chief():
            return
        if not os.path.exists(self.backup_dir):
            os.makedirs(self.backup_dir, exist_ok=True)
        if self.double_checkpoint and os.path.exists(self._weights_path):
            shutil.copyfile(self._weights_path, self._prev_weights_path)
        if self.double_checkpoint and os.path.exists(self._training_metadata_path):
            shutil.copyfile(self._training_metadata_path, self._prev_training_metadata_path)
        self.model.save_weights(filepath=self._weights_path, overwrite=True)
        with open(self._training_metadata_path, "w") as f:
            f.write(json.dumps({"epoch": self._current_epoch, "batch": self._last_batch_seen}))

    def _should_save_on_batch(self, batch):
        if self.save_freq == "epoch":
            return False
        if batch <= self._last_batch_seen:
            add_batches = batch + 1
        else:
            add_batches = batch - self._last_batch_seen
        self._batches_seen_since_last_saving += add_batches
        self._last_batch_seen = batch
        if self._batches_seen_since_last_saving >= self.save_freq:
            self._batches_seen_since_last_saving = 0
            return True
        return False

    def on_train_end(self, logs=None):
        if self.delete_checkpoint and os.path.exists(self.backup_dir) and _is_chief():
            shutil.rmtree(self.backup_dir)


@keras_export("keras.callbacks.TerminateOnNaN")
class TerminateOnNaN(Callback):
    def __init__(self, raise_error=False):
        super().__init__()
        self.raise_error = raise_error

    def on_batch_end(self, batch, logs=None):
        logs = logs or {}
        loss = logs.get("loss")
        if loss is not None:
            if np.isnan(loss) or np.isinf(loss):
                if self.raise_error:
                    raise RuntimeError(f"NaN or Inf loss encountered at batch {batch}. Loss value: {loss}. Training terminated.")
                io_utils.print_msg(f"Batch {batch}: Invalid loss, terminating training")
                self.model.stop_training = True


@keras_export("keras.callbacks.LearningRateScheduler")
class LearningRateScheduler(Callback):
    def __init__(self, schedule, verbose=0):
        super().__init__()
        self.schedule = schedule
        self.verbose = verbose

    def on_epoch_begin(self, epoch, logs=None):
        if not hasattr(self.model.optimizer, "learning_rate"):
            raise ValueError('Optimizer must have a "learning_rate" attribute.')
        try:
            learning_rate = float(np.asarray(_numpy(self.model.optimizer.learning_rate)))
            learning_rate = self.schedule(epoch, learning_rate)
        except TypeError:
            learning_rate = self.schedule(epoch)
        if not isinstance(learning_rate, (float, np.float32, np.float64)):
            raise ValueError(f"The output of the `schedule` function should be a float. Got: {learning_rate}")
        self.model.optimizer.learning_rate = float(learning_rate)
        if self.verbose > 0:
            io_utils.print_msg(f"\nEpoch {epoch + 1}: LearningRateScheduler setting learning rate to {learning_rate}.")

    def on_epoch_end(self, epoch, logs=None):
        if logs is not None:
            logs["learning_rate"] = float(np.asarray(_numpy(self.model.optimizer.learning_rate)))


def _numpy(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    return x


@keras_export("keras.callbacks.ReduceLROnPlateau")
class ReduceLROnPlateau(MonitorCallback):
    def __init__(self, monitor="val_loss", factor=0.1, patience=10, verbose=0, mode="auto", min_delta=1e-4, cooldown=0, min_lr=0.0, **kwargs):
        super().__init__(monitor, mode, min_delta=min_delta)
        if factor >= 1.0:
            raise ValueError(f"ReduceLROnPlateau does not support a factor >= 1.0. Received factor={factor}")
        self.factor = factor
        self.min_lr = min_lr
        self.patience = patience
        self.verbose = verbose
        self.cooldown = cooldown
        self.cooldown_counter = 0
        self.wait = 0

    def _reset(self):
        self.cooldown_counter = 0
        self.wait = 0

    def on_train_begin(self, logs=None):
        self._reset()

    def on_epoch_end(self, epoch, logs=None):
        if self.monitor_op is None:
            self._set_monitor_op()
        logs = logs if logs is not None else {}
        logs["learning_rate"] = float(np.asarray(_numpy(self.model.optimizer.learning_rate)))
        current = logs.get(self.monitor)
        if current is None:
            warnings.warn(f"Learning rate reduction is conditioned on metric `{self.monitor}` which is not available. Available metrics are: {','.join(list(logs.keys()))}.", stacklevel=2)
        else:
            if self.in_cooldown():
                self.cooldown_counter -= 1
                self.wait = 0
            if self._is_improvement(current, self.best):
                self.best = current
                self.wait = 0
            elif not self.in_cooldown():
                self.wait += 1
                if self.wait >= self.patience:
                    old_lr = float(np.asarray(_numpy(self.model.optimizer.learning_rate)))
                    if old_lr > np.float32(self.min_lr):
                        new_lr = max(old_lr * self.factor, self.min_lr)
                        self.model.optimizer.learning_rate = new_lr
                        if self.verbose > 0:
                            io_utils.print_msg(f"\nEpoch {epoch + 1}: ReduceLROnPlateau reducing learning rate to {new_lr}.")
                        self.cooldown_counter = self.cooldown
                        self.wait = 0

    def in_cooldown(self):
        return self.cooldown_counter > 0


@keras_export("keras.callbacks.CSVLogger")
class CSVLogger(Callback):
    def __init__(self, filename, separator=",", append=False):
        super().__init__()
        self.sep = separator
        self.filename = os.fspath(filename)
        self.append = append
        self.writer = None
        self.keys = None
        self.append_header = True
        self.csv_file = None

    def on_train_begin(self, logs=None):
        if self.append:
            if os.path.exists(self.filename):
                with open(self.filename, "r") as f:
                    self.append_header = not bool(len(f.readline()))
            mode = "a"
        else:
            mode = "w"
        if self.csv_file and not self.csv_file.closed:
            self.csv_file.close()
        self.csv_file = open(self.filename, mode)
        self.writer = None
        self.keys = None

    def on_epoch_end(self, epoch, logs=None):
        logs = logs or {}

        def handle_value(k):
            is_zero_dim_ndarray = isinstance(k, np.ndarray) and k.ndim == 0
            if isinstance(k, str):
                return k
            if isinstance(k, collections.abc.Iterable) and not is_zero_dim_ndarray:
                return f"\"[{', '.join(map(str, k))}]\""
            return k

        if self.keys is None:
            self.keys = sorted(logs.keys())
            val_keys_found = False
            for key in self.keys:
                if key.startswith("val_"):
                    val_keys_found = True
                    break
            if not val_keys_found and self.keys:
                self.keys.extend(["val_" + k for k in self.keys])
        if not self.writer:
            class CustomDialect(csv.excel):
                delimiter = self.sep

            fieldnames = ["epoch"] + (self.keys or [])
            self.writer = csv.DictWriter(self.csv_file, fieldnames=fieldnames, dialect=CustomDialect)
            if self.append_header:
                self.writer.writeheader()
        row_dict = collections.OrderedDict({"epoch": epoch})
        row_dict.update((key, handle_value(logs.get(key, "NA"))) for key in self.keys)
        self.writer.writerow(row_dict)
        self.csv_file.flush()

    def on_train_end(self, logs=None):
        if self.csv_file and not self.csv_file.closed:
            self.csv_file.close()
        self.writer = None


@keras_export("keras.callbacks.LambdaCallback")
class LambdaCallback(Callback):
    def __init__(self, on_epoch_begin=None, on_epoch_end=None, on_train_begin=None, on_train_end=None, on_train_batch_begin=None, on_train_batch_end=None, **kwargs):
        super().__init__()
        self.__dict__.update(kwargs)
        if on_epoch_begin is not None:
            self.on_epoch_begin = on_epoch_begin
        if on_epoch_end is not None:
            self.on_epoch_end = on_epoch_end
        if on_train_begin is not None:
            self.on_train_begin = on_train_begin
        if on_train_end is not None:
            self.on_train_end = on_train_end
        self._tb_begin = on_train_batch_begin
        self._tb_end = on_train_batch_end

    def on_train_batch_begin(self, batch, logs=None):
        if self._tb_begin is not None:
            self._tb_begin(batch, logs)

    def on_train_batch_end(self, batch, logs=None):
        if self._tb_end is not None:
            self._tb_end(batch, _py(logs))


@keras_export("keras.callbacks.RemoteMonitor")
class RemoteMonitor(Callback):
    def __init__(self, root="http://localhost:9000", path="/publish/epoch/end/", field="data", headers=None, send_as_json=False):
        super().__init__()
        self.root, self.path, self.field, self.headers, self.send_as_json = root, path, field, headers, send_as_json

    def on_epoch_end(self, epoch, logs=None):
        try:
            import requests
        except ImportError:
            raise ImportError("RemoteMonitor requires the `requests` library.")
        logs = logs or {}
        send = {"epoch": epoch}
        for k, v in logs.items():
            send[k] = v.item() if isinstance(v, (np.ndarray, np.generic)) else v
        try:
            if self.send_as_json:
                requests.post(self.root + self.path, json=send, headers=self.headers)
            else:
                requests.post(self.root + self.path, {self.field: json.dumps(send)}, headers=self.headers)
        except requests.exceptions.RequestException:
            warnings.warn(f"Could not reach RemoteMonitor root server at {self.root}", stacklevel=2)


@keras_export("keras.callbacks.SwapEMAWeights")
class SwapEMAWeights(Callback):
    def __init__(self, swap_on_epoch=False):
        super().__init__()
        self.swap_on_epoch = swap_on_epoch
        self._ema_weights_in_model = False

    def _swap_variables(self):
        opt = self.model.optimizer
        if hasattr(opt, "inner_optimizer"):
            opt = opt.inner_optimizer
        if not hasattr(opt, "_model_variables_moving_average"):
            raise ValueError(f"SwapEMAWeights must be used when `use_ema=True` is set on the optimizer. Received: use_ema={opt.use_ema}")
        if not opt.use_ema:
            raise ValueError(f"SwapEMAWeights must be used when `use_ema=True` is set on the optimizer. Received: use_ema={opt.use_ema}")
        with torch.no_grad():
            for var, average in zip(self.model.trainable_variables, opt._model_variables_moving_average):
                if average is None:
                    continue
                tmp = var._value.detach().clone()
                var._value.copy_(average._value)
                average._value.copy_(tmp)

    def _finalize_ema_values(self):
        opt = self.model.optimizer
        if hasattr(opt, "inner_optimizer"):
            opt = opt.inner_optimizer
        with torch.no_grad():
            for var, average in zip(self.model.trainable_variables, opt._model_variables_moving_average):
                if average is not None:
                    average._value.copy_(var._value)

    def on_epoch_begin(self, epoch, logs=None):
        if self.swap_on_epoch and self._ema_weights_in_model:
            self._swap_variables()
            self._ema_weights_in_model = False

    def on_epoch_end(self, epoch, logs=None):
        if self.swap_on_epoch and not self._ema_weights_in_model:
            self._swap_variables()
            self._ema_weights_in_model = True
            if epoch == self.params["epochs"] - 1:
                self._finalize_ema_values()

    def on_test_begin(self, logs=None):
        if not self._ema_weights_in_model:
            self._swap_variables()
            self._ema_weights_in_model = True

    def on_test_end(self, logs=None):
        if self._ema_weights_in_model:
            self._swap_variables()
            self._ema_weights_in_model = False

    def on_predict_begin(self, logs=None):
        if not self._ema_weights_in_model:
            self._swap_variables()
            self._ema_weights_in_model = True

    def on_predict_end(self, logs=None):
        if not self._ema_weights_in_model:
            self._swap_variables()
            self._ema_weights_in_model = False
