"""Callbacks that steer the run: ``EarlyStopping``, ``ReduceLROnPlateau``, ``LearningRateScheduler``, ``TerminateOnNaN``
(keras/src/callbacks/early_stopping.py, reduce_lr_on_plateau.py, learning_rate_scheduler.py, terminate_on_nan.py)."""

import math
import warnings

import numpy as np

from keras_b200.callbacks.base import Callback
from keras_b200.callbacks.watch import MonitorCallback, learning_rate_of
from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils


@keras_export("keras.callbacks.EarlyStopping")
class EarlyStopping(MonitorCallback):
    """Stops ``fit`` when the watched metric has not improved for ``patience`` epochs."""

    def __init__(self, monitor="val_loss", min_delta=0, patience=0, verbose=0, mode="auto", baseline=None, restore_best_weights=False,
                 start_from_epoch=0):
        super().__init__(monitor, mode, min_delta=min_delta)
        self.patience, self.verbose, self.baseline = patience, verbose, baseline
        self.restore_best_weights, self.start_from_epoch = restore_best_weights, start_from_epoch
        self._clear()

    def _clear(self):
        self.wait = 0            # epochs since the last improvement that also beat the baseline
        self.stopped_epoch = 0
        self.best = None
        self.best_weights = None
        self.best_epoch = 0

    def on_train_begin(self, logs=None):
        self._clear()

    def get_monitor_value(self, logs):
        logs = logs or {}
        value = logs.get(self.monitor)
        if value is None:
            warnings.warn(f"Early stopping conditioned on metric `{self.monitor}` which is not available. "
                          f"Available metrics are: {','.join(list(logs.keys()))}", stacklevel=2)
        return value

    def _snapshot(self, epoch):
        self.best_weights = self.model.get_weights()
        self.best_epoch = epoch

    def on_epoch_end(self, epoch, logs=None):
        self._ensure_direction()
        value = self.get_monitor_value(logs)
        if value is None or epoch < self.start_from_epoch:
            return
        if self.restore_best_weights and self.best_weights is None:
            self._snapshot(epoch)  # something to fall back to even if no epoch ever improves
        if self._is_improvement(value, self.best):
            self.best = value
            self.best_epoch = epoch
            if self.restore_best_weights:
                self._snapshot(epoch)
            # progress that still trails the baseline keeps the patience clock running
            beats_baseline = self.baseline is None or self._is_improvement(value, self.baseline)
            self.wait = 0 if beats_baseline else self.wait + 1
            return
        self.wait += 1
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


@keras_export("keras.callbacks.ReduceLROnPlateau")
class ReduceLROnPlateau(MonitorCallback):
    """Multiplies the learning rate by ``factor`` when the watched metric stalls for ``patience`` epochs, then holds off for
    ``cooldown`` epochs."""

    def __init__(self, monitor="val_loss", factor=0.1, patience=10, verbose=0, mode="auto", min_delta=1e-4, cooldown=0, min_lr=0.0, **kwargs):
        super().__init__(monitor, mode, min_delta=min_delta)
        if factor >= 1.0:
            raise ValueError(f"ReduceLROnPlateau does not support a factor >= 1.0. Received factor={factor}")
        self.factor, self.min_lr, self.patience, self.verbose, self.cooldown = factor, min_lr, patience, verbose, cooldown
        self._reset()

    def _reset(self):
        self.cooldown_counter = 0
        self.wait = 0

    def in_cooldown(self):
        return self.cooldown_counter > 0

    def on_train_begin(self, logs=None):
        self._reset()

    def on_epoch_end(self, epoch, logs=None):
        self._ensure_direction()
        logs = logs if logs is not None else {}
        optimizer = self.model.optimizer
        logs["learning_rate"] = learning_rate_of(optimizer)
        value = logs.get(self.monitor)
        if value is None:
            warnings.warn(f"Learning rate reduction is conditioned on metric `{self.monitor}` which is not available. "
                          f"Available metrics are: {','.join(list(logs.keys()))}.", stacklevel=2)
            return
        cooling = self.in_cooldown()
        if cooling:
            self.cooldown_counter -= 1
            self.wait = 0
        if self._is_improvement(value, self.best):
            self.best = value
            self.wait = 0
            return
        if self.in_cooldown():
            return
        self.wait += 1
        if self.wait < self.patience:
            return
        current = learning_rate_of(optimizer)
        if current > np.float32(self.min_lr):
            reduced = max(current * self.factor, self.min_lr)
            optimizer.learning_rate = reduced
            if self.verbose > 0:
                io_utils.print_msg(f"\nEpoch {epoch + 1}: ReduceLROnPlateau reducing learning rate to {reduced}.")
            self.cooldown_counter = self.cooldown
            self.wait = 0


@keras_export("keras.callbacks.LearningRateScheduler")
class LearningRateScheduler(Callback):
    """Sets the learning rate at the start of every epoch from ``schedule(epoch, lr)`` (or ``schedule(epoch)``)."""

    def __init__(self, schedule, verbose=0):
        super().__init__()
        self.schedule, self.verbose = schedule, verbose

    def on_epoch_begin(self, epoch, logs=None):
        optimizer = self.model.optimizer
        if not hasattr(optimizer, "learning_rate"):
            raise ValueError('Optimizer must have a "learning_rate" attribute.')
        try:
            rate = self.schedule(epoch, learning_rate_of(optimizer))
        except TypeError:  # a schedule that only takes the epoch index
            rate = self.schedule(epoch)
        if not isinstance(rate, (float, np.float32, np.float64)):
            raise ValueError(f"The output of the `schedule` function should be a float. Got: {rate}")
        optimizer.learning_rate = float(rate)
        if self.verbose > 0:
            io_utils.print_msg(f"\nEpoch {epoch + 1}: LearningRateScheduler setting learning rate to {rate}.")

    def on_epoch_end(self, epoch, logs=None):
        if logs is not None:
            logs["learning_rate"] = learning_rate_of(self.model.optimizer)


@keras_export("keras.callbacks.TerminateOnNaN")
class TerminateOnNaN(Callback):
    """Ends training (or raises, with ``raise_error``) as soon as a batch reports a loss that is not finite."""

    def __init__(self, raise_error=False):
        super().__init__()
        self.raise_error = raise_error

    def on_batch_end(self, batch, logs=None):
        loss = (logs or {}).get("loss")
        if loss is None:
            return
        value = float(loss)
        if math.isfinite(value):
            return
        if self.raise_error:
            raise RuntimeError(f"NaN or Inf loss encountered at batch {batch}. Loss value: {loss}. Training terminated.")
        io_utils.print_msg(f"Batch {batch}: Invalid loss, terminating training")
        self.model.stop_training = True
