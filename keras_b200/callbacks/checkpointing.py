"""Callbacks that write or swap model state: ``ModelCheckpoint``, ``BackupAndRestore``, ``SwapEMAWeights``
(keras/src/callbacks/model_checkpoint.py, backup_and_restore.py, swap_ema_weights.py).

Under a multi-process distribution only the chief process (rank 0) touches the file system; every process still takes
part in whatever collective the save needs (gathering sharded variables)."""

import json
import os
import shutil
import warnings

import torch

from keras_b200.callbacks.base import Callback, to_python
from keras_b200.callbacks.watch import BatchCadence, MonitorCallback, is_chief
from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils


@keras_export("keras.callbacks.ModelCheckpoint")
class ModelCheckpoint(MonitorCallback):
    """Saves the model (or its weights) every epoch or every ``save_freq`` batches, optionally only when the watched metric
    improved.  ``filepath`` may contain ``{epoch}``, ``{batch}`` and log keys as format fields."""

    def __init__(self, filepath, monitor="val_loss", verbose=0, save_best_only=False, save_weights_only=False, mode="auto", save_freq="epoch",
                 initial_value_threshold=None):
        super().__init__(monitor, mode, baseline=initial_value_threshold)
        self.verbose = verbose
        self.filepath = os.fspath(filepath)
        self.save_best_only, self.save_weights_only, self.save_freq = save_best_only, save_weights_only, save_freq
        if save_freq != "epoch" and not isinstance(save_freq, int):
            raise ValueError(f"Unrecognized save_freq: {self.save_freq}. Expected save_freq are 'epoch' or integer values")
        self._cadence = BatchCadence(save_freq)
        self._current_epoch = 0
        if save_weights_only:
            if not self.filepath.endswith(".weights.h5"):
                raise ValueError("When using `save_weights_only=True` in `ModelCheckpoint`, the filepath provided must end in `.weights.h5` "
                                 f"(Keras weights format). Received: filepath={self.filepath}")
        elif not self.filepath.endswith((".keras", ".h5")):
            raise ValueError(f"The filepath provided must end in `.keras` (Keras model format). Received: filepath={self.filepath}")

    # -- hooks ---------------------------------------------------------------------------
    def on_epoch_begin(self, epoch, logs=None):
        self._current_epoch = epoch

    def on_train_batch_end(self, batch, logs=None):
        if self._cadence.tick(batch):
            self._save_model(epoch=self._current_epoch, batch=batch, logs=to_python(logs))

    def on_epoch_end(self, epoch, logs=None):
        if not self._watch.resolved:
            try:
                self._set_monitor_op()
            except ValueError:
                if self.save_best_only:
                    raise  # without a direction "best" means nothing
        if self.save_freq == "epoch":
            self._save_model(epoch=epoch, batch=None, logs=logs)

    # -- decisions -----------------------------------------------------------------------
    def _get_file_path(self, epoch, batch, logs):
        fields = dict(logs or {})
        fields["epoch"] = epoch + 1
        if batch is not None and "batch" not in fields:
            fields["batch"] = batch + 1
        try:
            return self.filepath.format(**fields)
        except KeyError as e:
            raise KeyError(f'Failed to format this callback filepath: "{self.filepath}". Reason: {e}')

    def _should_save_model(self, epoch, batch, logs, filepath):
        if not self.save_best_only:
            if self.verbose > 0:
                io_utils.print_msg(f"\nEpoch {epoch + 1}: saving model to {filepath}")
            return True
        value = (logs or {}).get(self.monitor)
        if value is None:
            warnings.warn(f"Can save best model only with {self.monitor} available.", stacklevel=2)
            return True
        self._ensure_direction()
        if not self._is_improvement(value, self.best):
            if self.verbose > 0:
                io_utils.print_msg(f"\nEpoch {epoch + 1}: {self.monitor} did not improve from {self.best}")
            return False
        if self.verbose > 0:
            io_utils.print_msg(f"\nEpoch {epoch + 1}: {self.monitor} improved from {self.best} to {value:.5f}, saving model to {filepath}")
        self.best = value
        return True

    def _save_model(self, epoch, batch, logs):
        filepath = self._get_file_path(epoch, batch, logs)
        if not self._should_save_model(epoch, batch, logs, filepath):
            return
        if os.path.isdir(filepath):
            raise IOError(f"Please specify a non-directory filepath for ModelCheckpoint. Filepath used is an existing directory: {filepath}")
        folder = os.path.dirname(filepath)
        if folder:
            os.makedirs(folder, exist_ok=True)
        if not is_chief():
            return
        if self.save_weights_only:
            self.model.save_weights(filepath, overwrite=True)
        else:
            self.model.save(filepath, overwrite=True)

    def _checkpoint_exists(self, filepath):
        return os.path.exists(filepath)


@keras_export("keras.callbacks.BackupAndRestore")
class BackupAndRestore(Callback):
    """Keeps ``latest.weights.h5`` and ``training_metadata.json`` in ``backup_dir`` so that an interrupted ``fit`` picks up at
    the epoch it had reached.  With ``double_checkpoint`` the previous pair is kept as ``*.bkp`` and used when the latest
    one cannot be read."""

    def __init__(self, backup_dir, save_freq="epoch", double_checkpoint=False, delete_checkpoint=True):
        super().__init__()
        if not backup_dir:
            raise ValueError("Empty `backup_dir` argument passed")
        BatchCadence.validate(save_freq, "Invalid value for argument `save_freq`")
        self.backup_dir, self.save_freq = backup_dir, save_freq
        self.double_checkpoint, self.delete_checkpoint = double_checkpoint, delete_checkpoint
        self._cadence = BatchCadence(save_freq)
        self._current_epoch = 0
        self._weights_path = os.path.join(backup_dir, "latest.weights.h5")
        self._training_metadata_path = os.path.join(backup_dir, "training_metadata.json")
        self._prev_weights_path = self._weights_path + ".bkp"
        self._prev_training_metadata_path = self._training_metadata_path + ".bkp"

    def _pairs(self):
        return ((self._weights_path, self._prev_weights_path), (self._training_metadata_path, self._prev_training_metadata_path))

    def _load_model(self):
        model = self.model
        if not model.built:
            raise ValueError("To use the BackupAndRestore callback, you model must be built before you call `fit()`. "
                             f"Model {model} is unbuilt. You can build it beforehand by calling it on a batch of data.")
        if os.path.exists(self._weights_path):
            optimizer = model.optimizer
            if optimizer is not None and not optimizer.built:
                with torch.no_grad():
                    optimizer.build(model.trainable_variables)
            model.load_weights(self._weights_path)
        if os.path.exists(self._training_metadata_path):
            with open(self._training_metadata_path) as f:
                model._initial_epoch = json.load(f)["epoch"]

    def on_train_begin(self, logs=None):
        try:
            self._load_model()
        except OSError:
            if not os.path.exists(self._prev_weights_path):
                raise
            # the latest file is damaged (a crash while writing): step back to the previous pair
            for current, previous in self._pairs():
                if os.path.exists(previous):
                    if os.path.exists(current):
                        os.remove(current)
                    os.rename(previous, current)
            self._load_model()

    def _save_model(self):
        if not is_chief():
            return
        os.makedirs(self.backup_dir, exist_ok=True)
        if self.double_checkpoint:
            for current, previous in self._pairs():
                if os.path.exists(current):
                    shutil.copyfile(current, previous)
        self.model.save_weights(filepath=self._weights_path, overwrite=True)
        with open(self._training_metadata_path, "w") as f:
            json.dump({"epoch": self._current_epoch, "batch": self._cadence.last_index}, f)

    def on_epoch_end(self, epoch, logs=None):
        self._current_epoch = epoch + 1
        self._cadence.new_epoch()
        if self.save_freq == "epoch":
            self._save_model()

    def on_train_batch_end(self, batch, logs=None):
        if self._cadence.tick(batch):
            self._save_model()

    def on_train_end(self, logs=None):
        if self.delete_checkpoint and is_chief() and os.path.exists(self.backup_dir):
            shutil.rmtree(self.backup_dir)


@keras_export("keras.callbacks.SwapEMAWeights")
class SwapEMAWeights(Callback):
    """Puts the optimizer's exponential moving averages into the model for evaluation / prediction (and at epoch ends with
    ``swap_on_epoch``) and the raw weights back afterwards.  Needs an optimizer built with ``use_ema=True``."""

    def __init__(self, swap_on_epoch=False):
        super().__init__()
        self.swap_on_epoch = swap_on_epoch
        self._ema_weights_in_model = False

    def _ema_pairs(self):
        optimizer = self.model.optimizer
        optimizer = getattr(optimizer, "inner_optimizer", optimizer)
        if not getattr(optimizer, "use_ema", False) or not hasattr(optimizer, "_model_variables_moving_average"):
            raise ValueError("SwapEMAWeights must be used when `use_ema=True` is set on the optimizer. "
                             f"Received: use_ema={getattr(optimizer, 'use_ema', None)}")
        return [(v, a) for v, a in zip(self.model.trainable_variables, optimizer._model_variables_moving_average) if a is not None]

    def _swap_variables(self):
        with torch.no_grad():
            for variable, average in self._ema_pairs():
                raw = variable._value.detach().clone()
                variable.assign(average._value)
                average.assign(raw)

    def _finalize_ema_values(self):
        with torch.no_grad():
            for variable, average in self._ema_pairs():
                average.assign(variable._value)

    def _put(self, ema_in_model):
        if self._ema_weights_in_model != ema_in_model:
            self._swap_variables()
            self._ema_weights_in_model = ema_in_model

    def on_epoch_begin(self, epoch, logs=None):
        if self.swap_on_epoch:
            self._put(False)

    def on_epoch_end(self, epoch, logs=None):
        if self.swap_on_epoch and not self._ema_weights_in_model:
            self._put(True)
            if epoch == self.params["epochs"] - 1:
                self._finalize_ema_values()  # the run ends with the averages in the model: keep the optimizer's copy in line

    def on_test_begin(self, logs=None):
        self._put(True)

    def on_test_end(self, logs=None):
        self._put(False)

    def on_predict_begin(self, logs=None):
        self._put(True)

    def on_predict_end(self, logs=None):
        self._put(False)
