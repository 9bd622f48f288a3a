"""Callbacks that record or report: ``History``, ``ProgbarLogger``, ``CSVLogger``, ``RemoteMonitor``, ``LambdaCallback``
(keras/src/callbacks/history.py, progbar_logger.py, csv_logger.py, remote_monitor.py, lambda_callback.py)."""

import csv
import json
import os
import time
import warnings

import numpy as np

from keras_b200.callbacks.base import Callback, to_python
from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils
from keras_b200.utils.progbar import Progbar


@keras_export("keras.callbacks.History")
class History(Callback):
    """``history[name]`` is the list of per-epoch values of every logged quantity; ``epoch`` the epoch indices."""

    def __init__(self):
        super().__init__()
        self.history = {}

    def on_train_begin(self, logs=None):
        self.epoch = []

    def on_epoch_end(self, epoch, logs=None):
        self.epoch.append(epoch)
        for name, value in (logs or {}).items():
            self.history.setdefault(name, []).append(value)
        self.model.history = self  # `fit` returns this object


@keras_export("keras.callbacks.ProgbarLogger")
class ProgbarLogger(Callback):
    """Progress bar with running metrics.  Metric values live on the device; the bar converts them at most four times a
    second (and at the last step), so printing never forces a device read-back per step."""

    REFRESH_SECONDS = 0.25

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
        self.verbose = 1 if verbose == "auto" else verbose
        self.epochs = params["epochs"]
        self.target = params["steps"]

    # -- bar life cycle ------------------------------------------------------------------
    def _start_bar(self):
        self.seen = 0
        self.progbar = Progbar(target=self.target, verbose=self.verbose, unit_name="step")

    def _advance(self, batch, logs):
        if self.progbar is None:
            self._start_bar()
        self.seen = batch + 1
        if self.verbose != 1:
            return
        now = time.time()
        at_end = self.target is not None and self.seen >= self.target
        if not at_end and now - self._last_print < self.REFRESH_SECONDS:
            self.progbar._seen_so_far = self.seen
            return
        self._last_print = now
        values = to_python(logs or {})
        values.pop("outputs", None)
        self.progbar.update(self.seen, list(values.items()), finalize=False)

    def _finish(self, logs):
        if self.progbar is None:
            self._start_bar()
        if self.target is None:
            self.target = self.progbar.target = self.seen
        self.progbar.update(self.target, list(to_python(logs or {}).items()), finalize=True)

    # -- hooks ---------------------------------------------------------------------------
    def on_train_begin(self, logs=None):
        self._called_in_fit = True

    def on_epoch_begin(self, epoch, logs=None):
        self._start_bar()
        if self.verbose and self.epochs > 1:
            io_utils.print_msg(f"Epoch {epoch + 1}/{self.epochs}")

    def on_train_batch_end(self, batch, logs=None):
        self._advance(batch, logs)

    def on_epoch_end(self, epoch, logs=None):
        self._finish(logs)

    def on_test_begin(self, logs=None):
        if not self._called_in_fit:  # validation inside fit reports through the epoch's bar
            self._start_bar()

    def on_test_batch_end(self, batch, logs=None):
        if not self._called_in_fit:
            self._advance(batch, logs)

    def on_test_end(self, logs=None):
        if not self._called_in_fit:
            self._finish(logs)

    def on_predict_begin(self, logs=None):
        self._start_bar()

    def on_predict_batch_end(self, batch, logs=None):
        self._advance(batch, None)

    def on_predict_end(self, logs=None):
        self._finish(logs)


def _csv_cell(value):
    """Scalars as they are, sequences as one quoted ``[a, b]`` cell."""
    if isinstance(value, str) or (isinstance(value, np.ndarray) and value.ndim == 0):
        return value
    try:
        items = list(value)
    except TypeError:
        return value
    return '"[' + ", ".join(str(v) for v in items) + ']"'


@keras_export("keras.callbacks.CSVLogger")
class CSVLogger(Callback):
    """One row per epoch: ``epoch`` followed by the logged quantities in sorted order (validation columns are reserved even
    when the first epoch had none: a later epoch may bring them)."""

    def __init__(self, filename, separator=",", append=False):
        super().__init__()
        self.filename = os.fspath(filename)
        self.sep, self.append = separator, append
        self.csv_file = None
        self.writer = None
        self.keys = None
        self.append_header = True

    def on_train_begin(self, logs=None):
        if self.append and os.path.exists(self.filename):
            with open(self.filename) as existing:
                self.append_header = existing.readline() == ""
        if self.csv_file is not None and not self.csv_file.closed:
            self.csv_file.close()
        self.csv_file = open(self.filename, "a" if self.append else "w")
        self.writer = None
        self.keys = None

    def _open_writer(self, logs):
        self.keys = sorted(logs)
        if self.keys and not any(k.startswith("val_") for k in self.keys):
            self.keys += ["val_" + k for k in self.keys]
        dialect = type("_Dialect", (csv.excel,), {"delimiter": self.sep})
        self.writer = csv.DictWriter(self.csv_file, fieldnames=["epoch"] + self.keys, dialect=dialect)
        if self.append_header:
            self.writer.writeheader()

    def on_epoch_end(self, epoch, logs=None):
        logs = logs or {}
        if self.writer is None:
            self._open_writer(logs)
        row = {"epoch": epoch}
        for key in self.keys:
            row[key] = _csv_cell(logs.get(key, "NA"))
        self.writer.writerow(row)
        self.csv_file.flush()

    def on_train_end(self, logs=None):
        if self.csv_file is not None and not self.csv_file.closed:
            self.csv_file.close()
        self.writer = None


@keras_export("keras.callbacks.RemoteMonitor")
class RemoteMonitor(Callback):
    """POSTs the epoch logs to ``root + path`` (as JSON, or as a form field holding a JSON string)."""

    def __init__(self, root="http://localhost:9000", path="/publish/epoch/end/", field="data", headers=None, send_as_json=False):
        super().__init__()
        self.root, self.path, self.field, self.headers, self.send_as_json = root, path, field, headers, send_as_json

    def on_epoch_end(self, epoch, logs=None):
        try:
            import requests
        except ImportError:
            raise ImportError("RemoteMonitor requires the `requests` library.")
        payload = {"epoch": epoch}
        for name, value in (logs or {}).items():
            payload[name] = value.item() if isinstance(value, (np.ndarray, np.generic)) else value
        url = self.root + self.path
        try:
            if self.send_as_json:
                requests.post(url, json=payload, headers=self.headers)
            else:
                requests.post(url, {self.field: json.dumps(payload)}, headers=self.headers)
        except requests.exceptions.RequestException:
            warnings.warn(f"Could not reach RemoteMonitor root server at {self.root}", stacklevel=2)


@keras_export("keras.callbacks.LambdaCallback")
class LambdaCallback(Callback):
    """Callback assembled from plain functions: any hook name may be given as a keyword."""

    _HOOKS = ("on_epoch_begin", "on_epoch_end", "on_train_begin", "on_train_end", "on_test_begin", "on_test_end", "on_predict_begin",
              "on_predict_end", "on_test_batch_begin", "on_test_batch_end", "on_predict_batch_begin", "on_predict_batch_end")

    def __init__(self, on_epoch_begin=None, on_epoch_end=None, on_train_begin=None, on_train_end=None, on_train_batch_begin=None,
                 on_train_batch_end=None, **kwargs):
        super().__init__()
        given = dict(kwargs, on_epoch_begin=on_epoch_begin, on_epoch_end=on_epoch_end, on_train_begin=on_train_begin, on_train_end=on_train_end)
        for name, fn in given.items():
            if fn is not None or name not in self._HOOKS:
                setattr(self, name, fn)
        # the per-batch training hooks go through methods so that the dispatcher sees this class overrides them
        self._batch_begin, self._batch_end = on_train_batch_begin, on_train_batch_end

    def on_train_batch_begin(self, batch, logs=None):
        if self._batch_begin is not None:
            self._batch_begin(batch, logs)

    def on_train_batch_end(self, batch, logs=None):
        if self._batch_end is not None:
            self._batch_end(batch, to_python(logs))
