"""``TensorBoard`` callback: scalars, histograms, step timing and a device profiler.

Behaviour of keras/src/callbacks/tensorboard.py (log layout ``<log_dir>/train`` and
``<log_dir>/validation``, ``update_freq``, ``histogram_freq``, ``profile_batch`` parsing :344-404).
The reference has no profiler hook for its torch backend; here ``profile_batch`` drives
``torch.profiler`` (CUPTI) and every step is additionally timed with CUDA events.
"""

import os
import time
import warnings

import numpy as np
import torch

from keras_b200.callbacks.base import Callback
from keras_b200.core.export_registry import keras_export


@keras_export("keras.callbacks.TensorBoard")
class TensorBoard(Callback):
    def __init__(self, log_dir="logs", histogram_freq=0, write_graph=True, write_images=False, write_steps_per_second=False,
                 update_freq="epoch", profile_batch=0, embeddings_freq=0, embeddings_metadata=None):
        super().__init__()
        self.log_dir = str(log_dir)
        self.histogram_freq = histogram_freq
        self.write_graph = write_graph
        self.write_images = write_images
        self.write_steps_per_second = write_steps_per_second
        self.update_freq = 1 if update_freq == "batch" else update_freq
        self.embeddings_freq = embeddings_freq
        self.embeddings_metadata = embeddings_metadata
        self._writers = {}
        self._global_train_batch = 0
        self._previous_epoch_iterations = 0
        self._epoch_start_time = 0
        self._batch_start_time = 0
        self._start_batch, self._stop_batch = self._parse_profile_batch(profile_batch)
        self._profiler = None
        self._step_events = None

    @staticmethod
    def _parse_profile_batch(profile_batch):
        error = ValueError(
            "profile_batch must be a non-negative integer or 2-tuple of positive integers. A pair of positive integers "
            f"signifies a range of batches to profile. Found: {profile_batch}"
        )
        if isinstance(profile_batch, str):
            profile_batch = [int(p) for p in profile_batch.split(",")]
        if isinstance(profile_batch, int):
            if profile_batch < 0:
                raise error
            return profile_batch, profile_batch
        if isinstance(profile_batch, (tuple, list)) and len(profile_batch) == 2:
            a, b = profile_batch
            if a < 0 or b < a:
                raise error
            return a, b
        raise error

    def _writer(self, name):
        if name not in self._writers:
            try:
                from torch.utils.tensorboard import SummaryWriter
            except Exception as e:  # pragma: no cover
                raise ImportError(f"The TensorBoard callback needs the `tensorboard` package: {e}")
            self._writers[name] = SummaryWriter(os.path.join(self.log_dir, name))
        return self._writers[name]

    def set_model(self, model):
        super().set_model(model)
        self._train_step = 0
        self._val_step = 0

    def on_train_begin(self, logs=None):
        self._global_train_batch = 0
        self._previous_epoch_iterations = 0
        if self.write_graph and self.model is not None:
            try:
                self._writer("train").add_text("keras", self.model.to_json(), 0)
            except Exception:
                pass

    def on_train_end(self, logs=None):
        self._stop_profiler()
        for w in self._writers.values():
            w.close()
        self._writers = {}

    def on_epoch_begin(self, epoch, logs=None):
        if self.write_steps_per_second:
            self._previous_epoch_iterations = self._global_train_batch
            self._epoch_start_time = time.time()

    def on_train_batch_begin(self, batch, logs=None):
        self._global_train_batch += 1
        if self.write_steps_per_second:
            self._batch_start_time = time.time()
        if self._start_batch and self._global_train_batch == self._start_batch:
            self._start_profiler()
        if torch.cuda.is_available():
            self._step_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._step_events[0].record()

    def on_train_batch_end(self, batch, logs=None):
        if self._profiler is not None:
            self._profiler.step()
            if self._global_train_batch >= self._stop_batch:
                self._stop_profiler()
        write_now = isinstance(self.update_freq, int) and self._global_train_batch % self.update_freq == 0
        if self._step_events is not None:
            self._step_events[1].record()
        if write_now:
            from keras_b200.trainers.trainer import pythonify_logs

            w = self._writer("train")
            for k, v in pythonify_logs(logs or {}).items():
                if np.isscalar(v):
                    w.add_scalar("batch_" + k, v, self._global_train_batch)
            if self.write_steps_per_second:
                dt = time.time() - self._batch_start_time
                w.add_scalar("batch_steps_per_second", 1.0 / max(dt, 1e-9), self._global_train_batch)
            if self._step_events is not None:
                self._step_events[1].synchronize()
                w.add_scalar("batch_device_ms", self._step_events[0].elapsed_time(self._step_events[1]), self._global_train_batch)

    def on_epoch_end(self, epoch, logs=None):
        logs = logs or {}
        train_logs = {k: v for k, v in logs.items() if not k.startswith("val_")}
        val_logs = {k[4:]: v for k, v in logs.items() if k.startswith("val_")}
        if self.write_steps_per_second:
            elapsed = time.time() - self._epoch_start_time
            train_logs["steps_per_second"] = (self._global_train_batch - self._previous_epoch_iterations) / max(elapsed, 1e-9)
        opt = getattr(self.model, "optimizer", None)
        if opt is not None:
            try:
                lr = opt.learning_rate
                train_logs["learning_rate"] = float(lr)
            except Exception:
                pass
        for k, v in train_logs.items():
            if np.isscalar(v):
                self._writer("train").add_scalar("epoch_" + k, v, epoch)
        for k, v in val_logs.items():
            if np.isscalar(v):
                self._writer("validation").add_scalar("epoch_" + k, v, epoch)
        if self.histogram_freq and epoch % self.histogram_freq == 0:
            w = self._writer("train")
            for var in self.model.weights:
                w.add_histogram(var.path.replace(":", "_") + "/histogram", var.numpy().astype("float32"), epoch)
                if self.write_images and var.ndim in (2, 4):
                    arr = var.numpy().astype("float32")
                    if arr.ndim == 2:
                        arr = arr[None, :, :]
                        w.add_image(var.path + "/image", (arr - arr.min()) / max(float(np.ptp(arr)), 1e-9), epoch)
        if self.embeddings_freq and epoch % self.embeddings_freq == 0:
            from keras_b200.layers.core.embedding import Embedding

            for layer in self.model._flatten_layers():
                if isinstance(layer, Embedding) and layer.built:
                    self._writer("train").add_embedding(torch.as_tensor(layer._embeddings.numpy().astype("float32")), tag=layer.name, global_step=epoch)
        for w in self._writers.values():
            w.flush()

    def on_test_end(self, logs=None):
        if self.model is not None and getattr(self.model, "optimizer", None) is not None and logs:
            step = self._global_train_batch
            for k, v in logs.items():
                if np.isscalar(v):
                    self._writer("validation").add_scalar("evaluation_" + k + "_vs_iterations", v, step)

    def _start_profiler(self):
        try:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._profiler = torch.profiler.profile(
                activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(os.path.join(self.log_dir, "plugins", "profile")))
            self._profiler.__enter__()
        except Exception as e:  # pragma: no cover
            warnings.warn(f"Could not start the profiler: {e}")
            self._profiler = None

    def _stop_profiler(self):
        if self._profiler is not None:
            try:
                self._profiler.__exit__(None, None, None)
            except Exception:
                pass
            self._profiler = None
