"""Shared pieces of the callbacks that follow one metric or fire every N batches.

``MetricWatch`` answers two questions for a metric name: in which direction is it better, and is a new value better than
a reference by more than ``min_delta``.  ``MonitorCallback`` (the public base class, keras/src/callbacks/monitor_callback.py)
owns one.  ``BatchCadence`` counts batches across epoch boundaries for the callbacks that act every ``save_freq`` batches.
"""

import numpy as np

from keras_b200.callbacks.base import Callback

def _model_metric(model, name):
    """The metric object called ``name`` among the model's metrics (compile metrics unpacked), or None."""
    from keras_b200.trainers.compile_utils import CompileMetrics

    for metric in getattr(model, "metrics", []) or []:
        members = metric.metrics if isinstance(metric, CompileMetrics) else [metric]
        for m in members:
            if m.name == name:
                return m
    return None


class MetricWatch:
    def __init__(self, monitor, mode="auto", min_delta=0.0):
        if mode not in ("auto", "min", "max"):
            raise ValueError(f"mode '{mode}' is unknown: expected 'auto', 'min' or 'max'.")
        self.monitor, self.mode = monitor, mode
        self.margin = abs(min_delta)
        self.larger_is_better = None  # resolved on first use: needs the model for mode="auto"

    def resolve(self, model, owner="callback"):
        if self.mode != "auto":
            self.larger_is_better = self.mode == "max"
            return
        name = self.monitor[4:] if self.monitor.startswith("val_") else self.monitor
        if name == "loss":
            self.larger_is_better = False
        metric = _model_metric(model, name)
        direction = getattr(metric, "_direction", None)
        if direction is not None:
            self.larger_is_better = direction == "up"
        if self.larger_is_better is None:
            # no guessing from the metric's name: only "loss" and metrics that declare a direction are known
            raise ValueError(
                f"{owner} callback received monitor={self.monitor}, but Keras isn't able to automatically determine whether that metric "
                "should be maximized or minimized. Pass `mode='max'` in order to monitor based on the highest metric value, or pass "
                "`mode='min'` in order to use the lowest value.")

    @property
    def resolved(self):
        return self.larger_is_better is not None

    def improved(self, value, reference):
        if reference is None:
            return True
        if self.larger_is_better:
            return value - self.margin > reference
        return value + self.margin < reference


class MonitorCallback(Callback):
    """Base class of callbacks that watch one metric.  Public attributes: ``monitor``, ``mode``, ``best``, ``min_delta``
    and ``monitor_op`` (``numpy.less`` / ``numpy.greater`` once the direction is known)."""

    def __init__(self, monitor="val_loss", mode="auto", baseline=None, min_delta=0):
        super().__init__()
        if mode not in ("auto", "min", "max"):
            import warnings

            warnings.warn(f"{self.__class__.__name__} mode '{mode}' is unknown, fallback to auto mode.", stacklevel=2)
            mode = "auto"
        self._watch = MetricWatch(monitor, mode, min_delta)
        self.monitor, self.mode, self.best = monitor, mode, baseline
        self.min_delta = abs(min_delta)

    @property
    def monitor_op(self):
        if not self._watch.resolved:
            return None
        return np.greater if self._watch.larger_is_better else np.less

    def _set_monitor_op(self):
        self._watch.resolve(self.model, owner=self.__class__.__name__)

    def _ensure_direction(self):
        if not self._watch.resolved:
            self._set_monitor_op()

    def _is_improvement(self, monitor_value, reference_value):
        return self._watch.improved(monitor_value, reference_value)


class BatchCadence:
    """Fires once every ``every`` batches, counted over the whole run (batch indices restart at each epoch)."""

    def __init__(self, every):
        self.every = every          # an int, or "epoch" (never fires on batches)
        self.since_fire = 0
        self.last_index = 0

    @staticmethod
    def validate(every, what):
        if every != "epoch" and not isinstance(every, int):
            raise ValueError(f"{what}. Received: save_freq={every}. Expected either 'epoch' or an integer value.")

    def tick(self, batch):
        if self.every == "epoch":
            return False
        # an index at or below the last one means a new epoch began: `batch + 1` batches ran since then
        self.since_fire += batch + 1 if batch <= self.last_index else batch - self.last_index
        self.last_index = batch
        if self.since_fire >= self.every:
            self.since_fire = 0
            return True
        return False

    def new_epoch(self):
        self.last_index = 0


def is_chief():
    """True on the process that writes files (rank 0 of the job, or the only process)."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank() == 0
    except Exception:
        pass
    return True


def learning_rate_of(optimizer):
    """Current learning rate of ``optimizer`` as a Python float."""
    import torch

    value = optimizer.learning_rate
    if isinstance(value, torch.Tensor):
        value = value.detach().cpu().numpy()
    return float(np.asarray(value))
