"""Callback decision logic against the reference: both implementations are driven with the same sequence of epoch logs
on a stand-in model and their observable state is compared after every epoch."""

import csv
import os

import numpy as np
import pytest

import keras_b200 as keras
from tests import oracle


class _Optimizer:
    def __init__(self, lr):
        self.learning_rate = lr


class _Model:
    """What the watched-metric callbacks touch: stop flag, optimizer learning rate, weights, metric list."""

    def __init__(self, lr=0.1):
        self.stop_training = False
        self.optimizer = _Optimizer(lr)
        self.metrics = []
        self.weights_version = 0
        self.built = True

    def get_weights(self):
        return [np.array([self.weights_version])]

    def set_weights(self, w):
        self.weights_version = int(w[0][0])


CURVES = {
    "improves_then_stalls": [1.0, 0.8, 0.7, 0.71, 0.72, 0.69, 0.70, 0.70, 0.70, 0.70, 0.70],
    "noisy": [0.5, 0.6, 0.4, 0.45, 0.41, 0.39, 0.395, 0.394, 0.50, 0.38, 0.385, 0.386],
    "never_improves": [1.0, 1.1, 1.2, 1.3, 1.4, 1.5],
}


def _drive(callback, curve, key, model, epochs_param=None):
    callback.set_model(model)
    callback.set_params({"epochs": epochs_param or len(curve), "steps": 1, "verbose": 0})
    callback.on_train_begin()
    trace = []
    for epoch, value in enumerate(curve):
        model.weights_version = epoch
        callback.on_epoch_begin(epoch)
        logs = {key: value}
        callback.on_epoch_end(epoch, logs)
        trace.append((model.stop_training, round(float(model.optimizer.learning_rate), 10), getattr(callback, "wait", None),
                      None if getattr(callback, "best", None) is None else round(float(callback.best), 6), sorted(logs)))
        if model.stop_training:
            break
    callback.on_train_end()
    return trace, model.weights_version


@pytest.mark.parametrize("curve", sorted(CURVES))
@pytest.mark.parametrize("kwargs", [
    dict(patience=2), dict(patience=0), dict(patience=3, min_delta=0.02), dict(patience=2, restore_best_weights=True),
    dict(patience=2, baseline=0.6), dict(patience=1, start_from_epoch=3), dict(patience=2, mode="max"),
], ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_early_stopping_decisions(curve, kwargs):
    rk = oracle.ref()
    theirs = _drive(rk.callbacks.EarlyStopping(monitor="val_loss", **kwargs), CURVES[curve], "val_loss", _Model())
    ours = _drive(keras.callbacks.EarlyStopping(monitor="val_loss", **kwargs), CURVES[curve], "val_loss", _Model())
    assert ours == theirs


@pytest.mark.parametrize("curve", sorted(CURVES))
@pytest.mark.parametrize("kwargs", [dict(patience=2, factor=0.5), dict(patience=1, factor=0.1, cooldown=2), dict(patience=2, factor=0.5, min_lr=0.04),
                                    dict(patience=1, factor=0.5, min_delta=0.05)], ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_reduce_lr_on_plateau_decisions(curve, kwargs):
    rk = oracle.ref()
    theirs = _drive(rk.callbacks.ReduceLROnPlateau(monitor="loss", **kwargs), CURVES[curve], "loss", _Model())
    ours = _drive(keras.callbacks.ReduceLROnPlateau(monitor="loss", **kwargs), CURVES[curve], "loss", _Model())
    assert ours == theirs


def test_learning_rate_scheduler_and_direction_errors():
    rk = oracle.ref()
    schedule = lambda epoch, lr: lr * 0.5 if epoch % 2 else lr  # noqa: E731
    theirs = _drive(rk.callbacks.LearningRateScheduler(schedule), [1.0] * 5, "loss", _Model(0.2))
    ours = _drive(keras.callbacks.LearningRateScheduler(schedule), [1.0] * 5, "loss", _Model(0.2))
    assert ours == theirs
    for k in (rk, keras):
        with pytest.raises(ValueError):
            _drive(k.callbacks.EarlyStopping(monitor="my_metric"), [1.0, 2.0], "my_metric", _Model())
        with pytest.warns(UserWarning):
            assert k.callbacks.EarlyStopping(mode="sideways").mode == "auto"
        cb = k.callbacks.EarlyStopping(monitor="val_accuracy", patience=1, mode="max")
        trace, _ = _drive(cb, [0.1, 0.2, 0.15, 0.12], "val_accuracy", _Model())
        assert [t[0] for t in trace] == [False, False, True]  # larger is better: stops after the first drop


def test_csv_logger_and_history_rows(tmp_path):
    rk = oracle.ref()
    rows = [{"loss": 1.0, "acc": 0.5}, {"loss": 0.5, "acc": 0.75, "val_loss": 0.6}, {"loss": 0.25, "acc": np.array([0.8, 0.9])}]
    out = []
    for tag, k in (("ref", rk), ("ours", keras)):
        path = os.path.join(tmp_path, f"{tag}.csv")
        logger, history = k.callbacks.CSVLogger(path, separator=";"), k.callbacks.History()
        model = _Model()
        for cb in (logger, history):
            cb.set_model(model)
            cb.on_train_begin()
        for epoch, logs in enumerate(rows):
            for cb in (logger, history):
                cb.on_epoch_end(epoch, dict(logs))
        logger.on_train_end()
        with open(path) as f:
            out.append((list(csv.reader(f, delimiter=";")), history.epoch, {k_: [str(v) for v in vs] for k_, vs in history.history.items()}))
    assert out[1] == out[0]


def test_terminate_on_nan():
    rk = oracle.ref()
    for k in (rk, keras):
        model = _Model()
        cb = k.callbacks.TerminateOnNaN()
        cb.set_model(model)
        cb.on_batch_end(0, {"loss": 0.5})
        assert not model.stop_training
        cb.on_batch_end(1, {"loss": float("nan")})
        assert model.stop_training
