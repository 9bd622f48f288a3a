"""``Callback`` and ``CallbackList`` (keras/src/callbacks/callback.py, callback_list.py).

``CallbackList`` precomputes, per batch-level hook, the callbacks that actually override it, so a hook nobody listens to
costs nothing inside the step loop; epoch- and run-level hooks go to every callback.  Logs reach batch-level hooks as they
come out of the step (device tensors that convert lazily); epoch-level hooks receive plain Python numbers.
"""

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export


def to_python(logs):
    """Logs with every value converted to a Python number (reads device values back)."""
    from keras_b200.trainers.trainer import pythonify_logs

    return pythonify_logs(logs)


_py = to_python


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
        from keras_b200.callbacks.reporting import History, ProgbarLogger

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
    if callable(cb.__dict__.get(hook)):
        return True  # a hook attached to the instance (LambdaCallback)
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
