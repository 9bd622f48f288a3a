"""``FailureDetection``: aborts ``fit`` on every rank when a rank of the job is lost (no counterpart in the reference,
whose jobs wait inside the collective until the library's time-out)."""

from keras_b200.callbacks.base import Callback
from keras_b200.core.export_registry import keras_export


@keras_export("keras.callbacks.FailureDetection")
class FailureDetection(Callback):
    """Checks the host-side rank watchdog before every batch and raises ``RankFailure`` when a peer stopped its heartbeat,
    left, or reported an exception.  An exception that escapes ``fit`` on this rank is published to the others by
    ``on_train_end`` not being reached: wrap ``fit`` in ``with callback.guard():`` to publish it explicitly."""

    def __init__(self, interval_s=0.5, timeout_s=10.0):
        super().__init__()
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self.watchdog = None

    def _ensure(self):
        from keras_b200.parallel import process_groups
        from keras_b200.parallel.watchdog import RankWatchdog

        if self.watchdog is None and process_groups.is_initialized() and process_groups.world_size() > 1:
            self.watchdog = RankWatchdog(self.interval_s, self.timeout_s).start()
        return self.watchdog

    def on_train_begin(self, logs=None):
        self._ensure()

    def on_train_batch_begin(self, batch, logs=None):
        if self.watchdog is not None:
            self.watchdog.check()

    def on_epoch_begin(self, epoch, logs=None):
        if self.watchdog is not None:
            self.watchdog.check()

    def on_train_end(self, logs=None):
        if self.watchdog is not None:
            self.watchdog.stop()

    def guard(self):
        cb = self

        class _Guard:
            def __enter__(self_inner):
                cb._ensure()
                return cb

            def __exit__(self_inner, exc_type, exc, tb):
                from keras_b200.parallel.watchdog import RankFailure

                if exc is not None and cb.watchdog is not None and not isinstance(exc, RankFailure):
                    cb.watchdog.report_failure(exc)
                if cb.watchdog is not None:
                    cb.watchdog.stop()
                return False

        return _Guard()
