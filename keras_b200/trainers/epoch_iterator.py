"""``EpochIterator``: turns a data adapter into ``(begin_step, end_step, batches)`` per execution.

Behaviour of keras/src/trainers/epoch_iterator.py:49-177: ``steps_per_execution`` grouping,
``steps_per_epoch`` for infinite data, running-out-of-data warnings, debug caps.
"""

import contextlib
import warnings

from keras_b200.core import config
from keras_b200.trainers import data_adapters


class EpochIterator:
    def __init__(self, x, y=None, sample_weight=None, batch_size=None, steps_per_epoch=None, shuffle=False, class_weight=None, steps_per_execution=1):
        self.steps_per_epoch = steps_per_epoch
        self.steps_per_execution = steps_per_execution
        self._current_iterator = None
        self._epoch_iterator = None
        self._steps_seen = 0
        self.data_adapter = data_adapters.get_data_adapter(x=x, y=y, sample_weight=sample_weight, batch_size=batch_size,
                                                           steps_per_epoch=steps_per_epoch, shuffle=shuffle, class_weight=class_weight)
        self._num_batches = self.data_adapter.num_batches
        if config.max_steps_per_epoch() is not None:
            cap = config.max_steps_per_epoch()
            self.steps_per_epoch = cap if self.steps_per_epoch is None else min(cap, self.steps_per_epoch)

    def _get_iterator(self):
        return self.data_adapter.get_numpy_iterator()

    def _interrupted_warning(self):
        warnings.warn("Your input ran out of data; interrupting training. Make sure that your dataset or generator can generate at least `steps_per_epoch * epochs` batches. You may need to use the `.repeat()` function when building your dataset.", stacklevel=2)

    def reset(self):
        self._current_iterator = None
        self._num_batches = self.data_adapter.num_batches
        self._steps_seen = 0
        self._epoch_iterator = None
        self.data_adapter.on_epoch_end()

    def _enumerate_iterator(self):
        steps_per_epoch = self.steps_per_epoch or self._num_batches or -1
        if steps_per_epoch > 0:
            if self._current_iterator is None or self.steps_per_epoch is None:
                self._current_iterator = iter(self._get_iterator())
                self._steps_seen = 0
            for step in range(0, steps_per_epoch, self.steps_per_execution):
                if self._num_batches and self._steps_seen >= self._num_batches:
                    if self.steps_per_epoch:
                        self._interrupted_warning()
                    break
                self._steps_seen += self.steps_per_execution
                yield step, min(step + self.steps_per_execution, steps_per_epoch) - 1, self._current_iterator
            if self._num_batches and self._steps_seen >= self._num_batches:
                self._current_iterator = iter(self._get_iterator())
                self._steps_seen = 0
        else:
            iterator = iter(self._get_iterator())
            step = -self.steps_per_execution
            while True:
                step += self.steps_per_execution
                self._steps_seen = step + self.steps_per_execution
                yield step, step + self.steps_per_execution - 1, iterator
        self.data_adapter.on_epoch_end()

    def __iter__(self):
        self._epoch_iterator = self._enumerate_iterator()
        return self

    def __next__(self):
        buffer = []
        begin_step, end_step, iterator = next(self._epoch_iterator)
        with self.catch_stop_iteration():
            for _ in range(self.steps_per_execution):
                data = next(iterator)
                buffer.append(data)
            return begin_step, end_step, buffer
        if buffer:
            return begin_step, end_step, buffer
        raise StopIteration

    def enumerate_epoch(self):
        for begin_step, end_step, data in self:
            yield begin_step, end_step, data

    @contextlib.contextmanager
    def catch_stop_iteration(self):
        try:
            yield
        except StopIteration:
            if self._num_batches is None:
                self._num_batches = self._steps_seen
            self._interrupted_warning()
            self._current_iterator = None
            self.data_adapter.on_epoch_end()

    @property
    def num_batches(self):
        if self.steps_per_epoch:
            return self.steps_per_epoch
        return self._num_batches
