"""``EpochIterator``: cuts the batch stream of a data adapter into the step groups of one epoch.

One object serves all epochs of a ``fit`` / ``evaluate`` / ``predict`` call.  Iterating it yields
``(first_step, last_step, batches)`` where ``batches`` holds up to ``steps_per_execution`` batches.  The rules
(behaviour of keras/src/trainers/epoch_iterator.py:49-177):

* ``steps_per_epoch`` given: an epoch is that many steps and the batch stream is *not* restarted between epochs; it is
  restarted only after it ran dry, which also ends the epoch early with a warning;
* otherwise an epoch is one pass over the adapter; a stream of unknown length is followed until it stops and its length
  is remembered for the following epochs;
* ``keras.config.set_max_steps_per_epoch`` caps everything (debugging aid).

Each batch passes through ``transform`` as it is pulled (the trainers install the host-to-device stager there), so a
consumer that asks for the next group while the previous one is still computing overlaps the copy with the compute.
"""

import warnings

from keras_b200.core import config
from keras_b200.trainers import data_adapters

_OUT_OF_DATA = ("Your input ran out of data; interrupting training. Make sure that your dataset or generator can generate at least "
                "`steps_per_epoch * epochs` batches. You may need to use the `.repeat()` function when building your dataset.")


class EpochIterator:
    def __init__(self, x, y=None, sample_weight=None, batch_size=None, steps_per_epoch=None, shuffle=False, class_weight=None,
                 steps_per_execution=1, transform=None):
        self.data_adapter = data_adapters.get_data_adapter(x=x, y=y, sample_weight=sample_weight, batch_size=batch_size,
                                                           steps_per_epoch=steps_per_epoch, shuffle=shuffle, class_weight=class_weight)
        self.steps_per_execution = max(1, int(steps_per_execution or 1))
        self._user_steps = steps_per_epoch          # what the caller asked for (decides restart and warning rules)
        cap = config.max_steps_per_epoch()
        self.steps_per_epoch = steps_per_epoch if cap is None else (cap if steps_per_epoch is None else min(cap, steps_per_epoch))
        self.transform = transform
        self._stream = None                         # live batch iterator
        self._pulled = 0                            # batches taken from the live iterator
        self._length = self.data_adapter.num_batches

    # ------------------------------------------------------------------------------------
    @property
    def num_batches(self):
        """Steps of one epoch when known (drives progress bars), else ``None``."""
        return self.steps_per_epoch or self._length

    def reset(self):
        """Forget the live stream: the next epoch starts a new pass over the adapter."""
        self._stream = None
        self._pulled = 0
        self._length = self.data_adapter.num_batches
        self.data_adapter.on_epoch_end()

    def _open(self):
        self._stream = iter(self.data_adapter.get_numpy_iterator())
        self._pulled = 0

    def _pull(self):
        batch = next(self._stream)
        self._pulled += 1
        return batch if self.transform is None else self.transform(batch)

    def __iter__(self):
        return self._epoch()

    def enumerate_epoch(self):
        return self._epoch()

    def _epoch(self):
        bounded = self.steps_per_epoch is not None
        if self._stream is None or not bounded:
            self._open()
        limit = self.steps_per_epoch if bounded else self._length
        step, dry = 0, False
        while limit is None or step < limit:
            want = self.steps_per_execution if limit is None else min(self.steps_per_execution, limit - step)
            group = []
            for _ in range(want):
                if self._length is not None and self._pulled >= self._length:
                    dry = True  # a stream of known length: do not even ask it for more
                    break
                try:
                    group.append(self._pull())
                except StopIteration:
                    dry = True
                    break
            if group:
                yield step, step + len(group) - 1, group
                step += len(group)
            if dry:
                break
        if dry:
            if self._length is None:
                self._length = self._pulled
            if self._user_steps is not None and step < limit:
                warnings.warn(_OUT_OF_DATA, stacklevel=2)
            self._stream = None
        elif self._length is not None and self._pulled >= self._length:
            self._stream = None
        self.data_adapter.on_epoch_end()
