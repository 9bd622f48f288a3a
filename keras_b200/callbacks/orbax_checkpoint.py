"""``OrbaxCheckpoint``: step-numbered checkpoint directories holding the model state tree.

The reference callback (keras/src/callbacks/orbax_checkpoint.py:58-377) delegates to the
``orbax`` package, which is a JAX library.  Here the same interface (``directory``,
``save_freq``, ``max_to_keep``, ``save_on_background``, monitor/``save_best_only``) writes one
directory per step containing ``config.json``, the state tree as ``state.npz`` and ``assets``;
only the chief process writes, all processes meet at a host-side barrier afterwards.
"""

import json
import os
import shutil
import threading

import numpy as np

from keras_b200.callbacks.watch import MonitorCallback, is_chief as _is_chief
from keras_b200.core.export_registry import keras_export


def _flatten(prefix, tree_, out):
    for k, v in tree_.items():
        key = f"{prefix}/{k}" if prefix else k
        if isinstance(v, dict):
            _flatten(key, v, out)
        else:
            out[key] = v


@keras_export("keras.callbacks.OrbaxCheckpoint")
class OrbaxCheckpoint(MonitorCallback):
    def __init__(self, directory, monitor="val_loss", verbose=0, save_best_only=False, mode="auto", save_freq="epoch",
                 initial_value_threshold=None, max_to_keep=1, save_on_background=True, save_weights_only=False):
        super().__init__(monitor, mode, baseline=initial_value_threshold)
        self.directory = os.fspath(directory)
        self.verbose = verbose
        self.save_best_only = save_best_only
        self.save_freq = save_freq
        self.max_to_keep = max_to_keep
        self.save_on_background = save_on_background
        self.save_weights_only = save_weights_only
        self._batches_seen_since_last_saving = 0
        self._last_batch_seen = 0
        self._current_epoch = 0
        self._total_batches_seen = 0
        self._thread = None
        if save_freq != "epoch" and not isinstance(save_freq, int):
            raise ValueError(f"Unrecognized save_freq: {save_freq}")

    def _should_save_on_batch(self, batch):
        if self.save_freq == "epoch":
            return False
        add = batch + 1 if batch <= self._last_batch_seen else batch - self._last_batch_seen
        self._batches_seen_since_last_saving += add
        self._last_batch_seen = batch
        self._total_batches_seen += add
        if self._batches_seen_since_last_saving >= self.save_freq:
            self._batches_seen_since_last_saving = 0
            return True
        return False

    def _write(self, step, state, config_json):
        path = os.path.join(self.directory, str(step))
        tmp = path + ".tmp"
        os.makedirs(tmp, exist_ok=True)
        flat = {}
        _flatten("", state, flat)
        np.savez(os.path.join(tmp, "state.npz"), **{k.replace("/", "|"): v for k, v in flat.items()})
        with open(os.path.join(tmp, "config.json"), "w") as f:
            f.write(config_json)
        if os.path.exists(path):
            shutil.rmtree(path)
        os.rename(tmp, path)
        steps = sorted(int(d) for d in os.listdir(self.directory) if d.isdigit())
        if self.max_to_keep:
            for old in steps[:-self.max_to_keep]:
                shutil.rmtree(os.path.join(self.directory, str(old)), ignore_errors=True)

    def _save_checkpoint(self, step, logs=None):
        self.wait_until_finished()
        if _is_chief():
            os.makedirs(self.directory, exist_ok=True)
            state = self.model.get_state_tree(value_format="numpy_array")
            if self.save_weights_only:
                state = {k: v for k, v in state.items() if k in ("trainable_variables", "non_trainable_variables")}
            try:
                config_json = self.model.to_json()
            except Exception:
                config_json = json.dumps({})
            if self.save_on_background:
                self._thread = threading.Thread(target=self._write, args=(step, state, config_json), daemon=True)
                self._thread.start()
            else:
                self._write(step, state, config_json)
        _host_barrier()

    def wait_until_finished(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def on_train_batch_end(self, batch, logs=None):
        if self._should_save_on_batch(batch):
            self._save_checkpoint(self._total_batches_seen, logs)

    def on_epoch_begin(self, epoch, logs=None):
        self._current_epoch = epoch

    def on_epoch_end(self, epoch, logs=None):
        if self.save_freq != "epoch":
            return
        if self.save_best_only:
            if self.monitor_op is None:
                self._set_monitor_op()
            current = (logs or {}).get(self.monitor)
            if current is None or not self._is_improvement(current, self.best):
                return
            self.best = current
        self._save_checkpoint(epoch, logs)

    def on_train_end(self, logs=None):
        self.wait_until_finished()


def load_state_from_directory(model, directory, step=None):
    """Restore a model from a directory written by ``OrbaxCheckpoint`` (latest step by default)."""
    steps = sorted(int(d) for d in os.listdir(directory) if d.isdigit())
    if not steps:
        raise FileNotFoundError(f"No checkpoint steps found in {directory}")
    step = steps[-1] if step is None else step
    data = np.load(os.path.join(directory, str(step), "state.npz"))
    tree_ = {}
    for key in data.files:
        parts = key.replace("|", "/").split("/")
        cur = tree_
        for p in parts[:-1]:
            cur = cur.setdefault(p, {})
        cur[parts[-1]] = data[key]
    model.set_state_tree(tree_)
    return step


def _host_barrier():
    """Barrier on the CPU (gloo) group with a timeout; no-op in single-process runs."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            from keras_b200.parallel import process_groups

            dist.barrier(group=process_groups.host_group())
    except Exception:
        pass
