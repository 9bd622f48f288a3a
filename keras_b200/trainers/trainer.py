"""``Trainer``: ``compile`` / ``fit`` / ``evaluate`` / ``predict`` and the step functions.

Behaviour of keras/src/trainers/trainer.py:19-1228 (compile, loss / metric plumbing, symbolic
build, compile config) and keras/src/backend/torch/trainer.py:27-621 (the eager train step:
forward → zero grads → loss → scale → backward → optimizer).  Differences by design:

* batches move host→device through pinned staging on a copy stream, one step ahead;
* metrics stay on the device; logs are converted to Python floats only when a callback reads
  them (``LazyLogs``), so the step loop has no per-step device→host sync;
* under ``DataParallel`` / ``ModelParallel`` the gradient reduction and the optimizer update are
  run by ``keras_b200.parallel`` engines (fused all-reduce + update kernels) instead of a DDP
  wrapper, and metric state is reduced once per read as one packed buffer.
"""

import inspect
import platform
import warnings

import numpy as np
import torch

from keras_b200 import metrics as metrics_module
from keras_b200 import optimizers, tree
from keras_b200.core import config
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.core.tensor import convert_to_tensor, get_device
from keras_b200.trainers import data_adapters
from keras_b200.trainers.compile_utils import CompileLoss, CompileMetrics
from keras_b200.trainers.data_adapters import data_adapter_utils
from keras_b200.trainers.epoch_iterator import EpochIterator


class LazyLogs(dict):
    """Log dict whose values may be device scalars; ``float`` conversion happens on first read."""

    def _resolve(self, v):
        if isinstance(v, torch.Tensor):
            return float(v) if v.ndim == 0 else v.detach().cpu().numpy()
        return v

    def __getitem__(self, k):
        v = dict.__getitem__(self, k)
        if isinstance(v, torch.Tensor):
            v = self._resolve(v)
            dict.__setitem__(self, k, v)
        return v

    def get(self, k, default=None):
        return self[k] if k in self else default

    def items(self):
        return [(k, self[k]) for k in dict.keys(self)]

    def values(self):
        return [self[k] for k in dict.keys(self)]

    def copy(self):
        return LazyLogs(dict.items(self))


def pythonify_logs(logs):
    """Plain Python values, nested dicts flattened, keys in sorted order (keras/src/utils/python_utils.py:165-194: histories
    and ``evaluate(return_dict=True)`` list ``accuracy`` before ``loss``)."""
    out = {}
    for k, v in sorted((logs or {}).items()):
        if isinstance(v, dict):
            out.update(pythonify_logs(v))
        else:
            if isinstance(v, torch.Tensor):
                v = float(v) if v.ndim == 0 else v.detach().cpu().numpy()
            elif isinstance(v, np.generic):
                v = float(v)
            out[k] = v
    return out


class Trainer:
    def __init__(self):
        self._lock = False
        self._run_eagerly = False
        self._jit_compile = None
        self.compiled = False
        self.loss = None
        self.steps_per_execution = 1
        self._initial_epoch = None
        self._compute_loss_has_training_arg = "training" in inspect.signature(self.compute_loss).parameters
        self._compile_loss = None
        self._compile_metrics = None
        self._loss_tracker = None

    def _init_trainer_state(self):
        self.train_function = None
        self.test_function = None
        self.predict_function = None
        self.stop_training = False
        self._parallel_engine = None

    # -- compile -------------------------------------------------------------------------
    def compile(self, optimizer="rmsprop", loss=None, loss_weights=None, metrics=None, weighted_metrics=None, run_eagerly=False,
                steps_per_execution=1, jit_compile="auto", auto_scale_loss=True):
        optimizer = optimizers.get(optimizer)
        self.optimizer = optimizer
        if auto_scale_loss and self.dtype_policy.name == "mixed_float16" and self.optimizer and not isinstance(self.optimizer, optimizers.LossScaleOptimizer):
            self.optimizer = optimizers.LossScaleOptimizer(self.optimizer, name="loss_scale_optimizer")
        if hasattr(self, "output_names"):
            output_names = self.output_names
        else:
            output_names = None
        if loss is not None:
            self._compile_loss = CompileLoss(loss, loss_weights, output_names=output_names)
            self.loss = loss
        else:
            self._compile_loss = None
        if metrics is not None or weighted_metrics is not None:
            self._compile_metrics = CompileMetrics(metrics, weighted_metrics, output_names=output_names)
        else:
            self._compile_metrics = None
        # torch-style eager execution: a tracing compiler is never on the hot path
        self.jit_compile = False if jit_compile == "auto" else jit_compile
        self._jit_request = jit_compile  # "auto" and True allow the step to be captured for replay; False forbids it
        self.run_eagerly = run_eagerly
        self.stop_training = False
        self.compiled = True
        self._loss_tracker = metrics_module.Mean(name="loss")
        self.steps_per_execution = steps_per_execution
        self.train_function = None
        self.test_function = None
        self.predict_function = None
        self._parallel_engine = None
        self._compile_config = {
            "optimizer": optimizer, "loss": loss, "loss_weights": loss_weights, "metrics": metrics,
            "weighted_metrics": weighted_metrics, "run_eagerly": run_eagerly, "steps_per_execution": steps_per_execution,
            "jit_compile": jit_compile,
        }

    @property
    def jit_compile(self):
        return bool(self._jit_compile)

    @jit_compile.setter
    def jit_compile(self, value):
        self._jit_compile = value

    @property
    def run_eagerly(self):
        return self._run_eagerly

    @run_eagerly.setter
    def run_eagerly(self, value):
        self._run_eagerly = value

    @property
    def metrics(self):
        metrics = []
        if self.compiled:
            if self._loss_tracker is not None:
                metrics.append(self._loss_tracker)
            if self._compile_metrics is not None:
                metrics.append(self._compile_metrics)
            if self._compile_loss is not None:
                metrics.extend(self._compile_loss.metrics)
        metrics.extend(self._metrics)
        for layer in self._flatten_layers(include_self=False):
            if isinstance(layer, Trainer):
                continue
            metrics.extend(layer._metrics)
        return metrics

    @property
    def metrics_names(self):
        return [m.name for m in self.metrics]

    def reset_metrics(self):
        for m in self.metrics:
            m.reset_state()

    def _get_own_metrics(self):
        metrics = []
        if self._loss_tracker is not None:
            metrics.append(self._loss_tracker)
        if self._compile_metrics is not None:
            metrics.append(self._compile_metrics)
        if self._compile_loss is not None:
            metrics.extend(self._compile_loss.metrics)
        metrics.extend(self._metrics)
        return metrics

    # -- loss / metrics ------------------------------------------------------------------
    def compute_loss(self, x=None, y=None, y_pred=None, sample_weight=None, training=True):
        del x, training
        losses = []
        if self._compile_loss is not None:
            loss = self._compile_loss(y, y_pred, sample_weight)
            if loss is not None:
                losses.append(loss)
        for loss in self.losses:
            losses.append(self._aggregate_additional_loss(loss))
        if len(losses) == 1:
            return losses[0]
        if not losses:
            return torch.zeros((), device=get_device())
        total = losses[0]
        for l in losses[1:]:
            total = total + l
        return total

    def _compute_loss(self, x=None, y=None, y_pred=None, sample_weight=None, training=True):
        if self._compute_loss_has_training_arg:
            return self.compute_loss(x, y, y_pred, sample_weight, training=training)
        return self.compute_loss(x, y, y_pred, sample_weight)

    def _aggregate_additional_loss(self, loss):
        if not loss.dtype.is_floating_point:
            loss = loss.to(torch.float32)
        return torch.sum(loss)

    def stateless_compute_loss(self, trainable_variables, non_trainable_variables, metrics_variables, x=None, y=None, y_pred=None, sample_weight=None, training=True):
        from keras_b200.core.scopes import StatelessScope

        var_mapping = list(zip(self.trainable_variables, trainable_variables))
        var_mapping.extend(zip(self.non_trainable_variables, non_trainable_variables))
        var_mapping.extend(zip(self.metrics_variables, metrics_variables))
        with StatelessScope(state_mapping=var_mapping) as scope:
            loss = self._compute_loss(x, y, y_pred, sample_weight=sample_weight, training=training)
        non_trainable_variables = []
        for v in self.non_trainable_variables:
            nv = scope.get_current_value(v)
            non_trainable_variables.append(nv if nv is not None else v.value)
        metrics_variables = []
        for v in self.metrics_variables:
            nv = scope.get_current_value(v)
            metrics_variables.append(nv if nv is not None else v.value)
        return loss, (trainable_variables, non_trainable_variables, metrics_variables)

    def compute_metrics(self, x, y, y_pred, sample_weight=None):
        del x
        if self._compile_metrics is not None:
            self._compile_metrics.update_state(y, y_pred, sample_weight)
        return self.get_metrics_result()

    def get_metrics_result(self):
        engine = getattr(self, "_parallel_engine", None)
        mapping = engine.reduced_metric_state(self) if engine is not None else []
        if mapping:
            from keras_b200.core.scopes import StatelessScope

            # distributed: results come from the state summed over replicas; local state is left as it is
            with StatelessScope(state_mapping=mapping):
                return self._local_metrics_result()
        return self._local_metrics_result()

    def _local_metrics_result(self):
        return_metrics = LazyLogs()
        for metric in self.metrics:
            result = metric.result()
            if isinstance(result, dict):
                return_metrics.update(result)
            else:
                return_metrics[metric.name] = result
        return return_metrics

    # -- step functions ------------------------------------------------------------------
    def train_step(self, data):
        x, y, sample_weight = data_adapter_utils.unpack_x_y_sample_weight(data)
        if self._call_has_training_arg:
            y_pred = self(x, training=True)
        else:
            y_pred = self(x)
        loss = self._compute_loss(x=x, y=y, y_pred=y_pred, sample_weight=sample_weight, training=True)
        self._loss_tracker.update_state(loss, sample_weight=next(i for i in tree.flatten(x) if i is not None).shape[0])
        trainable_weights = self.trainable_weights
        if trainable_weights:
            if self.optimizer is not None:
                loss = self.optimizer.scale_loss(loss)
            engine = self._parallel_engine
            if engine is not None:
                engine.backward_and_apply(self, loss, trainable_weights)
            else:
                arena = self._gradient_arena(trainable_weights)
                params = [v._value for v in trainable_weights]
                if arena is None:
                    for p in params:
                        p.grad = None
                    loss.backward()
                    grads = [p.grad for p in params]
                elif arena.unused is None:
                    # first pass over this set of variables: run it unbound to see which variables the loss reaches at all
                    arena.unbind()
                    loss.backward()
                    arena.adopt()
                    grads = arena.gradients()
                else:
                    from keras_b200.kernels import shadow

                    with shadow.arena_backward():
                        loss.backward()
                    grads = arena.gradients()
                opt = self.optimizer
                opt._fused_zeroed_grads = False
                opt._gradients_are_step_storage = arena is not None  # the update may zero what it consumes
                try:
                    opt.apply(grads, trainable_weights)
                finally:
                    opt._gradients_are_step_storage = False
                if arena is None:
                    for p in params:
                        p.grad = None
                elif not opt._fused_zeroed_grads:
                    arena.zero()
        else:
            warnings.warn("The model does not have any trainable weights.")
        return self.compute_metrics(x, y, y_pred, sample_weight=sample_weight)

    def _gradient_arena(self, trainable_weights):
        """Persistent flat gradient storage: ``.grad`` of every trainable parameter is a view into
        one buffer, so pointers are stable across steps (fused optimizer tables are built once, the
        step is CUDA-graph friendly) and the optimizer kernel zeroes gradients as it consumes them."""
        from keras_b200.kernels import dispatch

        if not trainable_weights or not dispatch.enabled(trainable_weights[0]._value):
            return None
        arena = getattr(self, "_grad_arena", None)
        sig = tuple(id(v) for v in trainable_weights)
        if arena is None or arena.signature != sig:
            from keras_b200.parallel.grad_arena import GradArena

            arena = GradArena(trainable_weights)
            self._grad_arena = arena
            from keras_b200.kernels import shadow

            shadow.attach_for_model(self, trainable_weights)
        if arena.unused is not None:
            arena.bind()
        return arena

    def test_step(self, data):
        x, y, sample_weight = data_adapter_utils.unpack_x_y_sample_weight(data)
        if self._call_has_training_arg:
            y_pred = self(x, training=False)
        else:
            y_pred = self(x)
        loss = self._compute_loss(x=x, y=y, y_pred=y_pred, sample_weight=sample_weight, training=False)
        self._loss_tracker.update_state(loss, sample_weight=next(i for i in tree.flatten(x) if i is not None).shape[0])
        return self.compute_metrics(x, y, y_pred, sample_weight=sample_weight)

    def predict_step(self, data):
        x, _, _ = data_adapter_utils.unpack_x_y_sample_weight(data)
        if self._call_has_training_arg:
            return self(x, training=False)
        return self(x)

    @property
    def _call_has_training_arg(self):
        return self._plan.has_training

    def _to_device(self, data):
        """Host batch → device tensors (async from pinned memory when on CUDA)."""
        dev = get_device()

        def move(x):
            if x is None:
                return None
            if isinstance(x, torch.Tensor):
                if x.device != dev:
                    return x.to(dev, non_blocking=True)
                return x
            if isinstance(x, np.ndarray):
                if x.dtype == np.float64:
                    x = x.astype(np.float32)
                if x.dtype == np.uint16:
                    x = x.astype(np.int32)
                elif x.dtype in (np.uint32, np.uint64):
                    x = x.astype(np.int64)
                t = torch.from_numpy(np.ascontiguousarray(x))
                if dev.type == "cuda":
                    return t.pin_memory().to(dev, non_blocking=True)
                return t
            if isinstance(x, (int, float, bool)):
                return x
            return convert_to_tensor(x)

        return tree.map_structure(move, data)

    def make_train_function(self, force=False):
        if self.train_function is not None and not force:
            return self.train_function
        self._ensure_parallel_engine()

        step = self.train_step
        self._graphed_step = None
        if get_device().type == "cuda":
            from keras_b200.trainers.graph_step import GraphedTrainStep

            step = self._graphed_step = GraphedTrainStep(self)

        def multi_step(data_list):
            logs = None
            for data in data_list:
                logs = step(self._to_device(data))
            return logs

        self.train_function = multi_step
        return self.train_function

    def make_test_function(self, force=False):
        if self.test_function is not None and not force:
            return self.test_function
        self._ensure_parallel_engine()

        def multi_step(data_list):
            logs = None
            with torch.no_grad():
                for data in data_list:
                    logs = self.test_step(self._to_device(data))
            return logs

        self.test_function = multi_step
        return self.test_function

    def make_predict_function(self, force=False):
        if self.predict_function is not None and not force:
            return self.predict_function
        self._ensure_parallel_engine()

        def multi_step(data_list):
            outs = []
            with torch.no_grad():
                for data in data_list:
                    outs.append(self.predict_step(self._to_device(data)))
            if len(outs) == 1:
                return outs[0]
            return tree.map_structure(lambda *ts: torch.cat(ts, dim=0), *outs)

        self.predict_function = multi_step
        return self.predict_function

    def _ensure_parallel_engine(self):
        if getattr(self, "_parallel_engine", None) is not None:
            return
        from keras_b200.distribution import distribution_lib

        dist = distribution_lib.distribution()
        if dist is not None:
            from keras_b200.parallel import engine as parallel_engine

            self._parallel_engine = parallel_engine.make_engine(dist, self)

    # -- step loops ----------------------------------------------------------------------
    def _stager(self):
        from keras_b200.trainers.device_stager import DeviceStager

        stager = getattr(self, "_device_stager", None)
        if stager is None or stager.device != get_device():
            stager = self._device_stager = DeviceStager()
        return stager

    def _drive(self, epoch_iterator, run_group, on_begin, on_end, stop_flag):
        """Run one epoch of step groups with one group of look-ahead.

        The kernels of group i are launched first; only then group i+1 is pulled from the data adapter, which also issues
        its host-to-device copies on the stager's stream, so data loading and the copy overlap the compute of group i.
        ``on_end`` (callbacks, which may read metrics back and thereby wait for the device) runs after that."""
        stager = self._stager()
        groups = iter(epoch_iterator)
        pending = next(groups, None)
        logs = {}
        while pending is not None:
            first, last, staged = pending
            on_begin(first)
            logs = run_group([stager.acquire(b) for b in staged])
            pending = next(groups, None)
            on_end(last, logs)
            if getattr(self, stop_flag):
                break
        return logs

    def _epoch_source(self, x, y, sample_weight, batch_size, steps, shuffle, class_weight=None):
        return EpochIterator(x=x, y=y, sample_weight=sample_weight, batch_size=batch_size, steps_per_epoch=steps, shuffle=shuffle,
                             class_weight=class_weight, steps_per_execution=self.steps_per_execution, transform=self._stager().stage)

    def _callback_list(self, callbacks, verbose, epochs, steps, history=False):
        from keras_b200 import callbacks as callbacks_module

        if isinstance(callbacks, callbacks_module.CallbackList):
            return callbacks
        return callbacks_module.CallbackList(callbacks, add_history=history, add_progbar=verbose != 0, verbose=verbose, epochs=epochs, steps=steps,
                                             model=self)

    def fit(self, x=None, y=None, batch_size=None, epochs=1, verbose="auto", callbacks=None, validation_split=0.0, validation_data=None,
            shuffle=True, class_weight=None, sample_weight=None, initial_epoch=0, steps_per_epoch=None, validation_steps=None,
            validation_batch_size=None, validation_freq=1):
        self._assert_compile_called("fit")
        cap = config.max_epochs()
        if cap and cap < epochs:
            warnings.warn("Limiting epochs to %d" % cap)
            epochs = cap
        if validation_split and validation_data is None:
            from keras_b200.trainers.data_adapters import array_slicing

            (x, y, sample_weight), validation_data = array_slicing.train_validation_split((x, y, sample_weight), validation_split=validation_split)
        validation = None
        if validation_data is not None:
            validation = data_adapter_utils.unpack_x_y_sample_weight(validation_data)
        source = self._epoch_source(x, y, sample_weight, batch_size, steps_per_epoch, shuffle, class_weight)
        self._symbolic_build(iterator=source)
        source.reset()
        callbacks = self._callback_list(callbacks, verbose, epochs, source.num_batches, history=True)
        self.stop_training = False
        self._eval_epoch_iterator = None
        self.make_train_function()
        callbacks.on_train_begin()
        last_logs = {}
        for epoch in range(self._initial_epoch or initial_epoch, epochs):
            self.reset_metrics()
            callbacks.on_epoch_begin(epoch)
            step_logs = self._drive(source, self.train_function, callbacks.on_train_batch_begin, callbacks.on_train_batch_end, "stop_training")
            self._check_kernel_status()
            last_logs = dict(self._get_metrics_result_or_logs(step_logs))
            if validation is not None and self._should_eval(epoch, validation_freq):
                vx, vy, vw = validation
                if self._eval_epoch_iterator is None:
                    self._eval_epoch_iterator = self._epoch_source(vx, vy, vw, validation_batch_size or batch_size, validation_steps, False)
                scores = self.evaluate(x=vx, y=vy, sample_weight=vw, batch_size=validation_batch_size or batch_size, steps=validation_steps,
                                       callbacks=callbacks, return_dict=True, _use_cached_eval_dataset=True)
                last_logs.update({"val_" + name: value for name, value in scores.items()})
            callbacks.on_epoch_end(epoch, last_logs)
            if self.stop_training:
                break
        if isinstance(self.optimizer, optimizers.Optimizer) and epochs > 0:
            self.optimizer.finalize_variable_values(self.trainable_weights)
        self._eval_epoch_iterator = None
        callbacks.on_train_end(logs=last_logs)
        return self.history

    def evaluate(self, x=None, y=None, batch_size=None, verbose="auto", sample_weight=None, steps=None, callbacks=None, return_dict=False, **kwargs):
        self._assert_compile_called("evaluate")
        cached = kwargs.pop("_use_cached_eval_dataset", False)
        if kwargs:
            raise ValueError(f"Arguments not recognized: {kwargs}")
        source = self._eval_epoch_iterator if cached else self._epoch_source(x, y, sample_weight, batch_size, steps, False)
        self._symbolic_build(iterator=source)
        source.reset()
        callbacks = self._callback_list(callbacks, verbose, 1, source.num_batches)
        self.make_test_function()
        self.stop_evaluating = False
        callbacks.on_test_begin()
        self.reset_metrics()
        step_logs = self._drive(source, self.test_function, callbacks.on_test_batch_begin, callbacks.on_test_batch_end, "stop_evaluating")
        self._check_kernel_status()
        logs = pythonify_logs(self._get_metrics_result_or_logs(step_logs))
        callbacks.on_test_end(logs)
        return logs if return_dict else self._flatten_metrics_in_order(logs)

    def predict(self, x, batch_size=None, verbose="auto", steps=None, callbacks=None):
        from keras_b200.core.tensor import convert_to_numpy

        source = self._epoch_source(x, None, None, batch_size, steps, False)
        if not all(layer.built for layer in self._flatten_layers()):
            for _, _, staged in source:
                self._symbolic_build(data_batch=self._stager().acquire(staged[0]))
                break
            source.reset()
        callbacks = self._callback_list(callbacks, verbose, 1, source.num_batches)
        self.make_predict_function()
        self.stop_predicting = False
        callbacks.on_predict_begin()
        collected = []  # one host copy of the outputs per step group, concatenated at the end

        def run(batches):
            outputs = self.predict_function(batches)
            collected.append(tree.map_structure(lambda t: t.detach().to("cpu") if isinstance(t, torch.Tensor) else t, outputs))
            return {"outputs": outputs}

        self._drive(source, run, callbacks.on_predict_batch_begin, callbacks.on_predict_batch_end, "stop_predicting")
        self._check_kernel_status()
        callbacks.on_predict_end()
        if not collected:
            return None

        def join(*parts):
            return convert_to_numpy(torch.cat(parts, dim=0)) if isinstance(parts[0], torch.Tensor) else list(parts)

        return tree.map_structure(join, *collected)

    def _check_kernel_status(self):
        """Surface device-side time-outs (bounded waits that ran out in a collective or a tensor-core pipeline) before any
        callback can checkpoint weights that were updated from incomplete results."""
        engine = getattr(self, "_parallel_engine", None)
        if engine is not None and hasattr(engine, "check"):
            engine.check(wait=True)
        if get_device().type == "cuda":
            from keras_b200.kernels import attention as kattention, gemm as kgemm

            kgemm.check_errors()
            kattention.check_errors()
            from keras_b200.kernels import ops as kops

            kops.check_stream_kernels()

    def train_on_batch(self, x, y=None, sample_weight=None, class_weight=None, return_dict=False):
        self._assert_compile_called("train_on_batch")
        if class_weight is not None:
            if tree.is_nested(y):
                raise ValueError("`class_weight` is only supported for Models with a single output.")
            sample_weight = data_adapter_utils.class_weight_to_sample_weights(y, class_weight)
        data = (x, y, sample_weight)
        self._symbolic_build(data_batch=data)
        self.make_train_function()
        self.reset_metrics()
        logs = self.train_function([data])
        logs = pythonify_logs(logs)
        if return_dict:
            return logs
        return self._flatten_metrics_in_order(logs)

    def test_on_batch(self, x, y=None, sample_weight=None, return_dict=False):
        self._assert_compile_called("test_on_batch")
        data = (x, y, sample_weight)
        self._symbolic_build(data_batch=data)
        self.make_test_function()
        self.reset_metrics()
        logs = pythonify_logs(self.test_function([data]))
        if return_dict:
            return logs
        return self._flatten_metrics_in_order(logs)

    def predict_on_batch(self, x):
        from keras_b200.core.tensor import convert_to_numpy

        self.make_predict_function()
        batch_outputs = self.predict_function([(x,)])
        return tree.map_structure(convert_to_numpy, batch_outputs)

    # -- helpers -------------------------------------------------------------------------
    def _should_eval(self, epoch, validation_freq):
        epoch = epoch + 1
        if isinstance(validation_freq, int):
            return epoch % validation_freq == 0
        if isinstance(validation_freq, list):
            return epoch in validation_freq
        raise ValueError(f"Expected `validation_freq` to be a list or int. Received: validation_freq={validation_freq} of the type {type(validation_freq)}.")

    def _get_metrics_result_or_logs(self, logs):
        metric_logs = self.get_metrics_result()
        if isinstance(logs, dict) and set(logs.keys()) == set(metric_logs.keys()):
            return metric_logs
        return logs

    def _flatten_metrics_in_order(self, logs):
        metric_names = []
        for metric in self.metrics:
            if isinstance(metric, CompileMetrics):
                metric_names += [sub.name for sub in metric.metrics]
            else:
                metric_names.append(metric.name)
        results = []
        for name in metric_names:
            if name in logs:
                results.append(logs[name])
        for key in sorted(logs.keys()):
            if key not in metric_names:
                results.append(logs[key])
        if len(results) == 1:
            return results[0]
        return results

    def _assert_compile_called(self, method_name=None):
        if not self.compiled:
            msg = "You must call `compile()` before "
            msg += f"calling `{method_name}()`." if method_name else "using the model."
            raise ValueError(msg)

    def _symbolic_build(self, iterator=None, data_batch=None):
        model_unbuilt = not all(layer.built for layer in self._flatten_layers())
        compile_metrics_unbuilt = self._compile_metrics is not None and not self._compile_metrics.built
        compile_loss_unbuilt = self._compile_loss is not None and not self._compile_loss.built
        optimizer_unbuilt = getattr(self, "optimizer", None) is not None and not self.optimizer.built
        if model_unbuilt or compile_metrics_unbuilt or compile_loss_unbuilt:
            if data_batch is None:
                for _, _, data_or_iterator in iterator:
                    data_batch = data_or_iterator[0] if isinstance(data_or_iterator, (list, tuple)) and len(data_or_iterator) >= 1 and not isinstance(data_or_iterator, tuple) else data_or_iterator
                    break

            def to_spec(v):
                if v is None:
                    return None
                if isinstance(v, KerasTensor):
                    return v
                if hasattr(v, "shape") and hasattr(v, "dtype"):
                    d = standardize_dtype(v.dtype)
                    if d == "float64":
                        d = "float32"
                    return KerasTensor(tuple(v.shape), dtype=d)
                return v

            from keras_b200.trainers.device_stager import Staged

            if isinstance(data_batch, Staged):
                data_batch = data_batch.data
            data_batch = tree.map_structure(to_spec, data_batch)
            x, y, sample_weight = data_adapter_utils.unpack_x_y_sample_weight(data_batch)
            try:
                y_pred = self.compute_output_spec(x, training=False) if self._call_has_training_arg and not model_unbuilt else None
                if y_pred is None:
                    from keras_b200.core.tensor import compute_output_spec

                    if model_unbuilt:
                        # build eagerly with a zero batch: creates every variable with real shapes
                        y_pred = compute_output_spec(lambda xx: self(xx, training=False) if self._call_has_training_arg else self(xx), x)
                    else:
                        y_pred = compute_output_spec(lambda xx: self(xx), x)
            except Exception as e:
                raise RuntimeError(
                    "Unable to automatically build the model. Please build it yourself before calling fit/evaluate/predict. "
                    "A model is 'built' when its variables have been created and its `self.built` attribute is True. Usually, "
                    "calling the model on a batch of data is the right way to build it.\nException encountered:\n" f"'{e}'"
                )
            # variables created while tracing are registered for initialisation and get their values here, on the real device
            from keras_b200.core.variables import initialize_all_variables

            initialize_all_variables()
            if compile_metrics_unbuilt:
                self._compile_metrics.build(y, y_pred)
            if compile_loss_unbuilt:
                self._compile_loss.build(y, y_pred)
        if optimizer_unbuilt:
            with torch.no_grad():
                self.optimizer.build(self.trainable_variables)
        self._post_build()

    # -- compile config ------------------------------------------------------------------
    def get_compile_config(self):
        from keras_b200.saving import serialization_lib

        if self.compiled and hasattr(self, "_compile_config"):
            return serialization_lib.serialize_keras_object(dict(self._compile_config))

    def compile_from_config(self, config):
        from keras_b200.saving import serialization_lib

        has_overridden_compile = self.__class__.compile != Trainer.compile
        if has_overridden_compile:
            warnings.warn("`compile()` was not called as part of model loading because the model's `compile()` method is custom. All subclassed Models that have `compile()` overridden should also override `get_compile_config()` and `compile_from_config(config)`. Alternatively, you can call `compile()` manually after loading.", stacklevel=2)
            return
        config = serialization_lib.deserialize_keras_object(config)
        self.compile(**config)
        if hasattr(self, "optimizer") and self.built:
            with torch.no_grad():
                self.optimizer.build(self.trainable_variables)
