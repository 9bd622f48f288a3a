"""The training step as a replayed CUDA graph.

A training step of a small or medium model is hundreds to thousands of kernel launches; issued from Python, the host
becomes the limit long before the device does.  ``GraphedTrainStep`` runs the first steps eagerly (caches fill, lazily
created state appears), then captures one whole step (forward, loss, backward, optimizer update, metric updates)
into a CUDA graph and replays it: one launch per step, with the batch copied into the graph's input buffers first.

What makes the step replayable:

* parameter gradients live in one persistent arena, so every ``.grad`` pointer is fixed;
* the fused optimizer kernels read the learning rate and the iteration counter from device memory, so assigning a
  new learning rate or advancing the counter needs no re-capture;
* metric state lives in device variables that are updated in place.

Data-parallel steps are recordable too: the gradient and metric all-reduces are this package's peer-memory kernels,
whose epoch lives in a device counter, so their launch arguments never change; their status words are read back after
each replay.

A step is captured only when all of this holds: the model runs on CUDA devices (alone, or data parallel on those kernels),
``train_step`` is the stock one, the optimizer took its fused path with device-resident step scalars, and the batch
signature (shapes, dtypes) repeats.  A batch with another signature (the short last batch of an epoch) runs eagerly on
the same variables.  Drawing from a seeded random generator during capture aborts it (the seed is host state that a
replay would freeze) and the model stays eager.  ``compile(jit_compile=False)`` or ``KERAS_B200_CUDA_GRAPHS=0`` switch
capture off; ``jit_compile="auto"`` (the default) and ``True`` allow it.
"""

import os
import traceback
import warnings

import torch

from keras_b200 import tree
from keras_b200.kernels import ops as kops
from keras_b200.random import seed_generator
from keras_b200.trainers.data_adapters import data_adapter_utils

_EAGER_STEPS_BEFORE_CAPTURE = 3


def enabled_by_env():
    return os.environ.get("KERAS_B200_CUDA_GRAPHS", "1") != "0"


def _signature(leaves):
    sig = []
    for leaf in leaves:
        if isinstance(leaf, torch.Tensor):
            sig.append((tuple(leaf.shape), leaf.dtype, leaf.device.type, leaf.device.index))
        else:
            sig.append(("py", type(leaf).__name__, leaf if isinstance(leaf, (int, float, bool, str, type(None))) else id(leaf)))
    return tuple(sig)


class GraphedTrainStep:
    def __init__(self, model):
        self.model = model
        self.graph = None
        self.signature = None        # batch signature the graph was captured for
        self._candidate = None       # signature currently being counted towards capture
        self._seen = 0
        self.disabled = None         # reason string once capture is ruled out for good
        self.static_leaves = None
        self.structure = None
        self.out_structure = None
        self.out_leaves = None
        self.out_packed = None       # one tensor holding every 0-dim floating output (snapshotted per replay)
        self.out_packed_index = None
        self.replays = 0
        self.failure_traceback = None
        self._stream = None
        self.launches_per_replay = 0

    # -- eligibility ---------------------------------------------------------------------
    def _why_not_static(self):
        from keras_b200.trainers.trainer import Trainer

        model = self.model
        if not enabled_by_env():
            return "switched off by KERAS_B200_CUDA_GRAPHS=0"
        if getattr(model, "_jit_request", "auto") is False or model.run_eagerly:
            return "jit_compile=False or run_eagerly=True"
        engine = getattr(model, "_parallel_engine", None)
        if engine is not None and not (type(engine).__name__ == "DataParallelEngine" and engine.recordable()):
            return "the parallel engine's collectives cannot be recorded (library collectives, or model parallelism)"
        if type(model).train_step is not Trainer.train_step:
            return "train_step is overridden"
        return None

    def _why_not(self):
        """Everything that decides eligibility, once the optimizer has applied updates."""
        static = self._why_not_static()
        if static is not None:
            return static
        model = self.model
        engine = getattr(model, "_parallel_engine", None)
        opt = model.optimizer
        if opt is None or not getattr(opt, "_step_scalars_on_device", False) or not getattr(opt, "_fused_zeroed_grads", False):
            return "the optimizer update is not the fused one with device-resident step scalars"
        if getattr(model, "_grad_arena", None) is None and engine is None:
            return "no persistent gradient storage"
        return None

    # -- the step ------------------------------------------------------------------------
    def __call__(self, data):
        if self.disabled is not None:
            return self.model.train_step(data)
        data = data_adapter_utils.unpack_x_y_sample_weight(data)  # (x, y) and (x, y, None) are the same batch
        leaves = tree.flatten(data)
        if not any(isinstance(leaf, torch.Tensor) and leaf.is_cuda for leaf in leaves):
            self.disabled = "inputs are not on a CUDA device"
            return self.model.train_step(data)
        sig = _signature(leaves)
        if self.graph is not None:
            if sig == self.signature:
                return self._replay(leaves)
            return self.model.train_step(data)  # an odd batch: eager, same variables
        if sig != self._candidate:
            self._candidate, self._seen = sig, 0
        if self._seen == 0:
            # What rules capture out for good is known before any step runs; such a model never touches the side stream
            # (whose allocator pool would double its memory).  The first step also runs on the caller's stream: it is the one
            # that discovers unused variables and builds caches.
            self.disabled = self._why_not_static()
            self._seen = 1
            return self.model.train_step(data)
        if self._seen < _EAGER_STEPS_BEFORE_CAPTURE:
            self._seen += 1
            logs = self._eager_on_side_stream(data)
            if self._seen == _EAGER_STEPS_BEFORE_CAPTURE:
                self.disabled = self._why_not()
                if self.disabled is not None:
                    torch.cuda.empty_cache()  # the side stream's cached blocks are of no use to eager steps on the main stream
            return logs
        return self._capture(data, leaves, sig)

    def _eager_on_side_stream(self, data):
        """The eager steps that precede capture run on the stream the capture will use: autograd's gradient-accumulation
        nodes remember the stream they were made on, and one made on the default stream would tie the capture to it."""
        if self._stream is None:
            self._stream = torch.cuda.Stream()
        main = torch.cuda.current_stream()
        self._stream.wait_stream(main)
        with torch.cuda.stream(self._stream):
            logs = self.model.train_step(data)
        main.wait_stream(self._stream)
        for leaf in tree.flatten(data):
            if isinstance(leaf, torch.Tensor) and leaf.is_cuda:
                leaf.record_stream(self._stream)
        return logs

    def _capture(self, data, leaves, sig):
        model = self.model
        self.structure = data
        static = [torch.empty_like(leaf).copy_(leaf) if isinstance(leaf, torch.Tensor) else leaf for leaf in leaves]
        static_data = tree.pack_sequence_as(data, static)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        launches_before = kops.launch_count()
        seed_generator.begin_capture()
        try:
            with torch.cuda.graph(graph, stream=self._stream):
                logs = model.train_step(static_data)
                raw = dict(dict.items(logs)) if isinstance(logs, dict) else logs  # device scalars as they are: no read-back here
                out_leaves = tree.flatten(raw)
                packed_index = [i for i, leaf in enumerate(out_leaves)
                                if isinstance(leaf, torch.Tensor) and leaf.ndim == 0 and leaf.is_floating_point() and leaf.is_cuda]
                packed = torch.stack([out_leaves[i].detach().float() for i in packed_index]) if packed_index else None
        except Exception as e:  # capture ruled out: the step that was being captured has not run, so run it eagerly
            seed_generator.end_capture()
            self.disabled = f"capture failed: {type(e).__name__}: {e}"
            self.failure_traceback = traceback.format_exc()
            del graph
            torch.cuda.synchronize()
            if not isinstance(e, seed_generator.CaptureUnsafe):
                warnings.warn(f"The training step could not be captured in a CUDA graph and runs eagerly ({self.disabled}).", stacklevel=2)
            self._resync_host_state()
            torch.cuda.empty_cache()  # what the side-stream steps cached is of no use to the eager steps on the main stream
            return model.train_step(data)
        seed_generator.end_capture()
        self._resync_host_state()
        torch.cuda.empty_cache()      # the graph owns its pool; the warm-up's cached blocks go back to the device
        # launcher calls recorded into the graph: nothing ran yet, each replay runs that many kernels' launchers
        self.launches_per_replay = kops.launch_count() - launches_before
        kops.add_launches(-self.launches_per_replay)
        self.graph, self.signature, self.static_leaves = graph, sig, static
        self.out_structure, self.out_type = raw, type(logs)
        self.out_leaves, self.out_packed, self.out_packed_index = out_leaves, packed, packed_index
        # capture records the step without running it: this batch is the first replay
        return self._replay(leaves, copy_inputs=False)

    def _resync_host_state(self):
        """Recording a step runs its Python side (the optimizer's host mirror of the iteration counter moved) but not its
        kernels: re-read the mirror from the device."""
        opt = self.model.optimizer
        opt._host_step_version = -1
        opt._step()

    def _replay(self, leaves, copy_inputs=True):
        if copy_inputs:
            for dst, src in zip(self.static_leaves, leaves):
                if isinstance(dst, torch.Tensor):
                    dst.copy_(src, non_blocking=True)
        engine = getattr(self.model, "_parallel_engine", None)
        if engine is not None:
            engine.check()
        self.graph.replay()
        if engine is not None:
            engine.after_replay()
        self.replays += 1
        kops.add_launches(self.launches_per_replay)
        self.model.optimizer._note_replayed_step()
        # the graph's output buffers are rewritten by the next replay: hand out a snapshot (one small copy)
        out = list(self.out_leaves)
        if self.out_packed is not None:
            snap = self.out_packed.clone()
            for k, i in enumerate(self.out_packed_index):
                out[i] = snap[k]
        for i, leaf in enumerate(out):
            if isinstance(leaf, torch.Tensor) and leaf is self.out_leaves[i]:
                out[i] = leaf.detach().clone()
        result = tree.pack_sequence_as(self.out_structure, out)
        return self.out_type(result) if isinstance(result, dict) and self.out_type is not dict else result
