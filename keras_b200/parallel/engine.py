"""Execution engines behind ``keras.distribution``: what runs when ``fit`` is called under a distribution.

``DataParallelEngine`` is the counterpart of wrapping the model in DistributedDataParallel
(keras/src/backend/torch/trainer.py:45-92) plus the per-variable metric all-reduce (:207-244):

* at creation every variable (model and optimizer) is broadcast from the first rank of the replica group;
* gradients of all trainable variables live in one flat arena (reverse creation order).  On CUDA the arena is
  a symmetric buffer and one kernel pair per step all-reduces it in place over NVLink peer memory (mean over
  replicas); the fused optimizer kernel then consumes and zeroes it.  With ``KERAS_B200_COMM=nccl`` or on CPU the
  arena is reduced with one library all-reduce;
* metric state is reduced as ONE packed buffer when results are read, and never written back.

``ModelParallelEngine`` adds tensor-parallel variable shards on a second mesh axis (see ``tensor_parallel``).
"""

import torch
import torch.distributed as dist

from keras_b200.parallel import collectives, process_groups
from keras_b200.parallel.grad_arena import GradArena


def make_engine(distribution, model):
    from keras_b200.distribution import distribution_lib

    if isinstance(distribution, distribution_lib.ModelParallel):
        return ModelParallelEngine(distribution, model)
    return DataParallelEngine(distribution, model)


class DataParallelEngine:
    def __init__(self, distribution, model):
        self.distribution = distribution
        mesh = distribution.device_mesh
        self.groups = mesh.backend_mesh
        self.axis = distribution.batch_dim_name or mesh.axis_names[0]
        self.group = self.groups.get_group(self.axis)
        self.members = self.groups.members(self.axis)
        self.world = len(self.members) if process_groups.is_initialized() else 1
        self._arena = None
        self._reducer = None
        self._metric_reducer = None
        self._steps = 0
        self._synced_ids = set()
        self.sync_variables(model)

    # -- variables -----------------------------------------------------------------------
    def _replicated_variables(self, model):
        vs = list(model.variables)
        opt = getattr(model, "optimizer", None)
        if opt is not None and getattr(opt, "built", False):
            vs += list(opt.variables)
        return vs

    def sync_variables(self, model):
        """Broadcast every not-yet-synchronised replicated variable from the first rank of the replica group."""
        if self.world <= 1:
            return
        todo = [v for v in self._replicated_variables(model) if id(v) not in self._synced_ids and getattr(v, "_value", None) is not None]
        if not todo:
            return
        src = self.members[0]
        by_dtype = {}
        for v in todo:
            by_dtype.setdefault(v._value.dtype, []).append(v)
        with torch.no_grad():
            for dtype, vs in by_dtype.items():
                flat = torch.cat([v._value.detach().reshape(-1) for v in vs]) if vs else None
                if flat.dtype == torch.bool:
                    flat = flat.to(torch.uint8)
                collectives.broadcast(flat, src=src, group=self.group)
                off = 0
                for v in vs:
                    n = v._value.numel()
                    v._value.detach().copy_(flat[off:off + n].view(v._value.shape).to(v._value.dtype))
                    off += n
        for v in todo:
            self._synced_ids.add(id(v))

    # -- gradients -----------------------------------------------------------------------
    def _gradient_arena(self, trainable_weights):
        sig = tuple(id(v) for v in trainable_weights)
        if self._arena is not None and self._arena.signature == sig:
            return self._arena
        params = [v._value for v in trainable_weights]
        dev = params[0].device
        if self._reducer is not None:
            self._reducer.close()
            self._reducer = None
        flat = None
        if self.world > 1 and collectives.use_p2p(dev) and all(p.dtype == torch.float32 for p in params):
            numel = GradArena.required_numel(trainable_weights)
            self._reducer = collectives.P2PAllReducer(numel, self.group, self.members)
            flat = self._reducer.flat
        self._arena = GradArena(trainable_weights, flat=flat)
        return self._arena

    def backward_and_apply(self, model, loss, trainable_weights):
        opt = model.optimizer
        first = self._steps == 0
        if first:
            if not opt.built:
                opt.build(trainable_weights)
            self.sync_variables(model)
        arena = self._gradient_arena(trainable_weights)
        if arena.flat.is_cuda:
            from keras_b200.kernels import shadow

            shadow.attach_for_model(model, trainable_weights)
        reduced = False
        if arena.unused is None:
            # first pass over this set of variables: unbound, to see which variables the loss reaches (see GradArena.adopt)
            arena.unbind()
            loss.backward()
            arena.adopt()
        else:
            arena.bind()
            if arena.flat.is_cuda:
                overlap = self._overlap_for(arena, opt)
                if overlap is not None:
                    overlap.begin()
                    shadow.set_slot_observer(overlap.note)
                try:
                    with shadow.arena_backward():
                        loss.backward()
                finally:
                    if overlap is not None:
                        shadow.set_slot_observer(None)
                if overlap is not None:
                    reduced = overlap.finish()
            else:
                loss.backward()
        self._after_backward(trainable_weights)
        if self.world > 1 and not reduced:
            if self._reducer is not None:
                if first:
                    collectives.barrier()  # absorb start-up skew (lazy initialisation, autotuning) on the host
                self._reducer.all_reduce(scale=1.0 / self.world)
            else:
                collectives.all_reduce(arena.flat, group=self.group)
                arena.flat.div_(self.world)
        grads = arena.gradients()
        opt._fused_zeroed_grads = False
        opt._gradients_are_step_storage = True  # the arena is this engine's: the update may zero what it consumes
        try:
            opt.apply(grads, trainable_weights)
        finally:
            opt._gradients_are_step_storage = False
        if not opt._fused_zeroed_grads:
            arena.zero()
        self._steps += 1

    def _overlap_for(self, arena, opt):
        """The bucket schedule that reduces gradients during the backward pass, or ``None``: only the plain data-parallel
        engine with this package's all-reduce, and not while gradients are accumulated over several calls."""
        from keras_b200.parallel import overlap

        if type(self) is not DataParallelEngine or self.world <= 1 or self._reducer is None or not overlap.enabled():
            return None
        if getattr(opt, "gradient_accumulation_steps", None):
            return None
        current = getattr(self, "_overlap", None)
        if current is None or current.arena is not arena or current.reducer is not self._reducer:
            if current is not None:
                current.close()
            current = self._overlap = overlap.GradientOverlap(arena, self._reducer, self.world)
        return current

    def _after_backward(self, trainable_weights):
        """Hook between the backward pass and the replica reduction."""

    # -- metrics -------------------------------------------------------------------------
    def reduced_metric_state(self, model):
        """[(variable, value summed over replicas)] with one packed all-reduce; variables are left untouched."""
        vs = [v for v in model.metrics_variables if getattr(v, "_value", None) is not None]
        if self.world <= 1 or not vs:
            return []
        with torch.no_grad():
            flat = self._reduce_metric_state_p2p(vs)
            if flat is None:
                flat = torch.cat([v._value.detach().reshape(-1).to(torch.float64) for v in vs])
                collectives.all_reduce(flat, group=self.group)
            out, off = [], 0
            for v in vs:
                n = v._value.numel()
                out.append((v, flat[off:off + n].view(v._value.shape).to(v._value.dtype)))
                off += n
        return out

    def _reduce_metric_state_p2p(self, vs):
        """Metric state summed over replicas by this package's all-reduce kernel on a small symmetric buffer (fp32), or
        ``None`` when gradients do not use that path either.  No library collective, so the step stays recordable."""
        if self._reducer is None or not all(v._value.is_cuda for v in vs):
            return None
        n = sum(v._value.numel() for v in vs)
        mr = self._metric_reducer
        if mr is None or mr.numel < n:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("metric state grew while the step was being recorded")
            if mr is not None:
                mr.close()
            mr = self._metric_reducer = collectives.P2PAllReducer(max(1024, 2 * n), self.group, self.members)
            mr.flat.zero_()
        padded = (n + 3) // 4 * 4
        torch.cat([v._value.detach().reshape(-1).float() for v in vs], out=mr.flat[:n])
        mr.all_reduce(0, padded)
        return mr.flat[:n]

    def recordable(self):
        """True when every collective of a training step is (or, before the first step has built the gradient arena, will
        be) one of this package's kernels with device-side epochs."""
        if self.world <= 1 or self._reducer is not None:
            return True
        if self._arena is not None:
            return False  # the arena exists and is reduced by the library
        from keras_b200.core.tensor import get_device

        return collectives.use_p2p(get_device())

    def after_replay(self):
        """A recorded step was replayed: queue the status read-backs that the recorded collectives could not."""
        for r in (self._reducer, self._metric_reducer):
            if r is not None:
                r.post_status()

    def sync_metrics(self, model):
        return self.reduced_metric_state(model)

    def check(self, wait=False):
        for r in (self._reducer, self._metric_reducer):
            if r is not None:
                r.check(wait=wait)

    def close(self):
        if getattr(self, "_overlap", None) is not None:
            self._overlap.close()
            self._overlap = None
        if self._metric_reducer is not None:
            self._metric_reducer.close()
            self._metric_reducer = None
        if self._reducer is not None:
            self._reducer.close()
            self._reducer = None
            self._arena = None


class ModelParallelEngine(DataParallelEngine):
    """Data parallel over ``batch_dim_name`` plus sharded variables on the remaining mesh axes.

    Gradients of a sharded variable are reduced over the batch axis only (its shard differs between model-axis
    peers); replicated variables receive partial gradients on every model-axis peer, which the tensor-parallel
    layers already reduce through their backward collectives, so the same batch-axis reduction applies.
    """

    def __init__(self, distribution, model):
        super().__init__(distribution, model)
        from keras_b200.parallel import tensor_parallel

        self.plan = tensor_parallel.plan_for_model(distribution, model)
        self.sequence_parallel = tensor_parallel.enable_sequence_parallel(distribution, model)

    def _after_backward(self, trainable_weights):
        if self.sequence_parallel is not None:
            self.sequence_parallel.reduce_partial_gradients(trainable_weights)

    def check(self, wait=False):
        super().check(wait=wait)
        if self.sequence_parallel is not None and self.sequence_parallel.fused is not None and wait:
            self.sequence_parallel.fused.check()

    def close(self):
        if self.sequence_parallel is not None:
            from keras_b200.parallel import tensor_parallel

            tensor_parallel.disable_sequence_parallel()
            self.sequence_parallel = None
        super().close()

    def _replicated_variables(self, model):
        return [v for v in super()._replicated_variables(model) if getattr(v, "_shard_slices", None) is None]
