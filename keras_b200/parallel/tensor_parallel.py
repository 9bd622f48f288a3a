"""Sharded variables for ``ModelParallel`` (the reference realises this only through JAX/GSPMD,
keras/src/backend/jax/distribution_lib.py:32-106; its torch backend converts layouts to DTensor placements but
never applies them to variables, keras/src/backend/torch/distribution_lib.py:186-310).

A variable whose ``TensorLayout`` names mesh axes on some dimensions stores only this rank's shard
(``Variable._value``); ``Variable.shape`` stays the logical (global) shape.  Reading ``variable.value`` outside
a shard-aware layer all-gathers the shards with an autograd-aware collective (backward keeps this rank's slice of
the gradient), which is always correct; layers that recognise the column/row pattern read the shard directly and
communicate activations instead.

Initialisation draws the full value from the seeded initializer on every rank (identical by construction, the
global seed is agreed at ``initialize``) and keeps the local slice, so a sharded model starts from exactly the
values of the unsharded one.
"""

import contextlib

import numpy as np
import torch
import torch.distributed as dist

from keras_b200.core import global_state
from keras_b200.parallel import process_groups


def _axis_info(layout, mesh_groups):
    """[(dim, parts, index, group)] for every sharded dimension of ``layout`` on this rank."""
    out = []
    mesh = layout.device_mesh
    for dim, axis in enumerate(layout.axes):
        if axis is None:
            continue
        size = mesh.shape[mesh.axis_names.index(axis)]
        if size <= 1:
            continue
        out.append((dim, size, mesh_groups.index(axis), mesh_groups.get_group(axis)))
    return out


def shard_slices(shape, layout):
    """Index tuple selecting this rank's shard of a tensor of ``shape`` laid out as ``layout`` (None: replicated)."""
    if layout is None or layout.device_mesh is None or not process_groups.is_initialized():
        return None
    info = _axis_info(layout, layout.device_mesh.backend_mesh)
    if not info:
        return None
    idx = [slice(None)] * len(shape)
    for dim, parts, index, _ in info:
        if shape[dim] % parts != 0:
            raise ValueError(f"Dimension {dim} of shape {tuple(shape)} is not divisible by the {parts} shards of mesh axis {layout.axes[dim]!r}.")
        step = shape[dim] // parts
        idx[dim] = slice(index * step, (index + 1) * step)
    return tuple(idx)


def distribute_tensor(tensor, layout):
    """This rank's shard of a full tensor (a view; replicated layouts return the tensor itself)."""
    sl = shard_slices(tuple(tensor.shape), layout)
    if sl is None:
        return tensor
    return tensor[sl]


def shard_variable_init(distribution, variable, initializer):
    layout = variable._layout
    sl = shard_slices(tuple(variable._shape), layout)
    if sl is None:
        return None
    from keras_b200.core.tensor import convert_to_tensor

    full = convert_to_tensor(initializer(variable._shape, dtype=variable._dtype), dtype=variable._torch_dtype)
    variable._global_shape = tuple(variable._shape)
    variable._shard_slices = sl
    return full[sl].clone()


class _GatherShards(torch.autograd.Function):
    """Forward: all-gather along each sharded dim.  Backward: this rank's slice (model-axis peers see the same
    upstream gradient because they run the same replica of the batch)."""

    @staticmethod
    def forward(ctx, local, info, slices):
        ctx.slices = slices
        out = local
        for dim, parts, index, group in info:
            pieces = [torch.empty_like(out) for _ in range(parts)]
            dist.all_gather(pieces, out.contiguous(), group=group)
            out = torch.cat(pieces, dim=dim)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad[ctx.slices].contiguous(), None, None


def gather_variable(variable, local=None):
    """Full logical value of a sharded variable (autograd-aware)."""
    layout = variable._layout
    info = _axis_info(layout, layout.device_mesh.backend_mesh)
    local = variable._value if local is None else local
    if not info:
        return local
    return _GatherShards.apply(local, info, variable._shard_slices)


@contextlib.contextmanager
def local_shards():
    """Inside this scope ``Variable.value`` of a sharded variable is its local shard (optimizer updates)."""
    prev = global_state.get_global_attribute("tp_local_shards", False)
    global_state.set_global_attribute("tp_local_shards", True)
    try:
        yield
    finally:
        global_state.set_global_attribute("tp_local_shards", prev)


def in_local_shards():
    return bool(global_state.get_global_attribute("tp_local_shards", False))


def plan_for_model(distribution, model):
    """{variable path: layout axes} of every sharded variable of ``model`` (diagnostics and checkpoints)."""
    plan = {"kept_sharded": mark_pairs(model)} if hasattr(model, "_flatten_layers") else {}
    for v in model.variables:
        layout = getattr(v, "_layout", None)
        if layout is not None and any(a is not None for a in layout.axes):
            plan[v.path] = tuple(layout.axes)
    return plan


# ---------------------------------------------------------------------------- tensor-parallel layers
# A kernel sharded on a *free* dimension (one that survives into the output) makes the layer column-parallel: every rank
# computes its slice of the output from the full input.  A kernel sharded on a *contracted* dimension makes it
# row-parallel: every rank multiplies its slice of the input with its slice of the kernel and the partial products are
# summed over the model axis.  Outputs of column-parallel layers are all-gathered (correct for any consumer) unless
# the layer is marked ``_tp_keep_sharded`` — set by ``plan_for_model`` for layers whose outputs reach only
# row-parallel layers through elementwise layers, and by the attention layers for their head-sharded projections.
class _CopyToRegion(torch.autograd.Function):
    """Identity forward; backward sums the input gradient over the model axis (each rank holds a partial)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        dist.all_reduce(grad, group=ctx.group)
        return grad, None


class _ReduceFromRegion(torch.autograd.Function):
    """Sum over the model axis forward; identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _GatherDim(torch.autograd.Function):
    """All-gather along ``dim`` forward; backward keeps this rank's slice."""

    @staticmethod
    def forward(ctx, x, dim, group, index, parts):
        ctx.dim, ctx.index, ctx.parts = dim, index, parts
        pieces = [torch.empty_like(x) for _ in range(parts)]
        dist.all_gather(pieces, x.contiguous(), group=group)
        return torch.cat(pieces, dim=dim)

    @staticmethod
    def backward(ctx, grad):
        size = grad.shape[ctx.dim] // ctx.parts
        return grad.narrow(ctx.dim, ctx.index * size, size).contiguous(), None, None, None, None


class _ScatterDim(torch.autograd.Function):
    """Keep this rank's slice along ``dim`` forward; backward all-gathers the gradient slices."""

    @staticmethod
    def forward(ctx, x, dim, group, index, parts):
        ctx.dim, ctx.group, ctx.parts = dim, group, parts
        size = x.shape[dim] // parts
        return x.narrow(dim, index * size, size).contiguous()

    @staticmethod
    def backward(ctx, grad):
        pieces = [torch.empty_like(grad) for _ in range(ctx.parts)]
        dist.all_gather(pieces, grad.contiguous(), group=ctx.group)
        return torch.cat(pieces, dim=ctx.dim), None, None, None, None


def _single_shard(variable):
    """(dim, parts, index, group) when exactly one dimension of ``variable`` is sharded, else None."""
    if variable is None or getattr(variable, "_shard_slices", None) is None:
        return None
    info = _axis_info(variable._layout, variable._layout.device_mesh.backend_mesh)
    if len(info) != 1:
        return None
    return info[0]


def _local(variable, dtype):
    v = variable._value
    return v.to(dtype) if v.dtype != dtype else v


def dense(layer, inputs):
    """Tensor-parallel ``Dense``; returns ``None`` when the layout is not a plain column/row split."""
    shard = _single_shard(layer._kernel)
    if shard is None or layer.lora_enabled or getattr(layer, "_is_quantized", False) or not isinstance(inputs, torch.Tensor):
        return None
    dim, parts, index, group = shard
    w = _local(layer._kernel, inputs.dtype)
    bias = layer.bias
    sp, scope = _sp_state(), _call_scope()
    if dim == 1:  # column parallel
        b = None
        if bias is not None:
            b = _local(bias, inputs.dtype) if getattr(bias, "_shard_slices", None) is not None else bias.value.to(inputs.dtype).chunk(parts)[index]
        y = _fused_column(sp, scope, inputs, w, b)
        if y is None:
            if scope is not None and scope.is_shard(inputs):
                inputs = _GatherDim.apply(inputs, 0, group, index, parts)
            x = _CopyToRegion.apply(inputs, group)
            y = torch.matmul(x, w)
            if b is not None:
                y = y + b
        y = _activate(layer, y)
        if getattr(layer, "_tp_keep_sharded", False):
            return y
        return _GatherDim.apply(y, y.ndim - 1, group, index, parts)
    # row parallel
    k_local = w.shape[0]
    if inputs.shape[-1] == k_local * parts:
        x = _ScatterDim.apply(inputs, inputs.ndim - 1, group, index, parts)
    elif inputs.shape[-1] == k_local:
        x = inputs
    else:
        return None
    if scope is not None and scope.is_shard(x):
        # a row-parallel layer fed by a batch shard has no pairing column layer before it: work on the full batch
        x = _GatherDim.apply(x, 0, group, index, parts)
    y = _fused_row(sp, scope, x, w)
    sharded_out = y is not None
    if y is None:
        y = _ReduceFromRegion.apply(torch.matmul(x, w), group)
    if bias is not None:
        y = y + (bias.value.to(y.dtype) if getattr(bias, "_shard_slices", None) is None else gather_variable(bias).to(y.dtype))
        if sharded_out:
            sp.mark_partial(bias)
    y = _activate(layer, y)
    if sharded_out:
        scope.emitted.add(id(y))
    return y


def _activate(layer, y):
    from keras_b200 import activations

    act = layer.activation
    if act is not None and act is not activations.linear:
        y = act(y)
    return y


def einsum_dense(layer, inputs):
    """Tensor-parallel ``EinsumDense`` for kernels sharded on one dimension."""
    shard = _single_shard(layer._kernel)
    if shard is None or layer.lora_enabled or getattr(layer, "_is_quantized", False) or not isinstance(inputs, torch.Tensor):
        return None
    dim, parts, index, group = shard
    lhs, out_spec = layer.equation.replace(" ", "").split("->")
    in_spec, k_spec = lhs.split(",")
    if "." in layer.equation:
        return None
    letter = k_spec[dim]
    w = _local(layer._kernel, inputs.dtype)
    bias = layer.bias
    sp, scope = _sp_state(), _call_scope()
    plan = getattr(layer, "_gemm", None)
    if letter in out_spec:  # column-like: the sharded letter survives into the output
        odim = out_spec.index(letter)
        if plan is not None and scope is not None and scope.is_shard(inputs):
            nk = plan[0]
            kdim = 1
            for d in w.shape[:nk]:
                kdim *= d
            bflat = None
            if bias is not None and getattr(bias, "_shard_slices", None) is not None and tuple(bias._value.shape) == tuple(w.shape[nk:]):
                bflat = _local(bias, inputs.dtype).reshape(-1)
            if bias is None or bflat is not None:
                x2 = inputs.reshape(tuple(inputs.shape[: inputs.ndim - nk]) + (kdim,))
                y = _fused_column(sp, scope, x2, w.reshape(kdim, -1), bflat)
                if y is not None:
                    y = y.reshape(tuple(y.shape[:-1]) + tuple(w.shape[nk:]))
                    y = _activate(layer, y)
                    if getattr(layer, "_tp_keep_sharded", False):
                        return y
                    return _GatherDim.apply(y, odim, group, index, parts)
        if scope is not None and scope.is_shard(inputs):
            inputs = _GatherDim.apply(inputs, 0, group, index, parts)
        x = _CopyToRegion.apply(inputs, group)
        y = torch.einsum(layer.equation, x, w)
        if bias is not None:
            b = bias.value.to(y.dtype)
            if getattr(bias, "_shard_slices", None) is not None:
                b = _local(bias, y.dtype)
            elif layer.bias_axes and letter in layer.bias_axes:
                # bias dims follow the trailing output dims starting at the first bias axis
                first = min(out_spec.find(c) for c in layer.bias_axes)
                bdim = odim - first
                if 0 <= bdim < b.ndim and b.shape[bdim] == y.shape[odim] * parts:
                    b = b.chunk(parts, dim=bdim)[index]
            y = y + b
        y = _activate(layer, y)
        if getattr(layer, "_tp_keep_sharded", False):
            return y
        return _GatherDim.apply(y, odim, group, index, parts)
    # row-like: contraction over the sharded letter
    if letter not in in_spec:
        return None
    idim = in_spec.index(letter)
    local = w.shape[dim]
    if inputs.shape[idim] == local * parts:
        x = _ScatterDim.apply(inputs, idim, group, index, parts)
    elif inputs.shape[idim] == local:
        x = inputs
    else:
        return None
    if scope is not None and scope.is_shard(x):
        x = _GatherDim.apply(x, 0, group, index, parts)
    y = None
    if plan is not None and dim < plan[0]:
        nk = plan[0]
        kdim = 1
        for d in w.shape[:nk]:
            kdim *= d
        if x.shape[x.ndim - nk:] == w.shape[:nk]:
            x2 = x.reshape(tuple(x.shape[: x.ndim - nk]) + (kdim,))
            y = _fused_row(sp, scope, x2, w.reshape(kdim, -1))
            if y is not None:
                y = y.reshape(tuple(y.shape[:-1]) + tuple(w.shape[nk:]))
    sharded_out = y is not None
    if y is None:
        y = _ReduceFromRegion.apply(torch.einsum(layer.equation, x, w), group)
    if bias is not None:
        y = y + (bias.value.to(y.dtype) if getattr(bias, "_shard_slices", None) is None else gather_variable(bias).to(y.dtype))
        if sharded_out:
            sp.mark_partial(bias)
    y = _activate(layer, y)
    if sharded_out:
        scope.emitted.add(id(y))
    return y


def _is_row_parallel(layer):
    from keras_b200.layers.core.dense import Dense
    from keras_b200.layers.core.einsum_dense import EinsumDense

    k = getattr(layer, "_kernel", None)
    shard = _single_shard(k) if k is not None else None
    if shard is None:
        return False
    if isinstance(layer, Dense):
        return shard[0] == 0
    if isinstance(layer, EinsumDense):
        lhs, out_spec = layer.equation.replace(" ", "").split("->")
        return lhs.split(",")[1][shard[0]] not in out_spec
    return False


def _is_column_parallel(layer):
    from keras_b200.layers.core.dense import Dense
    from keras_b200.layers.core.einsum_dense import EinsumDense

    k = getattr(layer, "_kernel", None)
    shard = _single_shard(k) if k is not None else None
    if shard is None:
        return False
    if isinstance(layer, Dense):
        return shard[0] == 1
    if isinstance(layer, EinsumDense):
        lhs, out_spec = layer.equation.replace(" ", "").split("->")
        letter = lhs.split(",")[1][shard[0]]
        return letter in out_spec and out_spec.index(letter) == len(out_spec) - 1
    return False


def mark_pairs(model):
    """In a Functional model, let a column-parallel layer keep its output sharded when every path from it reaches a
    row-parallel layer through elementwise layers only (activation, dropout, multiply/add of equally sharded tensors)."""
    from keras_b200.layers.activations.activation_layers import Activation, ELU, LeakyReLU, ReLU
    from keras_b200.layers.merging.merging_layers import Add, Multiply, Subtract
    from keras_b200.layers.regularization.regularization_layers import Dropout
    from keras_b200.models.functional import Functional

    marked = []
    for m in [model] + [l for l in model._flatten_layers() if isinstance(l, Functional) and l is not model]:
        if not isinstance(m, Functional):
            continue
        nodes = m._ordered_nodes()
        consumers = {}
        producer = {}
        for n in nodes:
            for t in n.input_tensors:
                consumers.setdefault(id(t), []).append(n)
            for t in n.outputs:
                producer[id(t)] = n
        outputs = {id(t) for t in m._outputs}
        elementwise = (Activation, ReLU, LeakyReLU, ELU, Dropout)
        merges = (Multiply, Add, Subtract)

        def sharded_source(t, seen):
            """True when tensor ``t`` is (an elementwise function of) column-parallel outputs only."""
            n = producer.get(id(t))
            if n is None or id(n) in seen:
                return False
            seen.add(id(n))
            op = n.operation
            if _is_column_parallel(op):
                return True
            if isinstance(op, elementwise) or isinstance(op, merges):
                return all(sharded_source(i, seen) for i in n.input_tensors)
            return False

        def reaches_only_rows(t, seen):
            if id(t) in outputs:
                return False
            cons = consumers.get(id(t), [])
            if not cons:
                return False
            for c in cons:
                op = c.operation
                if _is_row_parallel(op):
                    rows.append(op)
                    continue
                if isinstance(op, elementwise):
                    if not reaches_only_rows(c.outputs[0], seen):
                        return False
                elif isinstance(op, merges):
                    if not all(sharded_source(i, set()) for i in c.input_tensors) or not reaches_only_rows(c.outputs[0], seen):
                        return False
                else:
                    return False
            return True

        for n in nodes:
            op = n.operation
            rows = []
            if _is_column_parallel(op) and len(op._inbound_nodes) == 1 and reaches_only_rows(n.outputs[0], set()):
                op._tp_keep_sharded = True
                for r in rows:
                    r._tp_local_input = True  # the layer's input-spec check sees the local width
                marked.append(op.path if hasattr(op, "path") else op.name)
    return marked


def mark_attention(layer, projections, output_dense):
    """Head-sharded attention: when every projection kernel is sharded on its heads dimension and the output kernel on
    the matching contracted heads dimension, the projections keep their outputs sharded (each rank attends over its
    own heads) and the output projection sums the partial results.  Returns (heads output dim, parts, index, group) or
    None when the layouts do not form that pattern."""
    cached = getattr(layer, "_tp_attention", False)
    if cached is not False:
        return cached
    result = None
    shards = [_single_shard(getattr(p, "_kernel", None)) for p in projections]
    out_shard = _single_shard(getattr(output_dense, "_kernel", None))
    if all(s is not None for s in shards) and out_shard is not None and _is_row_parallel(output_dense):
        dims = set()
        ok = True
        for p, sh in zip(projections, shards):
            lhs, out_spec = p.equation.replace(" ", "").split("->")
            letter = lhs.split(",")[1][sh[0]]
            # heads are the second-to-last output dimension of every projection
            if letter not in out_spec or out_spec.index(letter) != len(out_spec) - 2:
                ok = False
            dims.add(sh[1])
        if ok and len(dims) == 1 and out_shard[1] in dims:
            for p in projections:
                p._tp_keep_sharded = True
            output_dense._tp_local_input = True
            result = (-2, out_shard[1], out_shard[2], out_shard[3])
    layer._tp_attention = result
    return result


def gather_dim(x, dim, parts, index, group):
    return _GatherDim.apply(x, dim % x.ndim, group, index, parts)


# ------------------------------------------------------------------------ sequence-parallel execution of Functional graphs
# Between tensor-parallel blocks an activation is needed in full by nobody: it is the output of a row-parallel layer (a
# sum over the model axis) and feeds per-sample layers (normalisation, dropout, residual adds) until the next
# column-parallel layer.  So the row-parallel layer reduce-scatters its output over the batch dimension inside its GEMM
# (each rank keeps the samples [index*B/parts, (index+1)*B/parts)), the per-sample layers run on that shard, and the
# next column-parallel layer all-gathers the shard inside its GEMM (``fused_gemm``).  The Functional executor drives
# this: it wraps a batch shard in ``BatchShard``, unwraps it for layers that can work on a shard and gathers it for every
# other layer, so an unknown layer always sees the full tensor.
class BatchShard:
    """A tensor of which this rank holds the samples of its model-axis index (dimension 0)."""

    __slots__ = ("local",)

    def __init__(self, local):
        self.local = local


class _CallScope:
    """One executor-level layer call.  ``shard_batch``: leading extent of the batch shards handed to the layer (None when
    it received full tensors); a nested layer tells a shard from a full-batch tensor by that extent."""

    __slots__ = ("shard_batch", "emitted")

    def __init__(self, shard_batch):
        self.shard_batch = shard_batch
        self.emitted = set()

    def is_shard(self, x):
        return self.shard_batch is not None and x.ndim >= 1 and x.shape[0] == self.shard_batch


def _sp_state():
    return global_state.get_global_attribute("tp_sequence_parallel")


def _call_scope():
    sp = _sp_state()
    return sp.scope if sp is not None else None


class SequenceParallel:
    """Executor hook (``global_state`` attribute ``tp_sequence_parallel``) of one model-parallel group."""

    def __init__(self, parts, index, group, fused, emulate=False):
        self.parts, self.index, self.group, self.fused = parts, index, group, fused
        self.emulate = emulate  # no fused kernels (CPU): same data flow with library collectives around a plain matmul
        self.scope = None
        self.partial_variables = {}  # id -> variable whose gradient was computed from this rank's samples only

    # -- classification ----------------------------------------------------------------------------
    def _kind(self, op):
        from keras_b200.layers.activations.activation_layers import Activation, ELU, LeakyReLU, ReLU
        from keras_b200.layers.attention.attention_layers import GroupedQueryAttention, MultiHeadAttention
        from keras_b200.layers.core.dense import Dense
        from keras_b200.layers.core.einsum_dense import EinsumDense
        from keras_b200.layers.merging.merging_layers import Add, Multiply, Subtract
        from keras_b200.layers.normalization.normalization_layers import LayerNormalization, RMSNormalization
        from keras_b200.layers.regularization.regularization_layers import Dropout

        cached = getattr(op, "_tp_sp_kind", False)
        if cached is not False:
            return cached
        kind = None
        if isinstance(op, (Dense, EinsumDense)):
            if getattr(getattr(op, "_kernel", None), "_shard_slices", None) is not None and _single_shard(op._kernel) is not None:
                kind = "tp"
        elif isinstance(op, (MultiHeadAttention, GroupedQueryAttention)):
            q = getattr(op, "_query_dense", None)
            if q is not None and getattr(q._kernel, "_shard_slices", None) is not None:
                projections = [op._query_dense, op._key_dense, op._value_dense]
                gate = getattr(op, "_gate_dense", None)
                if gate is not None:
                    projections.append(gate)
                if mark_attention(op, projections, op._output_dense) is not None:
                    kind = "tp"
        elif isinstance(op, (LayerNormalization, RMSNormalization)):
            axis = op.axis if isinstance(op.axis, (list, tuple)) else [op.axis]
            if all(a != 0 for a in axis):
                kind = "per_sample"
        elif isinstance(op, (Dropout, Activation, ReLU, LeakyReLU, ELU, Add, Multiply, Subtract)):
            kind = "per_sample"
        if getattr(op, "built", True):
            try:
                op._tp_sp_kind = kind
            except Exception:
                pass
        return kind

    # -- executor entry points -----------------------------------------------------------------------
    def call(self, op, fn, args, kwargs):
        from keras_b200 import tree

        flat = tree.flatten((args, kwargs))
        shards = [a for a in flat if isinstance(a, BatchShard)]
        kind = self._kind(op)
        if shards and kind is None:
            args, kwargs = tree.map_structure(lambda a: self.gather(a) if isinstance(a, BatchShard) else a, (args, kwargs))
            shards = []
        if shards:
            full_batch = shards[0].local.shape[0] * self.parts

            def unwrap(a):
                if isinstance(a, BatchShard):
                    return a.local
                if isinstance(a, torch.Tensor) and a.ndim >= 1 and a.shape[0] == full_batch:
                    return _ScatterDim.apply(a, 0, self.group, self.index, self.parts)
                return a

            args, kwargs = tree.map_structure(unwrap, (args, kwargs))
            if kind == "per_sample":
                for v in getattr(op, "trainable_variables", ()):
                    self.partial_variables[id(v)] = v
        outer = self.scope
        scope = self.scope = _CallScope(shards[0].local.shape[0] if shards else None)
        try:
            result = fn(*args, **kwargs)
        finally:
            self.scope = outer
        per_sample = bool(shards) and kind == "per_sample"

        def wrap(r):
            if isinstance(r, torch.Tensor) and (per_sample or id(r) in scope.emitted):
                return BatchShard(r)
            return r

        return tree.map_structure(wrap, result)

    def gather(self, value):
        if isinstance(value, BatchShard):
            return _GatherDim.apply(value.local, 0, self.group, self.index, self.parts)
        return value

    finish = gather

    # -- used by the tensor-parallel layers -----------------------------------------------------------
    def fused_ok(self, rows, k, n, *tensors):
        from keras_b200.parallel import fused_gemm

        if rows % self.parts:
            return False
        if self.emulate:
            return True
        if self.fused is None:
            return False
        if not all(isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 for t in tensors):
            return False
        return fused_gemm.supported(rows // self.parts, k, n)

    def mark_partial(self, variable):
        if variable is not None:
            self.partial_variables[id(variable)] = variable

    def reduce_partial_gradients(self, trainable_weights):
        """Sum over the model axis the gradients that were computed from this rank's samples only (one packed all-reduce)."""
        if self.fused is not None:
            self.fused.drop_cache()
        todo = [v._value for v in trainable_weights if id(v) in self.partial_variables and v._value.grad is not None]
        if not todo:
            return
        flat = torch.cat([p.grad.reshape(-1).float() for p in todo])
        dist.all_reduce(flat, group=self.group)
        off = 0
        for p in todo:
            n = p.grad.numel()
            p.grad.copy_(flat[off:off + n].view(p.grad.shape))
            off += n


def enable_sequence_parallel(distribution, model):
    """Install the executor hook when the mesh has one sharded (model) axis of more than one rank on CUDA."""
    import os

    if os.environ.get("KERAS_B200_TP_FUSED", "1") == "0" or not process_groups.is_initialized():
        return None
    mesh = distribution.device_mesh
    groups = mesh.backend_mesh
    axes = [a for a in mesh.axis_names if a != distribution.batch_dim_name and groups.size(a) > 1]
    if len(axes) != 1:
        return None
    axis = axes[0]
    from keras_b200.core.tensor import get_device

    if get_device().type != "cuda":
        if os.environ.get("KERAS_B200_TP_SP_EMULATE") != "1":
            return None
        sp = SequenceParallel(groups.size(axis), groups.index(axis), groups.get_group(axis), None, emulate=True)
        global_state.set_global_attribute("tp_sequence_parallel", sp)
        return sp
    from keras_b200.kernels import loader

    if loader.get() is None:
        return None
    from keras_b200.parallel.fused_gemm import FusedGemmContext

    members = groups.members(axis)
    fused = FusedGemmContext(ranks=members, group=groups.get_group(axis))
    sp = SequenceParallel(groups.size(axis), groups.index(axis), groups.get_group(axis), fused)
    global_state.set_global_attribute("tp_sequence_parallel", sp)
    return sp


def disable_sequence_parallel():
    sp = _sp_state()
    if sp is not None:
        global_state.set_global_attribute("tp_sequence_parallel", None)
        if sp.fused is not None:
            sp.fused.close()


def _fused_column(sp, scope, x, w, bias):
    """Column-parallel product of a batch shard ``x`` [..., K]: all-gather -> GEMM.  None when the shapes do not qualify."""
    from keras_b200.parallel.fused_gemm import ColumnParallelLinear

    if sp is None or scope is None or not scope.is_shard(x):
        return None
    K, N = w.shape
    rows_local = x.numel() // K
    if not sp.fused_ok(rows_local * sp.parts, K, N, x, w):
        return None
    if sp.emulate:
        full = _CopyToRegion.apply(_GatherDim.apply(x, 0, sp.group, sp.index, sp.parts), sp.group)
        y = torch.matmul(full, w)
        return y if bias is None else y + bias
    x = x.contiguous()
    y = ColumnParallelLinear.apply(x.reshape(rows_local, K), w, bias, sp.fused)
    return y.reshape((x.shape[0] * sp.parts,) + tuple(x.shape[1:-1]) + (N,))


def _fused_row(sp, scope, x, w):
    """Row-parallel product reduce-scattered over the batch: GEMM -> reduce-scatter.  ``x``: [B, ..., K_local]."""
    from keras_b200.parallel.fused_gemm import RowParallelLinear

    if sp is None or scope is None or x.ndim < 2 or x.shape[0] % sp.parts:
        return None
    K, N = w.shape
    rows = x.numel() // K
    if not sp.fused_ok(rows, K, N, x, w):
        return None
    if sp.emulate:
        return _ScatterDim.apply(_ReduceFromRegion.apply(torch.matmul(x, w), sp.group), 0, sp.group, sp.index, sp.parts)
    x = x.contiguous()
    y = RowParallelLinear.apply(x.reshape(rows, K), w, sp.fused)
    return y.reshape((x.shape[0] // sp.parts,) + tuple(x.shape[1:-1]) + (N,))
