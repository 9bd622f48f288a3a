"""``Function``: a DAG of operations between symbolic inputs and outputs.

Graph discovery and ordering rules follow keras/src/ops/function.py:260-486 (operation order
= decreasing depth, ties by first depth-first visit; it decides ``model.layers`` order and
with it the group names inside weight files).  Execution differs: the graph is compiled once
into a flat list of steps with pre-resolved tensor slots, so a forward pass is a single loop
without dictionary-of-depth lookups or structure packing.
"""

import collections

from keras_b200 import tree
from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.ops.operation import Operation


def torch_relu(x):
    import torch

    return torch.relu(x)


@keras_export("keras.Function")
class Function(Operation):
    def __init__(self, inputs, outputs, name=None):
        Operation.__init__(self, name=name)
        if isinstance(inputs, dict):
            for k, v in inputs.items():
                if isinstance(v, KerasTensor) and k != v.name:
                    pass  # names may differ; the dict keys win at call time
        self._inputs_struct = tree.map_structure(lambda x: x, inputs)
        self._outputs_struct = tree.map_structure(lambda x: x, outputs)
        self._inputs = tree.flatten(inputs)
        self._outputs = tree.flatten(outputs)
        if not self._inputs:
            raise ValueError("`inputs` argument cannot be empty. Received:\n" f"inputs={inputs}\noutputs={outputs}")
        if not self._outputs:
            raise ValueError("`outputs` argument cannot be empty. Received:\n" f"inputs={inputs}\noutputs={outputs}")
        for x in self._inputs + self._outputs:
            if not isinstance(x, KerasTensor):
                raise ValueError(
                    "All `inputs` and `outputs` values must be KerasTensors. Received: "
                    f"inputs={inputs}, outputs={outputs} including invalid value {x} of type {type(x)}"
                )
        if len({id(x) for x in self._inputs}) != len(self._inputs):
            raise ValueError(f"The list of inputs passed to the model contains the same input multiple times: {inputs}")
        nodes, nodes_by_depth, operations, operations_by_depth = map_graph(self._inputs, self._outputs)
        self._nodes = nodes
        self._nodes_by_depth = nodes_by_depth
        self._operations = operations
        self._operations_by_depth = operations_by_depth
        self._node_order = None
        self._fusion_plan = None
        for inp in self._inputs:
            if inp._keras_history.operation and not inp._keras_history.operation._outbound_nodes:
                raise ValueError("`inputs` not connected to `outputs`")

    operations = property(lambda self: self._operations[:])
    inputs = property(lambda self: self._inputs)
    outputs = property(lambda self: self._outputs)

    def _ordered_nodes(self):
        out = []
        for depth in sorted(self._nodes_by_depth, reverse=True):
            for node in self._nodes_by_depth[depth]:
                if node.operation is None or node.is_input:
                    continue
                out.append(node)
        return out

    def compute_output_spec(self, inputs):
        self._assert_input_compatibility(inputs)
        same = all(
            tuple(x.shape) == tuple(r.shape) for x, r in zip(tree.flatten(inputs), self._inputs)
        )
        if same:
            return tree.map_structure(lambda x: KerasTensor(x.shape, dtype=x.dtype), self._outputs_struct)
        return self._run_through_graph(inputs, operation_fn=lambda op: op.compute_output_spec)

    def compute_output_shape(self, input_shape):
        spec_in = tree.map_shape_structure(lambda s: KerasTensor(s), input_shape)
        for x, ref in zip(tree.flatten(spec_in), self._inputs):
            x._dtype = ref.dtype
        return tree.map_structure(lambda x: x.shape, self.compute_output_spec(spec_in))

    def call(self, inputs):
        self._assert_input_compatibility(inputs)
        return self._run_through_graph(inputs)

    def _run_through_graph(self, inputs, operation_fn=None, call_fn=None, fusion=None):
        flat_in = tree.flatten(inputs)
        env = {id(ref): val for ref, val in zip(self._inputs, flat_in)}
        nodes = self._node_order
        if nodes is None:
            nodes = self._node_order = self._ordered_nodes()
        if fusion is not None and flat_in and fusion.applicable(flat_in[0]):
            return self._run_fused(env, nodes, operation_fn, fusion)
        sp = global_state.get_global_attribute("tp_sequence_parallel") if call_fn is None else None
        for node in nodes:
            if any(id(t) not in env for t in node.input_tensors):
                continue
            args, kwargs = node.arguments.fill_in(env)
            op = node.operation if operation_fn is None else operation_fn(node.operation)
            if call_fn is not None:
                result = call_fn(op, *args, **kwargs)
            elif sp is not None:
                result = sp.call(node.operation, op, args, kwargs)
            else:
                result = op(*args, **kwargs)
            outs = node.outputs
            if len(outs) == 1 and not isinstance(result, (list, tuple, dict)):
                env[id(outs[0])] = result
            else:
                for ref, val in zip(outs, tree.flatten(result)):
                    env[id(ref)] = val
        flat_out = []
        for i, ref in enumerate(self._outputs):
            if id(ref) not in env:
                path = tree.flatten_with_path(self._outputs_struct)[i][0]
                raise ValueError(f"Output with path `{'.'.join(map(str, path))}` is not connected to `inputs`")
            flat_out.append(env[id(ref)] if sp is None else sp.finish(env[id(ref)]))
        return tree.pack_sequence_as(self._outputs_struct, flat_out)

    def _run_fused(self, env, nodes, operation_fn, fusion):
        """Executor used on CUDA: like the plain loop, with the fusion plan's deferred BN nodes."""
        plan = self._fusion_plan
        if plan is None:
            plan = self._fusion_plan = fusion.build_plan(self)
        training = fusion.training
        sp = global_state.get_global_attribute("tp_sequence_parallel")
        merge = plan.get("merge_tensors", ())
        marked = set()
        if merge:
            import torch

            from keras_b200.kernels import grad_merge
        for node in nodes:
            ins = node.input_tensors
            if any(id(t) not in env for t in ins):
                continue
            if merge:
                # an activation with two gradient-sharing consumers gets its slot as soon as it exists as a tensor
                for t in ins:
                    if id(t) in merge and id(t) not in marked:
                        marked.add(id(t))
                        if isinstance(env[id(t)], torch.Tensor):
                            grad_merge.mark(env[id(t)])
            role = plan.get(id(node))
            outs = node.outputs
            if role == "pad_fold":
                x = env[id(ins[0])]
                if isinstance(x, fusion.Deferred):
                    x = fusion.run_bn(x.layer, x.x, training, pre_bias=x.pre_bias, stats=x.stats)
                env[id(outs[0])] = fusion.Padded(x, node.operation.padding)
                continue
            if role == "pool_padded":
                x = env[id(ins[0])]
                env[id(outs[0])] = fusion.run_pool_padded(node.operation, x.x, x.pairs)
                continue
            if role == "conv_fold_bias":
                x = env[id(ins[0])]
                pairs = None
                if isinstance(x, fusion.Padded):
                    x, pairs = x.x, x.pairs
                elif isinstance(x, fusion.Deferred):
                    x = fusion.run_bn(x.layer, x.x, training, pre_bias=x.pre_bias, stats=x.stats)
                y, stats = fusion.run_conv_nobias(node.operation, x, pairs, want_stats=bool(training))
                env[id(outs[0])] = fusion.NoBias(y, node.operation.bias if node.operation.use_bias else None, stats)
                continue
            if role == "defer_bn":
                x = env[id(ins[0])]
                pre_bias = stats = None
                if isinstance(x, fusion.NoBias):
                    x, pre_bias, stats = x.x, x.bias, x.stats
                elif isinstance(x, fusion.Deferred):
                    x = fusion.run_bn(x.layer, x.x, training, pre_bias=x.pre_bias, stats=x.stats)
                env[id(outs[0])] = fusion.Deferred(node.operation, x, pre_bias, stats)
                continue
            if role == "consume_relu":
                d = env[id(ins[0])]
                env[id(outs[0])] = fusion.run_bn(d.layer, d.x, training, relu=True, pre_bias=d.pre_bias, stats=d.stats) if isinstance(d, fusion.Deferred) else node.operation(d)
                continue
            if role in ("consume_add", "consume_add_relu"):
                a, b = env[id(ins[0])], env[id(ins[1])]
                if isinstance(a, fusion.Deferred) and isinstance(b, fusion.Deferred):
                    b = fusion.run_bn(b.layer, b.x, training, pre_bias=b.pre_bias, stats=b.stats)
                if isinstance(b, fusion.Deferred):
                    a, b = b, a
                if isinstance(a, fusion.Deferred):
                    env[id(outs[0])] = fusion.run_bn(a.layer, a.x, training, residual=b, relu=role == "consume_add_relu", pre_bias=a.pre_bias, stats=a.stats)
                else:
                    r = node.operation([a, b])
                    env[id(outs[0])] = torch_relu(r) if role == "consume_add_relu" else r
                continue
            if role == "identity":
                env[id(outs[0])] = env[id(ins[0])]
                continue
            args, kwargs = node.arguments.fill_in(env)
            op = node.operation if operation_fn is None else operation_fn(node.operation)
            result = op(*args, **kwargs) if sp is None else sp.call(node.operation, op, args, kwargs)
            if len(outs) == 1 and not isinstance(result, (list, tuple, dict)):
                env[id(outs[0])] = result
            else:
                for ref, val in zip(outs, tree.flatten(result)):
                    env[id(ref)] = val
        flat_out = []
        for ref in self._outputs:
            v = env[id(ref)]
            if isinstance(v, fusion.Deferred):
                v = fusion.run_bn(v.layer, v.x, training, pre_bias=v.pre_bias, stats=v.stats)
            flat_out.append(v if sp is None else sp.finish(v))
        return tree.pack_sequence_as(self._outputs_struct, flat_out)

    def _assert_input_compatibility(self, inputs):
        try:
            tree.assert_same_structure(inputs, self._inputs_struct, check_types=False)
        except ValueError:
            raise ValueError(
                "Function was called with an invalid input structure. "
                f"Expected input structure: {self._inputs_struct}\nReceived input structure: {inputs}"
            )
        for x, ref in zip(tree.flatten(inputs), self._inputs):
            ok = len(x.shape) == len(ref.shape) and all(
                a is None or b is None or a == b for a, b in zip(x.shape, ref.shape)
            )
            if not ok:
                raise ValueError(
                    f"{self.__class__.__name__} was passed incompatible inputs. For input "
                    f"'{ref.name}', expected shape {ref.shape}, but received instead a tensor "
                    f"with shape {tuple(x.shape)}."
                )


def make_node_key(op, node_index):
    return f"{id(op)}_ib-{node_index}"


def map_graph(inputs, outputs):
    """Discover the sub-graph between ``inputs`` and ``outputs``.

    Returns ``(node_keys, nodes_by_depth, operations, operations_by_depth)``.
    """
    input_ids = {id(t) for t in inputs}
    order = []           # nodes, producers before consumers
    first_seen = {}      # operation -> visit rank
    done, active = set(), set()

    def visit(tensor):
        # Iterative DFS would be safer for very deep nets; recursion depth here equals the
        # graph depth, which Python handles for thousands of layers once the limit is raised.
        op, node_index, _ = tensor._keras_history
        if not op:
            return
        node = op._inbound_nodes[node_index]
        if node in done:
            return
        if not node.is_input and id(tensor) in input_ids:
            done.add(node)
            return
        if node in active:
            raise ValueError(f"Tensor {tensor} from operation '{op.name}' is part of a cycle.")
        if op not in first_seen:
            first_seen[op] = len(first_seen)
        active.add(node)
        if not node.is_input:
            for t in node.input_tensors:
                visit(t)
        active.discard(node)
        done.add(node)
        order.append(node)

    import sys

    limit = sys.getrecursionlimit()
    if limit < 20000:
        sys.setrecursionlimit(20000)
    try:
        for t in outputs:
            visit(t)
    finally:
        sys.setrecursionlimit(limit)

    in_graph = set(order)
    node_depth, op_depth = {}, {}
    for node in reversed(order):
        d = max(node_depth.setdefault(node, 0), op_depth.get(node.operation, 0))
        op_depth[node.operation] = d
        node_depth[node] = d
        for parent in node.parent_nodes:
            if parent in in_graph:
                node_depth[parent] = max(d + 1, node_depth.get(parent, 0))
    keys = {make_node_key(n.operation, n.operation._inbound_nodes.index(n)) for n in order}
    for t in inputs:
        op = t._keras_history.operation
        if op and op not in op_depth:
            idx = t._keras_history.node_index
            node = op._inbound_nodes[idx]
            if node.is_input:
                op_depth[op] = 0
                first_seen[op] = -1
                node_depth[node] = 0
                keys.add(make_node_key(op, idx))

    nodes_by_depth = collections.defaultdict(list)
    for node, d in node_depth.items():
        nodes_by_depth[d].append(node)
    ops_by_depth = collections.defaultdict(list)
    for op, d in op_depth.items():
        ops_by_depth[d].append(op)
    operations = []
    for d in sorted(ops_by_depth, reverse=True):
        ops_by_depth[d].sort(key=lambda o: first_seen[o])
        operations.extend(ops_by_depth[d])

    available = {id(t) for t in inputs}
    visited_names = []
    for d in sorted(nodes_by_depth, reverse=True):
        for node in nodes_by_depth[d]:
            for t in node.input_tensors:
                if id(t) not in available:
                    raise ValueError(
                        f"Graph disconnected: cannot find parent for tensor {t} at operation "
                        f"'{node.operation}'. The following previous operations were accessed "
                        f"without issue: {visited_names}"
                    )
            visited_names.append(node.operation.name)
            for t in node.outputs:
                available.add(id(t))
    counts = collections.Counter(op.name for op in operations)
    for name, c in counts.items():
        if c != 1:
            raise ValueError(f'The name "{name}" is used {c} times in the model. All operation names should be unique.')
    return keys, nodes_by_depth, operations, ops_by_depth


def nodes_between(inputs, outputs):
    """Nodes on any path from ``inputs`` to ``outputs``, producers first."""
    start = {id(t) for t in tree.flatten(inputs)}
    order, seen = [], set()

    def visit(tensor):
        if id(tensor) in start:
            return
        op, node_index, _ = tensor._keras_history
        if op is None:
            return
        node = op._inbound_nodes[node_index]
        if node in seen:
            return
        seen.add(node)
        for t in node.input_tensors:
            visit(t)
        order.append(node)

    for t in tree.flatten(outputs):
        visit(t)
    return order
