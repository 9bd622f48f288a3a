"""``Model.summary()``: a box-drawn table of layers, output shapes and parameter counts followed by totals
(keras/src/utils/summary_utils.py:122-390; the reference renders through ``rich``, this renders plain text
with the same columns and totals)."""

import math
import re
import shutil

import numpy as np

from keras_b200 import tree
from keras_b200.utils import io_utils


def count_params(weights):
    shapes = [tuple(v.shape) for v in weights]
    return int(sum(math.prod(p) for p in shapes))


def _dtype_bytes(dtype):
    name = str(dtype)
    m = re.search(r"(\d+)", name)
    if "bool" in name:
        return 1
    return int(m.group(1)) // 8 if m else 4


def weight_memory_size(weights):
    """Total bytes of the unique variables in ``weights``."""
    seen, total = set(), 0
    for w in weights:
        if id(w) in seen:
            continue
        seen.add(id(w))
        total += math.prod(tuple(w.shape)) * _dtype_bytes(w.dtype)
    return total


def readable_memory_size(weight_memory_size):
    units = ["B", "KB", "MB", "GB", "TB", "PB"]
    scale = 1024
    for unit in units:
        if weight_memory_size / scale < 1:
            return f"{weight_memory_size:.2f} {unit}"
        weight_memory_size /= scale
    return f"{weight_memory_size:.2f} {units[-1]}"


def format_layer_shape(layer):
    if not layer._inbound_nodes and not getattr(layer, "_build_shapes_dict", None):
        return "?"

    def fmt(shape):
        return "(" + ", ".join("None" if d is None else str(d) for d in shape) + ")"

    if len(layer._inbound_nodes) > 0:
        for i in range(len(layer._inbound_nodes)):
            outputs = layer._inbound_nodes[i].output_tensors
            shapes = tree.map_structure(lambda x: fmt(x.shape), outputs)
    else:
        try:
            if hasattr(layer, "output_shape"):
                shapes = fmt(layer.output_shape)
            else:
                outputs = layer.compute_output_shape(**layer._build_shapes_dict)
                shapes = tree.map_shape_structure(lambda x: fmt(x), outputs)
        except NotImplementedError:
            return "?"
    if len(shapes) == 1 and not isinstance(shapes, str):
        return shapes[0]
    out = str(shapes)
    return out.replace("'", "")


def get_layer_index_bound_by_layer_name(layers, layer_range=None):
    if layer_range is not None:
        if len(layer_range) != 2:
            raise ValueError(f"layer_range must be a list or tuple of length 2. Received: layer_range = {layer_range} of length {len(layer_range)}")
        if not isinstance(layer_range[0], str) or not isinstance(layer_range[1], str):
            raise ValueError(f"layer_range should contain string type only. Received: {layer_range}")
    else:
        return [0, len(layers)]
    lower = [idx for idx, layer in enumerate(layers) if re.match(layer_range[0], layer.name)]
    upper = [idx for idx, layer in enumerate(layers) if re.match(layer_range[1], layer.name)]
    if not lower or not upper:
        raise ValueError(f"Passed layer_names do not match the layer names in the model. Received: {layer_range}")
    if min(lower) > max(upper):
        return [min(upper), max(lower) + 1]
    return [min(lower), max(upper) + 1]


def _wrap(text, width):
    text = str(text)
    if width <= 0:
        return [text]
    out = []
    while len(text) > width:
        cut = text.rfind(" ", 0, width + 1)
        cut = width if cut <= 0 else cut
        out.append(text[:cut])
        text = text[cut:].lstrip()
    out.append(text)
    return out


def print_summary(model, line_length=None, positions=None, print_fn=None, expand_nested=False, show_trainable=False, layer_range=None):
    from keras_b200.models import Functional, Sequential

    if not print_fn and not io_utils.is_interactive_logging_enabled():
        print_fn = io_utils.print_msg
    if isinstance(model, Sequential):
        sequential_like = True
        layers = model.layers
    elif not isinstance(model, Functional):
        sequential_like = True
        layers = model.layers
    else:
        layers = model._operations
        sequential_like = True
        nodes_by_depth = model._nodes_by_depth.values()
        nodes = []
        for v in nodes_by_depth:
            if (len(v) > 1) or (len(v) == 1 and len(tree.flatten(v[0].input_tensors)) > 1):
                sequential_like = False
                break
            nodes += v
        if sequential_like:
            for layer in model.layers:
                flag = False
                for node in layer._inbound_nodes:
                    if node in nodes:
                        if flag:
                            sequential_like = False
                            break
                        flag = True
                if not sequential_like:
                    break
    if sequential_like:
        default_line_length = 88
        positions = positions or [0.45, 0.80, 1.0]
        header = ["Layer (type)", "Output Shape", "Param #"]
        alignment = ["<", "<", ">"]
    else:
        default_line_length = 108
        positions = positions or [0.3, 0.56, 0.74, 1.0]
        header = ["Layer (type)", "Output Shape", "Param #", "Connected to"]
        alignment = ["<", "<", ">", "<"]
        relevant_nodes = []
        for v in model._nodes_by_depth.values():
            relevant_nodes += v
    if show_trainable:
        default_line_length += 12
        positions = [p * 0.90 for p in positions] + [1.0]
        header.append("Trainable")
        alignment.append("^")
    if line_length is None:
        line_length = min(default_line_length, shutil.get_terminal_size().columns - 4)
    line_length = max(line_length, 40)
    if positions[-1] <= 1:
        positions = [int(line_length * p) for p in positions]
    widths = []
    prev = 0
    for p, h in zip(positions, header):
        widths.append(max(p - prev - 3, len(h)))
        prev = p

    def get_connections(layer):
        connections = ""
        for node in layer._inbound_nodes:
            if relevant_nodes and node not in relevant_nodes:
                continue
            for kt in node.input_tensors:
                keras_history = kt._keras_history
                inbound_layer = keras_history.operation
                node_index = node._keras_history_index if False else keras_history.node_index
                tensor_index = keras_history.tensor_index
                if connections:
                    connections += ", "
                connections += f"{inbound_layer.name}[{node_index}][{tensor_index}]"
        if not connections:
            connections = "-"
        return connections

    def get_layer_fields(layer, prefix=""):
        output_shape = format_layer_shape(layer)
        name = prefix + layer.name
        cls_name = layer.__class__.__name__
        name = f"{name} ({cls_name})"
        if not hasattr(layer, "built"):
            params = "0"
        elif not layer.built:
            params = "0 (unbuilt)"
        else:
            params = f"{layer.count_params():,}"
        fields = [name, output_shape, params]
        if not sequential_like:
            fields.append(get_connections(layer))
        if show_trainable:
            if hasattr(layer, "weights") and len(layer.weights) > 0:
                fields.append("Y" if layer.trainable else "N")
            else:
                fields.append("-")
        return fields

    rows = []

    def add_layer(layer, nested_level=0):
        prefix = "   " * nested_level + ("└ " if nested_level else "")
        rows.append(get_layer_fields(layer, prefix=prefix))
        if expand_nested and hasattr(layer, "layers") and layer.layers:
            for nested in layer.layers:
                add_layer(nested, nested_level + 1)

    layer_range = get_layer_index_bound_by_layer_name(layers, layer_range)
    for layer in layers[layer_range[0]: layer_range[1]]:
        add_layer(layer)

    lines = []

    def rule(left, mid, right, fill):
        return left + mid.join(fill * (w + 2) for w in widths) + right

    def render(fields, bold=False):
        cells = [_wrap(f, w) for f, w in zip(fields, widths)]
        height = max(len(c) for c in cells)
        for i in range(height):
            parts = []
            for c, w, a in zip(cells, widths, alignment):
                text = c[i] if i < len(c) else ""
                parts.append(" " + format(text, f"{a}{w}") + " ")
            lines.append("│" + "│".join(parts) + "│")

    title = f'Model: "{model.name}"'
    lines.append(title)
    lines.append(rule("┏", "┳", "┓", "━"))
    cells = [format(h, f"{a}{w}") for h, w, a in zip(header, widths, alignment)]
    lines.append("┃" + "┃".join(" " + c + " " for c in cells) + "┃")
    lines.append(rule("┡", "╇", "┩", "━"))
    for i, r in enumerate(rows):
        render(r)
        if i != len(rows) - 1:
            lines.append(rule("├", "┼", "┤", "─"))
    lines.append(rule("└", "┴", "┘", "─"))

    if hasattr(model, "_collected_trainable_weights"):
        trainable_count = count_params(model._collected_trainable_weights)
        trainable_memory_size = weight_memory_size(model._collected_trainable_weights)
    else:
        trainable_count = count_params(model.trainable_weights)
        trainable_memory_size = weight_memory_size(model.trainable_weights)
    non_trainable_count = count_params(model.non_trainable_weights)
    non_trainable_memory_size = weight_memory_size(model.non_trainable_weights)
    if getattr(model, "compiled", False) and model.optimizer and model.optimizer.built:
        optimizer_weight_count = count_params(model.optimizer.variables)
        optimizer_memory_size = weight_memory_size(model.optimizer.variables)
        optimizer_built = True
    else:
        optimizer_weight_count = optimizer_memory_size = 0
        optimizer_built = False
    total_count = trainable_count + non_trainable_count + optimizer_weight_count
    total_memory_size = trainable_memory_size + non_trainable_memory_size + optimizer_memory_size
    lines.append(f" Total params: {total_count:,} ({readable_memory_size(total_memory_size)})")
    lines.append(f" Trainable params: {trainable_count:,} ({readable_memory_size(trainable_memory_size)})")
    lines.append(f" Non-trainable params: {non_trainable_count:,} ({readable_memory_size(non_trainable_memory_size)})")
    if optimizer_built:
        lines.append(f" Optimizer params: {optimizer_weight_count:,} ({readable_memory_size(optimizer_memory_size)})")
    text = "\n".join(lines)
    if print_fn:
        print_fn(text)
    else:
        io_utils.print_msg(text)


def print_quantization_summary(model, verbose=True):
    """Bytes before/after quantization per layer; returns ``(total_before, total_after)``."""
    from keras_b200.quantizers import QuantizationReport

    report = QuantizationReport.from_model(model)
    if verbose:
        io_utils.print_msg(str(report))
    return report
