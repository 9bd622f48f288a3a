"""Calibrated weight-only quantisation of a whole model: ``model.quantize("gptq" | "awq", config=...)``.

The model is described by a *structure*: the layers that turn token ids into the first block's input
(``pre_block_layers``) and the blocks themselves in order (``sequential_blocks``); it comes from the config's
``quantization_layer_structure`` or from ``model.get_quantization_layer_structure(mode)``.  Calibration walks the blocks
once.  For each block it taps the inputs of every ``Dense`` / ``EinsumDense`` inside while the calibration activations
flow through, hands the collected statistics to the solver (``weight_only.gptq_solve`` or ``weight_only.awq_solve``),
stores the integer kernel in the layer, and only then computes the block's outputs, so the next block is calibrated on
what the quantised block actually produces (keras/src/quantizers/gptq_core.py:258-410, awq_core.py).
"""

import math
import re
from contextlib import contextmanager

import numpy as np
import torch

from keras_b200.quantizers import weight_only


# -------------------------------------------------------------------------------------- calibration data
def calibration_windows(tokenizer, sequence_length, dataset, num_samples=128, *, strategy="strided", seed=42, stride=None, eos_id=None):
    """``num_samples`` windows of ``sequence_length`` token ids cut from the dataset (strings are tokenised, arrays are
    taken as ids; a short dataset is repeated).  Returns ``int32 [num_samples, 1, sequence_length]``."""
    if not hasattr(dataset, "__iter__") or isinstance(dataset, (str, bytes)):
        raise TypeError("The `dataset` argument must be an iterable (e.g., a list of strings, a generator, or a NumPy array). Got type: "
                        f"{type(dataset).__name__}. Please pass the loaded dataset directly.")
    items = list(dataset)
    if not items:
        raise ValueError("Provided dataset is empty.")
    from keras_b200.core.tensor import convert_to_numpy

    pieces = []
    for position, item in enumerate(items):
        if isinstance(item, str):
            pieces.append(np.asarray(convert_to_numpy(tokenizer.tokenize(item))).reshape(-1).astype(np.int32))
            if eos_id is not None and position < len(items) - 1:
                pieces.append(np.array([eos_id], dtype=np.int32))  # windows should not read across documents unmarked
        else:
            pieces.append(np.asarray(convert_to_numpy(item)).reshape(-1).astype(np.int32))
    stream = np.concatenate(pieces) if len(pieces) > 1 else pieces[0]
    needed = num_samples * sequence_length
    if stream.size < needed:
        stream = np.tile(stream, math.ceil(needed / max(1, stream.size)))
    last_start = stream.size - sequence_length
    if last_start < 0:
        raise ValueError(f"Not enough tokens to form one sample of length {sequence_length} (have {stream.size}).")
    if strategy == "random":
        starts = np.random.default_rng(seed).integers(0, last_start + 1, size=num_samples, dtype=np.int64)
    elif strategy == "linspace":
        starts = np.linspace(0, last_start, num_samples, dtype=np.int64)
    elif strategy == "strided":
        step = stride if stride is not None else max(1, (last_start + 1) // num_samples)
        offset = abs(hash(("gptq-calib", seed))) % (last_start + 1) if last_start > 0 else 0
        starts = (offset + np.arange(num_samples, dtype=np.int64) * step) % (last_start + 1)
    else:
        raise ValueError(f"Unknown strategy: {strategy}")
    windows = np.lib.stride_tricks.sliding_window_view(stream, sequence_length)[starts]
    return windows.astype(np.int32)[:, None, :]


# ------------------------------------------------------------------------------------------- layer picking
def passes_filters(layer, filters):
    """``filters``: None (everything), a regular expression or a list of them searched in the layer's name, or a callable."""
    if filters is None:
        return True
    if isinstance(filters, str):
        return bool(re.search(filters, layer.name))
    if isinstance(filters, (list, tuple)):
        return any(re.search(pattern, layer.name) for pattern in filters)
    return bool(filters(layer))


def projection_layers(block, filters=None):
    """{path: layer} of the ``Dense`` / ``EinsumDense`` layers inside ``block`` that pass the filters."""
    from keras_b200.layers.core.dense import Dense
    from keras_b200.layers.core.einsum_dense import EinsumDense

    return {layer.path: layer for layer in block._flatten_layers() if isinstance(layer, (Dense, EinsumDense)) and passes_filters(layer, filters)}


def _matrix_view(layer):
    """The layer's float kernel as ``[in, out]`` and that shape."""
    from keras_b200.layers.core.einsum_dense import EinsumDense

    kernel = layer._kernel.value.detach()
    rows, columns = EinsumDense.calibrated_matrix_shape(kernel.shape) if kernel.ndim != 2 else tuple(kernel.shape)
    return kernel.reshape(rows, columns), rows, columns


# ------------------------------------------------------------------------------------------ per-layer jobs
class _GPTQJob:
    def __init__(self, layer, config):
        self.layer, self.config = layer, config
        _, self.rows, _ = _matrix_view(layer)
        self.statistic = weight_only.HessianEstimate(self.rows)

    def observe(self, x2d):
        self.statistic.add(x2d)

    def finish(self):
        matrix, _, _ = _matrix_view(self.layer)
        c = self.config
        codes, scale, zero, g_idx = weight_only.gptq_solve(
            matrix.T, self.statistic.damped(c.hessian_damping), bits=c.weight_bits, group_size=c.group_size, symmetric=c.symmetric,
            per_channel=c.per_channel, activation_order=c.activation_order)
        self.layer._store_calibrated("gptq", codes, scale, zero, g_idx)


class _AWQJob:
    def __init__(self, layer, config):
        self.layer, self.config = layer, config
        _, self.rows, _ = _matrix_view(layer)
        self.statistic = weight_only.ActivationProfile(self.rows, keep_sample=bool(getattr(config, "apply_clip", False)))

    def observe(self, x2d):
        self.statistic.add(x2d)

    def finish(self):
        matrix, _, _ = _matrix_view(self.layer)
        c = self.config
        codes, scale, zero, channel_scales, g_idx = weight_only.awq_solve(
            matrix.T, self.statistic.magnitudes, num_grid_points=c.num_grid_points, group_size=c.group_size,
            activation_sample=self.statistic.sample if getattr(c, "apply_clip", False) else None)
        self.layer._store_calibrated("awq", codes, scale, zero, g_idx, awq_scales=channel_scales)


_JOBS = {"gptq": _GPTQJob, "awq": _AWQJob}


@contextmanager
def tapped(jobs):
    """While active, every job's layer reports the (flattened) input of each call to its job."""
    originals = {}

    def tap(job, call):
        def observed(*args, **kwargs):
            x = args[0] if args else kwargs["inputs"]
            job.observe(x.detach().reshape(-1, job.rows))
            return call(*args, **kwargs)

        return observed

    try:
        for path, job in jobs.items():
            originals[path] = job.layer.call
            job.layer.call = tap(job, job.layer.call)
        yield
    finally:
        for path, job in jobs.items():
            job.layer.call = originals[path]


# ------------------------------------------------------------------------------------------------ driver
def _as_batch(samples):
    samples = [s.unsqueeze(0) if s.ndim == 2 else s for s in samples]
    return samples[0] if len(samples) == 1 else torch.cat(samples, dim=0)


def calibrate_blocks(windows, mode, config, structure, filters=None):
    from keras_b200.core.tensor import convert_to_tensor
    from keras_b200.utils.progbar import Progbar

    blocks = structure.get("sequential_blocks", [])
    if not blocks:
        raise ValueError("No sequential blocks found in the provided structure to quantize.")
    activations = []
    with torch.no_grad():
        for window in windows:
            x = convert_to_tensor(window, dtype="int32")
            for layer in structure.get("pre_block_layers", []):
                x = layer(x)
            activations.append(x)
        activations = activations[: min(config.num_samples, len(activations))]
        per_pass = max(1, int(getattr(config, "calibration_batch_size", 1) or 1))
        bar = Progbar(target=len(blocks))
        for index, block in enumerate(blocks):
            jobs = {path: _JOBS[mode](layer, config) for path, layer in projection_layers(block, filters).items()
                    if getattr(layer, "_kernel", None) is not None and layer.quantization_mode == mode}
            if jobs:
                with tapped(jobs):
                    for start in range(0, len(activations), per_pass):
                        block(_as_batch(activations[start:start + per_pass]))
                for job in jobs.values():
                    job.finish()
            if index < len(blocks) - 1:
                produced = []
                for start in range(0, len(activations), per_pass):
                    chunk = activations[start:start + per_pass]
                    out = block(_as_batch(chunk))
                    out = out[0] if isinstance(out, (list, tuple)) else out
                    produced.extend(out[i] for i in range(len(chunk)))
                activations = produced
            bar.update(index + 1)


def calibrated_quantize(model, mode, config, filters=None):
    """Entry point of ``Model.quantize`` for the calibrated modes."""
    if config.dataset is None or config.tokenizer is None:
        raise ValueError(f"{mode.upper()} quantization requires a dataset and a tokenizer. Please provide them in the `{type(config).__name__}`.")
    structure = config.quantization_layer_structure
    if structure is None and hasattr(model, "get_quantization_layer_structure"):
        structure = model.get_quantization_layer_structure(mode)
    if structure is None:
        raise ValueError(f"For '{mode}' mode, a valid quantization structure must be provided either via `config.quantization_layer_structure` or "
                         "by overriding `model.get_quantization_layer_structure(mode)`. The structure should be a dictionary with keys "
                         "'pre_block_layers' and 'sequential_blocks'.")
    # every projection inside the blocks gets its integer state (and keeps computing with its float kernel for now)
    for block in structure.get("sequential_blocks", []):
        for layer in projection_layers(block, filters).values():
            if not getattr(layer, "_is_quantized", False):
                layer.quantize(mode, config=config)
    windows = calibration_windows(config.tokenizer, config.sequence_length, config.dataset, num_samples=config.num_samples)
    calibrate_blocks(windows[: config.num_samples], mode, config, structure, filters=filters)
