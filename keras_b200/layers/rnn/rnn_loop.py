"""Time loop shared by the recurrent layers (counterpart of ``backend.rnn``, keras/src/backend/torch/rnn.py:14-372)."""

import torch

from keras_b200 import tree
from keras_b200.core.tensor import convert_to_tensor


def _expand_mask(mask_t, like):
    while mask_t.ndim < like.ndim:
        mask_t = mask_t.unsqueeze(-1)
    return mask_t


def rnn(step_function, inputs, initial_states, go_backwards=False, mask=None, constants=None, unroll=False, input_length=None, time_major=False,
        zero_output_for_mask=False, return_all_outputs=True):
    """Iterate ``step_function(inputs_t, states + constants) -> (output_t, new_states)`` over time.

    Returns ``(last_output, outputs, new_states)``; ``outputs`` is ``[batch, time, ...]`` (or ``[batch, 1, ...]``
    holding the last output when ``return_all_outputs=False``).  At masked steps the previous output (zeros if
    ``zero_output_for_mask``) and the previous states are carried over.
    """
    inputs = tree.map_structure(convert_to_tensor, inputs)
    flat_inputs = tree.flatten(inputs)
    if not time_major:
        flat_inputs = [x.transpose(0, 1) for x in flat_inputs]
    steps = flat_inputs[0].shape[0]
    if mask is not None:
        mask = convert_to_tensor(mask).to(torch.bool)
        if not time_major:
            mask = mask.transpose(0, 1)
    constants = list(constants) if constants else []
    states = tuple(initial_states)
    order = range(steps - 1, -1, -1) if go_backwards else range(steps)
    outputs = []
    last_output = None
    prev_output = None
    for t in order:
        x_t = tree.pack_sequence_as(inputs, [x[t] for x in flat_inputs])
        out, new_states = step_function(x_t, tuple(states) + tuple(constants))
        new_states = list(new_states) if isinstance(new_states, (list, tuple)) else [new_states]
        if mask is not None:
            m = mask[t]
            if prev_output is None:
                prev_output = torch.zeros_like(out)
            keep = _expand_mask(m, out)
            masked_out = torch.where(keep, out, torch.zeros_like(out) if zero_output_for_mask else prev_output)
            prev_output = torch.where(keep, out, prev_output)
            flat_new, flat_old = tree.flatten(new_states), tree.flatten(list(states))
            merged = [torch.where(_expand_mask(m, n), n, o) for n, o in zip(flat_new, flat_old)]
            new_states = tree.pack_sequence_as(new_states, merged)
            out_store = masked_out
            last_output = prev_output if not zero_output_for_mask else masked_out
        else:
            out_store = out
            last_output = out
        if return_all_outputs:
            outputs.append(out_store)
        states = tuple(new_states)
    if steps == 0:
        raise ValueError("RNN inputs must have at least one time step.")
    if return_all_outputs:
        stacked = torch.stack(outputs, dim=0)
    else:
        stacked = last_output.unsqueeze(0)
    if not time_major:
        stacked = stacked.transpose(0, 1)
    return last_output, stacked, list(states)
