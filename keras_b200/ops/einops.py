"""``keras.ops.rearrange``: einops-style reshaping (keras/src/ops/einops.py)."""

import re

from keras_b200.ops._dispatch import op
from keras_b200.ops.numpy import _t


def _parse(side):
    tokens, i = [], 0
    for m in re.finditer(r"\(([^)]*)\)|(\S+)", side):
        if m.group(1) is not None:
            tokens.append(m.group(1).split())
        else:
            tokens.append(m.group(2))
    return tokens


@op()
def rearrange(tensor, pattern, **axes_lengths):
    x = _t(tensor)
    if "->" not in pattern:
        raise ValueError(f"Pattern must contain '->'. Received: {pattern}")
    lhs, rhs = [s.strip() for s in pattern.split("->")]
    left, right = _parse(lhs), _parse(rhs)
    if len(left) != x.ndim:
        raise ValueError(f"Pattern {lhs!r} has {len(left)} axes but the tensor has rank {x.ndim}.")
    sizes = dict(axes_lengths)
    flat_names = []
    for tok, dim in zip(left, x.shape):
        if isinstance(tok, list):
            known = 1
            unknown = [n for n in tok if n not in sizes and n != "1"]
            for n in tok:
                if n in sizes:
                    known *= sizes[n]
            if len(unknown) > 1:
                raise ValueError(f"Cannot infer sizes of {unknown} in group {tok}.")
            if unknown:
                sizes[unknown[0]] = dim // known
            flat_names.extend(tok)
        else:
            sizes[tok] = dim
            flat_names.append(tok)
    x = x.reshape([1 if n == "1" else sizes[n] for n in flat_names])
    out_names = []
    for tok in right:
        out_names.extend(tok if isinstance(tok, list) else [tok])
    named = [n for n in flat_names if n != "1"]
    x = x.reshape([sizes[n] for n in named])
    perm = [named.index(n) for n in out_names if n != "1"]
    x = x.permute(perm)
    shape = []
    for tok in right:
        if isinstance(tok, list):
            s = 1
            for n in tok:
                s *= 1 if n == "1" else sizes[n]
            shape.append(s)
        else:
            shape.append(1 if tok == "1" else sizes[tok])
    return x.reshape(shape)
