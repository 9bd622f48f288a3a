"""Nested-structure utilities (``keras.tree``).

Own implementation over Python containers; semantics of keras/src/tree/tree_api.py:
dict entries are visited in sorted-key order, ``None`` is a leaf, namedtuples keep their type.
"""

import collections
import collections.abc

from keras_b200.core.export_registry import keras_export


class _MapToNone:
    def __repr__(self):
        return "keras.tree.MAP_TO_NONE"


MAP_TO_NONE = _MapToNone()
keras_export("keras.tree.MAP_TO_NONE")(MAP_TO_NONE)

_REGISTERED = {}  # type -> (flatten_fn, unflatten_fn)


def register_tree_node_class(cls):
    """Register a class with ``tree_flatten()`` / ``tree_unflatten(aux, children)``."""
    _REGISTERED[cls] = (lambda o: o.tree_flatten(), cls.tree_unflatten)
    return cls


def register_tree_node(cls, flatten_func=None, unflatten_func=None):
    if flatten_func is None:
        flatten_func = lambda o: o.tree_flatten()
    if unflatten_func is None:
        unflatten_func = cls.tree_unflatten
    _REGISTERED[cls] = (flatten_func, unflatten_func)
    return cls


def _is_namedtuple(x):
    return isinstance(x, tuple) and hasattr(x, "_fields")


def _sorted_keys(d):
    if isinstance(d, collections.OrderedDict):
        pass
    try:
        return sorted(d)
    except TypeError:
        return list(d)


def _children(x):
    """Return (keys, values, rebuild) or None for a leaf."""
    t = type(x)
    if t in _REGISTERED:
        fl, un = _REGISTERED[t]
        children, aux = fl(x)
        children = list(children)
        return list(range(len(children))), children, lambda vals: un(aux, vals)
    if isinstance(x, dict):
        keys = _sorted_keys(x)

        def rebuild(vals, _x=x, _keys=keys):
            mapping = dict(zip(_keys, vals))
            if isinstance(_x, collections.defaultdict):
                out = collections.defaultdict(_x.default_factory)
                for k in _x:
                    out[k] = mapping[k]
                return out
            if type(_x) is dict or getattr(type(_x), "_tree_rebuild_as_dict", False):
                return {k: mapping[k] for k in _x}
            try:
                return type(_x)((k, mapping[k]) for k in _x)
            except TypeError:
                return {k: mapping[k] for k in _x}

        return keys, [x[k] for k in keys], rebuild
    if _is_namedtuple(x):
        return list(x._fields), list(x), lambda vals, _t=t: _t(*vals)
    if isinstance(x, (list, tuple)):
        tx = type(x)

        def rebuild(vals, _tx=tx):
            if _tx is list or _tx is tuple:
                return _tx(vals)
            if getattr(_tx, "_tree_rebuild_as_list", False):
                return list(vals)
            try:
                return _tx(vals)
            except TypeError:
                return list(vals)

        return list(range(len(x))), list(x), rebuild
    if isinstance(x, collections.abc.Mapping) and not isinstance(x, (str, bytes)):
        keys = _sorted_keys(x)
        return keys, [x[k] for k in keys], lambda vals, _k=keys: dict(zip(_k, vals))
    return None


@keras_export("keras.tree.is_nested")
def is_nested(structure):
    return _children(structure) is not None


# The recursive helpers below are module-level functions on purpose: a nested function that calls itself refers to itself
# through a closure cell, i.e. every call would leave a reference cycle that keeps whatever it captured (tensors with
# their autograd graphs, in the training step) alive until the cyclic garbage collector runs.
def _flatten_into(x, out):
    ch = _children(x)
    if ch is None:
        out.append(x)
    else:
        for v in ch[1]:
            _flatten_into(v, out)


@keras_export("keras.tree.flatten")
def flatten(structure):
    out = []
    _flatten_into(structure, out)
    return out


def _flatten_paths_into(x, path, out):
    ch = _children(x)
    if ch is None:
        out.append((path, x))
    else:
        for k, v in zip(ch[0], ch[1]):
            _flatten_paths_into(v, path + (k,), out)


@keras_export("keras.tree.flatten_with_path")
def flatten_with_path(structure):
    out = []
    _flatten_paths_into(structure, (), out)
    return out


def _traverse_top_down(func, x):
    r = func(x)
    if r is MAP_TO_NONE:
        return None
    if r is not None:
        return r
    ch = _children(x)
    if ch is None:
        return x
    return ch[2]([_traverse_top_down(func, v) for v in ch[1]])


def _traverse_bottom_up(func, x):
    ch = _children(x)
    if ch is not None:
        x = ch[2]([_traverse_bottom_up(func, v) for v in ch[1]])
    r = func(x)
    if r is MAP_TO_NONE:
        return None
    return x if r is None else r


@keras_export("keras.tree.traverse")
def traverse(func, structure, top_down=True):
    if not callable(func):
        raise TypeError(f"`func` must be callable, got {func} of type {type(func)}")
    return _traverse_top_down(func, structure) if top_down else _traverse_bottom_up(func, structure)


def _structure_mismatch(a, b, path="", check_types=True):
    ca, cb = _children(a), _children(b)
    if (ca is None) != (cb is None):
        return f"at {path or '<root>'}: {type(a).__name__} vs {type(b).__name__}"
    if ca is None:
        return None
    if check_types:
        ta, tb = type(a), type(b)
        if ta is not tb and not (isinstance(a, dict) and isinstance(b, dict)):
            return f"at {path or '<root>'}: type {ta.__name__} vs {tb.__name__}"
    if len(ca[0]) != len(cb[0]) or (isinstance(a, dict) and list(ca[0]) != list(cb[0])):
        return f"at {path or '<root>'}: children {ca[0]} vs {cb[0]}"
    for k, va, vb in zip(ca[0], ca[1], cb[1]):
        msg = _structure_mismatch(va, vb, f"{path}/{k}", check_types)
        if msg:
            return msg
    return None


@keras_export("keras.tree.assert_same_structure")
def assert_same_structure(a, b, check_types=None):
    msg = _structure_mismatch(a, b, check_types=True if check_types is None else check_types)
    if msg:
        raise ValueError(
            f"The two structures don't have the same nested structure ({msg}).\n"
            f"First structure: {a!r}\nSecond structure: {b!r}"
        )


@keras_export("keras.tree.assert_same_paths")
def assert_same_paths(a, b):
    pa = {p for p, _ in flatten_with_path(a)}
    pb = {p for p, _ in flatten_with_path(b)}
    if pa != pb:
        raise ValueError(
            "`a` and `b` don't have the same paths. "
            f"Paths in `a` missing in `b`: {sorted(map(str, pa - pb))}; "
            f"paths in `b` missing in `a`: {sorted(map(str, pb - pa))}"
        )


@keras_export("keras.tree.map_structure")
def map_structure(func, *structures, none_is_leaf=True):
    if not callable(func):
        raise TypeError(f"`func` must be callable, got {func} of type {type(func)}")
    if not structures:
        raise ValueError("Must provide at least one structure")
    first = structures[0]
    if len(structures) == 1:
        return _map_one(func, first)
    for other in structures[1:]:
        assert_same_structure(first, other, check_types=False)
    return _map_many(func, structures)


def _map_one(func, x):
    ch = _children(x)
    if ch is None:
        return func(x)
    return ch[2]([_map_one(func, v) for v in ch[1]])


def _map_many(func, xs):
    ch = _children(xs[0])
    if ch is None:
        return func(*xs)
    others = [_children(x)[1] for x in xs[1:]]
    return ch[2]([_map_many(func, (v, *[o[i] for o in others])) for i, v in enumerate(ch[1])])


def _map_up_to(func, shallow, xs):
    ch = _children(shallow)
    if ch is None:
        return func(*xs)
    subs = []
    for x in xs:
        cx = _children(x)
        if cx is None or len(cx[1]) != len(ch[1]):
            raise ValueError(
                f"Structure {x!r} does not match the shallow structure {shallow!r}."
            )
        subs.append(cx[1])
    return ch[2]([_map_up_to(func, v, [s[i] for s in subs]) for i, v in enumerate(ch[1])])


@keras_export("keras.tree.map_structure_up_to")
def map_structure_up_to(shallow_structure, func, *structures):
    return _map_up_to(func, shallow_structure, structures)


@keras_export("keras.tree.pack_sequence_as")
def pack_sequence_as(structure, flat_sequence, sequence_fn=None):
    flat = list(flat_sequence)
    if not is_nested(structure):
        if len(flat) != 1:
            raise ValueError(
                "Incorrect number of elements: the structure is a scalar but "
                f"`len(flat_sequence)`={len(flat)}"
            )
        return flat[0]
    pos = [0]
    out = _pack(structure, flat, pos)
    if pos[0] != len(flat):
        raise ValueError(
            f"Could not pack sequence: structure had {pos[0]} leaves but flat_sequence had "
            f"{len(flat)} items."
        )
    return out


def _pack(x, flat, pos):
    ch = _children(x)
    if ch is None:
        if pos[0] >= len(flat):
            raise ValueError(
                f"Could not pack sequence: structure has more leaves than {len(flat)} values."
            )
        v = flat[pos[0]]
        pos[0] += 1
        return v
    return ch[2]([_pack(v, flat, pos) for v in ch[1]])


@keras_export("keras.tree.lists_to_tuples")
def lists_to_tuples(structure):
    ch = _children(structure)
    if ch is None:
        return structure
    vals = [lists_to_tuples(v) for v in ch[1]]
    if type(structure) is list:
        return tuple(vals)
    return ch[2](vals)


def _is_shape(x):
    return isinstance(x, (list, tuple)) and all(isinstance(e, int) or e is None for e in x)


@keras_export("keras.tree.map_shape_structure")
def map_shape_structure(func, structure):
    """Like ``map_structure`` but tuples/lists made only of ints/None count as leaves."""
    if _is_shape(structure):
        return func(tuple(structure))
    ch = _children(structure)
    if ch is None:
        if structure is None:
            return None
        return func(structure)
    return ch[2]([map_shape_structure(func, v) for v in ch[1]])
