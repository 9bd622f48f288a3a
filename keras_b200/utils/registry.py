"""Helpers to build ``get / serialize / deserialize`` triplets for identifier registries."""

import inspect

from keras_b200.core.naming import to_snake_case


def build_lookup(objects, aliases=None):
    table = {}
    for obj in objects:
        table[obj.__name__] = obj
        table[to_snake_case(obj.__name__)] = obj
    if aliases:
        table.update(aliases)
    return table
