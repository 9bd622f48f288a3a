"""Automatic object names: ``dense``, ``dense_1`` … (keras/src/utils/naming.py)."""

from keras_b200.core.export_registry import keras_export

import collections
import re

from keras_b200.core import global_state


def to_snake_case(name):
    name = re.sub(r"\W+", "", name)
    name = re.sub("(.)([A-Z][a-z]+)", r"\1_\2", name)
    name = re.sub("([a-z])([A-Z])", r"\1_\2", name).lower()
    return name


def uniquify(name):
    counts = global_state.get_global_attribute(
        "name_uids", default=collections.defaultdict(int), set_to_default=True
    )
    n = counts[name]
    counts[name] = n + 1
    return f"{name}_{n}" if n > 0 else name


def auto_name(prefix):
    return uniquify(to_snake_case(prefix))


@keras_export("keras.backend.get_uid")
def get_uid(prefix=""):
    counts = global_state.get_global_attribute(
        "object_uids", default=collections.defaultdict(int), set_to_default=True
    )
    counts[prefix] += 1
    return counts[prefix]


def reset_uids():
    global_state.set_global_attribute("name_uids", collections.defaultdict(int))
    global_state.set_global_attribute("object_uids", collections.defaultdict(int))


def get_object_name(obj):
    if hasattr(obj, "name"):
        return obj.name
    if hasattr(obj, "__name__"):
        return to_snake_case(obj.__name__)
    if hasattr(obj, "__class__"):
        return to_snake_case(obj.__class__.__name__)
    return to_snake_case(str(obj))
