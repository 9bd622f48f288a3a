"""Every public symbol of the reference's ``keras`` namespace (three levels deep) exists here under the same name."""

import types

import keras_b200 as keras
from tests import oracle

# packaging artefacts of the reference, not API
NOT_API = {"keras.api", "keras.src"}


def test_public_namespace_covers_the_reference():
    rk = oracle.ref()
    missing = []

    def walk(theirs, ours, path, depth):
        for name in dir(theirs):
            if name.startswith("_"):
                continue
            full = f"{path}.{name}"
            if full in NOT_API:
                continue
            value = getattr(theirs, name)
            try:
                mine = getattr(ours, name)
            except AttributeError:
                missing.append(full)
                continue
            if isinstance(value, types.ModuleType) and value.__name__.startswith("keras") and depth < 3:
                walk(value, mine, full, depth + 1)

    walk(rk, keras, "keras", 0)
    assert not missing, missing
