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


def test_exported_paths_match_the_pinned_listing():
    """Adding or removing a public symbol has to come with an update of tests/golden_api.txt
    (``python -m keras_b200.api_listing > tests/golden_api.txt``)."""
    import os

    from keras_b200 import api_listing

    with open(os.path.join(os.path.dirname(__file__), "golden_api.txt")) as f:
        pinned = [line.strip() for line in f if line.strip()]
    current = api_listing.public_paths()
    assert current == pinned, {"added": sorted(set(current) - set(pinned)), "removed": sorted(set(pinned) - set(current))}
