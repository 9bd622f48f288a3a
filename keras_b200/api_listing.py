"""Listing of the public API: every path registered with ``keras_export``, one per line, sorted.

``python -m keras_b200.api_listing`` prints it; ``tests/golden_api.txt`` pins it so that a symbol cannot leave or enter the
public surface unnoticed (the reference keeps generated ``keras/api`` files under version control for the same purpose:
api_gen.py, keras/api/_tf_keras).
"""

import sys


def public_paths():
    import importlib
    import pkgutil

    import keras_b200
    from keras_b200.core.export_registry import all_exports

    # some packages load on first use: import every module so that every export decorator has run
    for info in pkgutil.walk_packages(keras_b200.__path__, prefix="keras_b200."):
        if ".kernels.csrc" in info.name or info.name.endswith("__main__"):
            continue
        try:
            importlib.import_module(info.name)
        except ImportError:
            pass  # a bridge to a package that is not installed
    return sorted(all_exports())


def main(argv=None):
    out = sys.stdout
    for path in public_paths():
        out.write(path + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
