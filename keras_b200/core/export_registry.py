"""Registry of public names.

``@keras_export("keras.layers.Dense")`` records the canonical public path of a symbol.  The
path doubles as the *serialization* identity (``module="keras.layers"``,
``class_name="Dense"``), which is what makes files interchangeable with reference Keras
(keras/src/api_export.py:7-49, keras/src/saving/serialization_lib.py:328-360).
"""

_PATH_TO_OBJ = {}
_OBJ_TO_PATHS = {}


class keras_export:
    def __init__(self, path):
        self.paths = [path] if isinstance(path, str) else list(path)

    def __call__(self, symbol):
        for p in self.paths:
            _PATH_TO_OBJ[p] = symbol
        try:
            _OBJ_TO_PATHS[symbol] = self.paths
            symbol._api_export_path = self.paths
        except (TypeError, AttributeError):
            pass
        return symbol


def get_symbol_from_name(name):
    return _PATH_TO_OBJ.get(name)


def get_name_from_symbol(symbol):
    paths = getattr(symbol, "_api_export_path", None)
    if paths is None:
        return None
    # An inherited attribute does not count: the subclass itself must be exported.
    if isinstance(symbol, type) and "_api_export_path" not in symbol.__dict__:
        return None
    return paths[0]


def all_exports():
    return dict(_PATH_TO_OBJ)
