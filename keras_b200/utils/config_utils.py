"""``keras.utils.Config``: attribute-style, JSON-serialisable, freezable configuration record
(keras/src/utils/config.py:12-190)."""

import copy
import difflib
import json

from keras_b200.core.export_registry import keras_export


@keras_export("keras.utils.Config")
class Config:
    __attrs__ = None

    def __init__(self, **kwargs):
        self._config = kwargs
        self._frozen = False
        self.__attrs__ = set(dir(self))

    @property
    def frozen(self):
        return self._frozen

    def freeze(self):
        self._frozen = True

    def unfreeze(self):
        self._frozen = False

    def _raise_if_frozen(self):
        if self._frozen:
            raise ValueError("Cannot mutate attribute(s) because the config is frozen.")

    def as_dict(self):
        return copy.copy(self._config)

    def to_json(self):
        return json.dumps(self._config)

    def keys(self):
        return self._config.keys()

    def values(self):
        return self._config.values()

    def items(self):
        return self._config.items()

    def pop(self, *args):
        self._raise_if_frozen()
        return self._config.pop(*args)

    def update(self, *args, **kwargs):
        self._raise_if_frozen()
        return self._config.update(*args, **kwargs)

    def get(self, keyname, value=None):
        return self._config.get(keyname, value)

    def __setattr__(self, name, value):
        attrs = object.__getattribute__(self, "__attrs__")
        if attrs is None or name in attrs:
            return object.__setattr__(self, name, value)
        self._raise_if_frozen()
        self._config[name] = value

    def __getattr__(self, name):
        attrs = object.__getattribute__(self, "__attrs__")
        if attrs is None or name in attrs:
            return object.__getattribute__(self, name)
        if name in self._config:
            return self._config[name]
        msg = f"Unknown attribute: '{name}'."
        matches = difflib.get_close_matches(name, self._config.keys(), n=1, cutoff=0.7)
        if matches:
            msg += f" Did you mean '{matches[0]}'?"
        raise AttributeError(msg)

    def __setitem__(self, key, item):
        self._raise_if_frozen()
        self._config[key] = item

    def __getitem__(self, key):
        return self._config[key]

    def __repr__(self):
        return f"<Config {self._config}>"

    def __iter__(self):
        keys = sorted(self._config.keys())
        for k in keys:
            yield k

    def __len__(self):
        return len(self._config)

    def __delitem__(self, key):
        self._raise_if_frozen()
        del self._config[key]

    def __contains__(self, item):
        return item in self._config
