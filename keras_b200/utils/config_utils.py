"""``keras.utils.Config``: a record of named settings that reads like an object (``cfg.lr``) and like a mapping
(``cfg["lr"]``), serialises to JSON and can be frozen against changes (behaviour of keras/src/utils/config.py:12-190).

The entries live in one dict kept under a private slot of the instance; everything that is not one of the instance's own
two slots is an entry, so no table of reserved attribute names is needed.
"""

import difflib
import json
from collections.abc import MutableMapping

from keras_b200.core.export_registry import keras_export

_SLOTS = ("_config", "_frozen")


@keras_export("keras.utils.Config")
class Config(MutableMapping):
    def __init__(self, **entries):
        vars(self)["_config"] = dict(entries)
        vars(self)["_frozen"] = False

    # -- freezing ------------------------------------------------------------------------
    @property
    def frozen(self):
        return self._frozen

    def freeze(self):
        vars(self)["_frozen"] = True

    def unfreeze(self):
        vars(self)["_frozen"] = False

    def _writable(self):
        if self._frozen:
            raise ValueError("Cannot mutate attribute(s) because the config is frozen.")
        return self._config

    # -- mapping protocol (MutableMapping derives pop, update, get, keys, values, items, __contains__ from these) ---
    def __getitem__(self, key):
        return self._config[key]

    def __setitem__(self, key, value):
        self._writable()[key] = value

    def __delitem__(self, key):
        del self._writable()[key]

    def __iter__(self):
        return iter(sorted(self._config))

    def __len__(self):
        return len(self._config)

    def __contains__(self, key):
        return key in self._config

    def keys(self):
        return self._config.keys()

    def values(self):
        return self._config.values()

    def items(self):
        return self._config.items()

    def get(self, keyname, value=None):
        return self._config.get(keyname, value)

    def pop(self, *args):
        return self._writable().pop(*args)

    def update(self, *args, **kwargs):
        return self._writable().update(*args, **kwargs)

    # -- attribute protocol --------------------------------------------------------------
    def __getattr__(self, name):
        # reached only when normal lookup failed: the name is an entry or a mistake
        entries = vars(self).get("_config", {})
        if name in entries:
            return entries[name]
        hint = difflib.get_close_matches(name, list(entries), n=1, cutoff=0.7)
        raise AttributeError(f"Unknown attribute: '{name}'." + (f" Did you mean '{hint[0]}'?" if hint else ""))

    def __setattr__(self, name, value):
        if name in _SLOTS or isinstance(getattr(type(self), name, None), property):
            object.__setattr__(self, name, value)
        else:
            self._writable()[name] = value

    # -- export --------------------------------------------------------------------------
    def as_dict(self):
        return dict(self._config)

    def to_json(self):
        return json.dumps(self._config)

    def __repr__(self):
        return f"<Config {self._config}>"
