"""Process-global, thread-local attribute bag.

Behaviour follows keras/src/backend/common/global_state.py:7-98: every scoped piece of
state (distribution, dtype policy, name-scope stack, stateless/symbolic scopes, uid counters)
lives in one thread-local dictionary so that ``clear_session`` can reset it in one place.
"""

import gc
import threading

_STATE = threading.local()


def _bag():
    bag = getattr(_STATE, "bag", None)
    if bag is None:
        bag = {}
        _STATE.bag = bag
    return bag


def set_global_attribute(name, value):
    _bag()[name] = value


def get_global_attribute(name, default=None, set_to_default=False):
    try:
        bag = _STATE.bag  # hot path: called several times per layer call
    except AttributeError:
        bag = _bag()
    value = bag.get(name)
    if value is None and default is not None:
        value = default
        if set_to_default:
            bag[name] = value
    return value


def clear_session(free_memory=True):
    """Drop every piece of global state (name uids, scopes, policies)."""
    _STATE.bag = {}
    if free_memory:
        gc.collect()
        try:
            import torch

            if torch.cuda.is_available():
                torch.cuda.empty_cache()
        except Exception:  # pragma: no cover
            pass
