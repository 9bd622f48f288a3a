"""Pickling of saveables through an in-memory ``.keras`` archive (keras/src/saving/keras_saveable.py:4-38)."""

import io


def _unpickle_model(data):
    from keras_b200.saving import saving_lib

    return saving_lib._load_model_from_fileobj(io.BytesIO(data), custom_objects=None, compile=True, safe_mode=False)


def reduce_saveable(obj):
    from keras_b200.saving import saving_lib

    buf = io.BytesIO()
    saving_lib._save_model_to_fileobj(obj, buf, "h5")
    return (_unpickle_model, (buf.getvalue(),))
