"""Version of the framework and of the Keras API level it reproduces (keras/src/version.py:4)."""

from keras_b200.core.export_registry import keras_export

__version__ = "0.1.0"
# Files written by this framework declare this Keras version in metadata.json so that
# reference Keras accepts them.
KERAS_API_VERSION = "3.16.0"


@keras_export("keras.version")
def version():
    return __version__
