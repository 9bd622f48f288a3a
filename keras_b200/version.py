"""Version of the framework and of the Keras API level it reproduces (keras/src/version.py:4)."""

__version__ = "0.1.0"
# Files written by this framework declare this Keras version in metadata.json so that
# reference Keras accepts them.
KERAS_API_VERSION = "3.16.0"


def version():
    return __version__
