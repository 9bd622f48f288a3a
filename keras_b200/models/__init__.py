from keras_b200.models.functional import Functional  # noqa: F401
from keras_b200.models.model import Model  # noqa: F401
from keras_b200.models.sequential import Sequential  # noqa: F401
from keras_b200.models.cloning import clone_model  # noqa: F401
