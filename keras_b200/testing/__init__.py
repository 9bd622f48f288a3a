from keras_b200.testing.test_case import TestCase, torch_uses_gpu, uses_gpu  # noqa: F401
from keras_b200.testing.test_utils import get_test_data, named_product  # noqa: F401
