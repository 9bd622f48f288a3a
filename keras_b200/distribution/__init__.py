from keras_b200.distribution.distribution_lib import (  # noqa: F401
    DataParallel, DeviceMesh, Distribution, LayoutMap, ModelParallel, TensorLayout, distribute_tensor, distribution,
    get_device_count, initialize, list_devices, set_distribution,
)
