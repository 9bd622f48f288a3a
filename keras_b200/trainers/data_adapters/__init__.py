from keras_b200.trainers.data_adapters.adapters import (  # noqa: F401
    ArrayDataAdapter, DataAdapter, GeneratorDataAdapter, PyDataset, PyDatasetAdapter, TorchDataLoaderAdapter, get_data_adapter,
)
