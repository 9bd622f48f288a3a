"""``keras.distribution``: ``DeviceMesh``, ``TensorLayout``, ``LayoutMap``, ``DataParallel``,
``ModelParallel`` and process bootstrap.

API and validation rules follow keras/src/distribution/distribution_lib.py:64-833.  The
realisation differs from the reference (whose torch backend only wraps the model in DDP and never
applies layouts, keras/src/backend/torch/trainer.py:50-92): one process drives one B200; variable
layouts are applied at creation (each rank materialises only its shard); gradient reduction,
sharded GEMMs and metric reduction are executed by ``keras_b200.parallel`` over NVLink.
"""

import collections
import contextlib
import os
import re
import warnings

import numpy as np
import torch

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export

DEFAULT_BATCH_DIM_NAME = "batch"
GLOBAL_ATTRIBUTE_NAME = "distribution"


@keras_export("keras.distribution.list_devices")
def list_devices(device_type=None):
    """Devices of the whole job as ``"gpu:i"`` / ``"cpu:i"`` strings (one per process on GPU)."""
    device_type = device_type.lower() if device_type else None
    if device_type in ("gpu", "cuda") or (device_type is None and torch.cuda.is_available()):
        n = get_device_count("gpu")
        return [f"gpu:{i}" for i in range(n)]
    if device_type in (None, "cpu"):
        return [f"cpu:{i}" for i in range(max(num_processes(), 1))]
    return []


@keras_export("keras.distribution.get_device_count")
def get_device_count(device_type=None):
    device_type = device_type.lower() if device_type else None
    if device_type in ("gpu", "cuda") or (device_type is None and torch.cuda.is_available()):
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            return torch.distributed.get_world_size()
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    if device_type in (None, "cpu"):
        return max(num_processes(), 1)
    return 0


@keras_export("keras.distribution.initialize")
def initialize(job_addresses=None, num_processes=None, process_id=None):
    """Join the job: one process per GPU, NCCL for device traffic and a gloo group for host control."""
    if job_addresses is None and "KERAS_DISTRIBUTION_JOB_ADDRESSES" in os.environ:
        job_addresses = os.environ["KERAS_DISTRIBUTION_JOB_ADDRESSES"]
    if num_processes is None and "KERAS_DISTRIBUTION_NUM_PROCESSES" in os.environ:
        num_processes = int(os.environ["KERAS_DISTRIBUTION_NUM_PROCESSES"])
    if process_id is None and "KERAS_DISTRIBUTION_PROCESS_ID" in os.environ:
        process_id = int(os.environ["KERAS_DISTRIBUTION_PROCESS_ID"])
    from keras_b200.parallel import process_groups

    process_groups.initialize(job_addresses, num_processes, process_id)


def num_processes():
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.distributed.get_world_size()
    return 1


def process_id():
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.distributed.get_rank()
    return 0


@keras_export("keras.distribution.DeviceMesh")
class DeviceMesh:
    def __init__(self, shape, axis_names, devices=None):
        if not shape or not axis_names:
            raise ValueError(f"Shape and axis_names cannot be empty. Received: shape={shape}, axis_names={axis_names}")
        if len(shape) != len(axis_names):
            raise ValueError(f"Shape and axis_names should have same size. Received: shape={shape}, axis_names={axis_names}")
        if devices is None:
            devices = list_devices()
        devices = np.array(devices)
        if np.prod(shape) != np.prod(devices.shape):
            raise ValueError(f"Shape does not match the number of devices. Received: shape={shape}; devices.shape={devices.shape}")
        self._shape = tuple(shape)
        self._axis_names = list(axis_names)
        self._devices = np.reshape(devices, shape)

    shape = property(lambda self: self._shape)
    axis_names = property(lambda self: self._axis_names)
    devices = property(lambda self: self._devices)

    @property
    def backend_mesh(self):
        if not hasattr(self, "_backend_mesh"):
            from keras_b200.parallel import process_groups

            self._backend_mesh = process_groups.MeshGroups(self)
        return self._backend_mesh

    def __repr__(self):
        return f"<{self.__class__.__name__} shape={self.shape}, axis_names={self.axis_names}>"

    def __str__(self):
        return self.__repr__()


@keras_export("keras.distribution.TensorLayout")
class TensorLayout:
    def __init__(self, axes, device_mesh=None):
        self._axes = tuple(axes)
        self._device_mesh = device_mesh
        self._validate_axes()

    axes = property(lambda self: self._axes)

    @property
    def device_mesh(self):
        return self._device_mesh

    @device_mesh.setter
    def device_mesh(self, device_mesh):
        if self._device_mesh is not None:
            raise ValueError(f"Cannot override device mesh value. Existing value is {self._device_mesh}")
        self._device_mesh = device_mesh
        self._validate_axes()

    @property
    def backend_layout(self):
        return self

    def _validate_axes(self):
        if self._device_mesh:
            valid = set(self._device_mesh.axis_names)
            axis_names = set(self._axes) - {None}
            if axis_names - valid:
                raise ValueError(f"Invalid axis names for Layout. Valid axis names: {valid}, Got {axis_names}")

    def __repr__(self):
        return f"<{self.__class__.__name__} axes={self.axes}, device_mesh={self.device_mesh}>"

    def __str__(self):
        return self.__repr__()


class Distribution:
    def __init__(self, device_mesh, batch_dim_name=None, auto_shard_dataset=True):
        self._device_mesh = device_mesh
        self._batch_dim_name = batch_dim_name
        self._auto_shard_dataset = auto_shard_dataset
        self._num_processes = num_processes()
        self._process_id = process_id()

    def get_data_layout(self, data_shape):
        raise NotImplementedError()

    def get_variable_layout(self, variable):
        raise NotImplementedError()

    def get_tensor_layout(self, path):
        raise NotImplementedError()

    @contextlib.contextmanager
    def scope(self):
        original = distribution()
        set_distribution(self)
        try:
            yield
        finally:
            set_distribution(original)

    device_mesh = property(lambda self: self._device_mesh)
    batch_dim_name = property(lambda self: self._batch_dim_name)
    auto_shard_dataset = property(lambda self: self._auto_shard_dataset)

    @auto_shard_dataset.setter
    def auto_shard_dataset(self, value):
        self._auto_shard_dataset = value

    @property
    def num_model_replicas(self):
        if not self._batch_dim_name:
            return 1
        mesh_batch_dim_index = self.device_mesh.axis_names.index(self._batch_dim_name)
        return self.device_mesh.shape[mesh_batch_dim_index]

    @property
    def num_data_shards(self):
        return min(self.num_model_replicas, self._num_processes)

    @property
    def data_shard_id(self):
        """Index of the data shard this process reads: its coordinate on the batch axis."""
        if self.num_data_shards <= 1:
            return 0
        mesh = self.device_mesh
        idx = mesh.axis_names.index(self._batch_dim_name)
        coords = np.unravel_index(self._process_id % int(np.prod(mesh.shape)), mesh.shape)
        return int(coords[idx])

    def distribute_dataset(self, dataset):
        return dataset

    def __repr__(self):
        return f"<{self.__class__.__name__} device_mesh={self.device_mesh}>"

    def __str__(self):
        return self.__repr__()


@keras_export("keras.distribution.DataParallel")
class DataParallel(Distribution):
    def __init__(self, device_mesh=None, devices=None, auto_shard_dataset=True):
        if device_mesh:
            self._initialize_with_device_mesh(device_mesh, auto_shard_dataset)
        elif devices:
            self._initialize_mesh_from_devices(devices, auto_shard_dataset)
        else:
            self._initialize_mesh_from_list_devices(auto_shard_dataset)
        self._is_multi_process = self._num_processes > 1

    def _initialize_with_device_mesh(self, device_mesh, auto_shard_dataset):
        if not isinstance(device_mesh, DeviceMesh):
            raise ValueError(f"Expect `mesh` to be an instance of `DeviceMesh`. Received: mesh={device_mesh} (of type {type(device_mesh)})")
        super().__init__(device_mesh, device_mesh.axis_names[0], auto_shard_dataset)
        if self.device_mesh.devices.ndim != 1:
            warnings.warn("Expect the input mesh to be 1D, but received mesh.devices.ndim=%d. The first axis will be used for data-parallel sharding." % device_mesh.devices.ndim)

    def _initialize_mesh_from_devices(self, devices, auto_shard_dataset):
        devices = np.array(devices)
        device_mesh = DeviceMesh(shape=devices.shape, axis_names=[DEFAULT_BATCH_DIM_NAME], devices=devices)
        super().__init__(device_mesh, DEFAULT_BATCH_DIM_NAME, auto_shard_dataset)

    def _initialize_mesh_from_list_devices(self, auto_shard_dataset):
        devices = np.array(list_devices())
        device_mesh = DeviceMesh(shape=devices.shape, axis_names=[DEFAULT_BATCH_DIM_NAME], devices=devices)
        super().__init__(device_mesh, DEFAULT_BATCH_DIM_NAME, auto_shard_dataset)

    def get_data_layout(self, data_shape):
        data_shard_spec = [None] * len(data_shape)
        data_shard_spec[0] = self.batch_dim_name
        return TensorLayout(data_shard_spec, self.device_mesh)

    def get_variable_layout(self, variable):
        if getattr(variable, "_layout", None) is not None:
            return variable._layout
        return None

    def get_tensor_layout(self, path):
        return None


@keras_export("keras.distribution.ModelParallel")
class ModelParallel(Distribution):
    def __init__(self, *, layout_map=None, batch_dim_name=None, auto_shard_dataset=True, **kwargs):
        kwargs.pop("device_mesh", None)
        if layout_map is None:
            raise ValueError("You must specify a layout_map argument.")
        if not isinstance(layout_map, LayoutMap):
            raise ValueError(f"Argument `layout_map` must be a `LayoutMap` instance. Received: layout_map={layout_map}")
        device_mesh = layout_map.device_mesh
        batch_dim_name = batch_dim_name or device_mesh.axis_names[0]
        super().__init__(device_mesh, batch_dim_name, auto_shard_dataset)
        self._layout_map = layout_map
        self._is_multi_process = self._num_processes > 1

    def get_data_layout(self, data_shape):
        data_shard_spec = [None] * len(data_shape)
        data_shard_spec[0] = self.batch_dim_name
        return TensorLayout(data_shard_spec, self.device_mesh)

    def get_variable_layout(self, variable):
        if getattr(variable, "_layout", None) is not None:
            return variable._layout
        variable_layout = self._layout_map[variable.path]
        if variable_layout is not None:
            return variable_layout
        return TensorLayout([None] * len(variable.shape), self.device_mesh)

    def get_tensor_layout(self, path):
        return self._layout_map[path]

    def shard_variable_init(self, variable, initializer):
        """Initialise only this rank's shard of ``variable`` (values equal the unsharded init)."""
        from keras_b200.parallel import tensor_parallel

        return tensor_parallel.shard_variable_init(self, variable, initializer)


@keras_export("keras.distribution.LayoutMap")
class LayoutMap(collections.abc.MutableMapping):
    def __init__(self, device_mesh):
        self._layout_map = collections.OrderedDict()
        self._device_mesh = device_mesh

    def __getitem__(self, key):
        if key in self._layout_map:
            return self._layout_map[key]
        matching_keys = []
        for k in self._layout_map:
            if re.search(k, key):
                matching_keys.append(k)
        if len(matching_keys) > 1:
            raise ValueError(f"Path '{key}' matches multiple layout specification keys: {matching_keys}. Please make sure each tensor/variable path only matches at most one layout specification key in the LayoutMap.")
        elif len(matching_keys) == 1:
            return self._layout_map[matching_keys[0]]
        return None

    def __setitem__(self, key, layout):
        if key in self._layout_map:
            raise ValueError(f"{key} already exist in the LayoutMap with value {self._layout_map[key]}. Please make sure to not use duplicated keys.")
        if isinstance(layout, tuple):
            layout = TensorLayout(axes=layout, device_mesh=None)
        if not isinstance(layout, TensorLayout):
            raise ValueError(f"{layout} should be a TensorLayout type, got {type(layout)}")
        self._maybe_populate_device_mesh(layout)
        self._layout_map[key] = layout

    def __delitem__(self, key):
        return self._layout_map.pop(key)

    def __len__(self):
        return len(self._layout_map)

    def __iter__(self):
        return iter(self._layout_map)

    device_mesh = property(lambda self: self._device_mesh)

    def _maybe_populate_device_mesh(self, layout):
        if layout.device_mesh is None and self.device_mesh is not None:
            layout.device_mesh = self.device_mesh


LayoutMap.get = collections.abc.Mapping.get


@keras_export("keras.distribution.distribute_tensor")
def distribute_tensor(tensor, layout):
    """Re-lay out ``tensor`` (a full/replicated value on this rank) as ``layout``: returns this rank's shard."""
    from keras_b200.core.keras_tensor import KerasTensor

    if isinstance(tensor, KerasTensor):
        return tensor
    from keras_b200.parallel import tensor_parallel

    return tensor_parallel.distribute_tensor(tensor, layout)


@keras_export("keras.distribution.distribution")
def distribution():
    return global_state.get_global_attribute(GLOBAL_ATTRIBUTE_NAME)


@keras_export("keras.distribution.set_distribution")
def set_distribution(value):
    global_state.set_global_attribute(GLOBAL_ATTRIBUTE_NAME, value)
