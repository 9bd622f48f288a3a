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


def _require(condition, message):
    if not condition:
        raise ValueError(message)


@keras_export("keras.distribution.DeviceMesh")
class DeviceMesh:
    """An N-dimensional grid of devices with one name per grid axis.  Device strings are ``"gpu:<rank>"``: one process
    drives one GPU, so a device is a process rank."""

    def __init__(self, shape, axis_names, devices=None):
        _require(shape and axis_names, f"Shape and axis_names cannot be empty. Received: shape={shape}, axis_names={axis_names}")
        _require(len(shape) == len(axis_names), f"Shape and axis_names should have same size. Received: shape={shape}, axis_names={axis_names}")
        grid = np.array(list_devices() if devices is None else devices)
        _require(int(np.prod(shape)) == grid.size, f"Shape does not match the number of devices. Received: shape={shape}; devices.shape={grid.shape}")
        self._shape = tuple(int(n) for n in shape)
        self._axis_names = list(axis_names)
        self._devices = grid.reshape(self._shape)
        self._groups = None

    @property
    def shape(self):
        return self._shape

    @property
    def axis_names(self):
        return self._axis_names

    @property
    def devices(self):
        return self._devices

    def axis_size(self, name):
        """Extent of the mesh along the axis called ``name``."""
        return self._shape[self._axis_names.index(name)]

    def coordinates_of(self, rank):
        """Grid coordinates of process ``rank`` (ranks fill the grid in row-major order)."""
        return tuple(int(c) for c in np.unravel_index(rank % self._devices.size, self._shape))

    @property
    def backend_mesh(self):
        """Process groups per mesh axis, created on first use."""
        if self._groups is None:
            from keras_b200.parallel import process_groups

            self._groups = process_groups.MeshGroups(self)
        return self._groups

    def __repr__(self):
        return f"<{type(self).__name__} shape={self.shape}, axis_names={self.axis_names}>"

    __str__ = __repr__


@keras_export("keras.distribution.TensorLayout")
class TensorLayout:
    """Per tensor dimension, the mesh axis it is split over (or ``None``: not split).  The mesh may be attached later, once
    (a ``LayoutMap`` does that for the layouts it receives)."""

    def __init__(self, axes, device_mesh=None):
        self._axes = tuple(axes)
        self._device_mesh = None
        if device_mesh is not None:
            self._bind(device_mesh)

    def _bind(self, mesh):
        known = set(mesh.axis_names)
        used = {a for a in self._axes if a is not None}
        _require(used <= known, f"Invalid axis names for Layout. Valid axis names: {known}, Got {used}")
        self._device_mesh = mesh

    @property
    def axes(self):
        return self._axes

    @property
    def device_mesh(self):
        return self._device_mesh

    @device_mesh.setter
    def device_mesh(self, mesh):
        _require(self._device_mesh is None, f"Cannot override device mesh value. Existing value is {self._device_mesh}")
        self._bind(mesh)

    @property
    def backend_layout(self):
        return self  # the sharding code reads `axes` and `device_mesh` directly

    def _validate_axes(self):
        if self._device_mesh is not None:
            self._bind(self._device_mesh)

    def __repr__(self):
        return f"<{type(self).__name__} axes={self.axes}, device_mesh={self.device_mesh}>"

    __str__ = __repr__


@keras_export("keras.distribution.LayoutMap")
class LayoutMap(collections.abc.MutableMapping):
    """Ordered ``pattern -> TensorLayout`` table.  A lookup returns the layout stored under exactly that key, else the layout
    of the one pattern that matches the *whole* path (``re.fullmatch``); two matching patterns are an error, none gives
    ``None``.  A plain tuple is accepted as a layout."""

    def __init__(self, device_mesh):
        self._device_mesh = device_mesh
        self._layout_map = collections.OrderedDict()
        self._compiled = {}

    @property
    def device_mesh(self):
        return self._device_mesh

    def __getitem__(self, path):
        direct = self._layout_map.get(path)
        if direct is not None:
            return direct
        hits = []
        for pattern in self._layout_map:
            matcher = self._compiled.get(pattern)
            if matcher is None:
                matcher = self._compiled[pattern] = re.compile(pattern)
            if matcher.fullmatch(path):
                hits.append(pattern)
        if len(hits) > 1:
            raise ValueError(f"Path '{path}' matches multiple layout specification keys: {hits}. Please make sure each tensor/variable path "
                             "only matches at most one layout specification key in the LayoutMap.")
        return self._layout_map[hits[0]] if hits else None

    def __setitem__(self, pattern, layout):
        _require(pattern not in self._layout_map, f"{pattern} already exist in the LayoutMap with value {self._layout_map.get(pattern)}. "
                 "Please make sure to not use duplicated keys.")
        if isinstance(layout, tuple):
            layout = TensorLayout(axes=layout)
        _require(isinstance(layout, TensorLayout), f"{layout} should be a TensorLayout type, got {type(layout)}")
        self._maybe_populate_device_mesh(layout)
        self._layout_map[pattern] = layout

    def __delitem__(self, pattern):
        self._compiled.pop(pattern, None)
        return self._layout_map.pop(pattern)

    def __len__(self):
        return len(self._layout_map)

    def __iter__(self):
        return iter(self._layout_map)

    def _maybe_populate_device_mesh(self, layout):
        if layout.device_mesh is None and self._device_mesh is not None:
            layout.device_mesh = self._device_mesh


LayoutMap.get = collections.abc.Mapping.get


class Distribution:
    """Base of the distribution strategies: a mesh, the name of its batch axis, and how this process fits into it."""

    def __init__(self, device_mesh, batch_dim_name=None, auto_shard_dataset=True):
        self._device_mesh = device_mesh
        self._batch_dim_name = batch_dim_name
        self._auto_shard_dataset = auto_shard_dataset
        self._num_processes = num_processes()
        self._process_id = process_id()

    # what a strategy decides ------------------------------------------------------------
    def get_data_layout(self, data_shape):
        raise NotImplementedError()

    def get_variable_layout(self, variable):
        raise NotImplementedError()

    def get_tensor_layout(self, path):
        raise NotImplementedError()

    def _batch_sharded(self, rank):
        """Layout of a rank-``rank`` input: first dimension over the batch axis, the rest whole."""
        return TensorLayout((self._batch_dim_name,) + (None,) * (rank - 1), self._device_mesh)

    # facts ------------------------------------------------------------------------------
    @property
    def device_mesh(self):
        return self._device_mesh

    @property
    def batch_dim_name(self):
        return self._batch_dim_name

    @property
    def auto_shard_dataset(self):
        return self._auto_shard_dataset

    @auto_shard_dataset.setter
    def auto_shard_dataset(self, value):
        self._auto_shard_dataset = value

    @property
    def num_model_replicas(self):
        """Copies of the model = extent of the batch axis (1 without one)."""
        return self._device_mesh.axis_size(self._batch_dim_name) if self._batch_dim_name else 1

    @property
    def num_data_shards(self):
        return min(self.num_model_replicas, self._num_processes)

    @property
    def data_shard_id(self):
        """Which slice of the data this process reads: its coordinate on the batch axis."""
        if self.num_data_shards <= 1:
            return 0
        axis = self._device_mesh.axis_names.index(self._batch_dim_name)
        return self._device_mesh.coordinates_of(self._process_id)[axis]

    def distribute_dataset(self, dataset):
        return dataset  # the data adapters shard by `data_shard_id` / `num_data_shards`

    @contextlib.contextmanager
    def scope(self):
        previous = distribution()
        set_distribution(self)
        try:
            yield
        finally:
            set_distribution(previous)

    def __repr__(self):
        return f"<{type(self).__name__} device_mesh={self.device_mesh}>"

    __str__ = __repr__


@keras_export("keras.distribution.DataParallel")
class DataParallel(Distribution):
    """Every process holds the whole model and a slice of each batch.  Built from a mesh (its first axis is the batch axis),
    a device list, or all devices of the job."""

    def __init__(self, device_mesh=None, devices=None, auto_shard_dataset=True):
        if device_mesh:
            _require(isinstance(device_mesh, DeviceMesh),
                     f"Expect `mesh` to be an instance of `DeviceMesh`. Received: mesh={device_mesh} (of type {type(device_mesh)})")
            if device_mesh.devices.ndim != 1:
                warnings.warn("Expect the input mesh to be 1D, but received mesh.devices.ndim=%d. The first axis will be used for "
                              "data-parallel sharding." % device_mesh.devices.ndim)
            mesh, batch_axis = device_mesh, device_mesh.axis_names[0]
        else:
            grid = np.array(devices if devices else list_devices())
            mesh, batch_axis = DeviceMesh(shape=grid.shape, axis_names=[DEFAULT_BATCH_DIM_NAME], devices=grid), DEFAULT_BATCH_DIM_NAME
        super().__init__(mesh, batch_axis, auto_shard_dataset)
        self._is_multi_process = self._num_processes > 1

    def get_data_layout(self, data_shape):
        return self._batch_sharded(len(data_shape))

    def get_variable_layout(self, variable):
        own = getattr(variable, "_layout", None)
        if own is not None:
            return own
        return TensorLayout((None,) * len(variable.shape), self._device_mesh)  # replicated

    def get_tensor_layout(self, path):
        return None


@keras_export("keras.distribution.ModelParallel")
class ModelParallel(Distribution):
    """Variables are split as the ``LayoutMap`` says (looked up by variable path), batches over ``batch_dim_name`` (default:
    the mesh's first axis).  Paths without an entry stay whole on every process."""

    def __init__(self, *, layout_map=None, batch_dim_name=None, auto_shard_dataset=True, **kwargs):
        kwargs.pop("device_mesh", None)  # accepted for compatibility: the layout map already names the mesh
        _require(layout_map is not None, "You must specify a layout_map argument.")
        _require(isinstance(layout_map, LayoutMap), f"Argument `layout_map` must be a `LayoutMap` instance. Received: layout_map={layout_map}")
        mesh = layout_map.device_mesh
        super().__init__(mesh, batch_dim_name or mesh.axis_names[0], auto_shard_dataset)
        self._layout_map = layout_map
        self._is_multi_process = self._num_processes > 1

    def get_data_layout(self, data_shape):
        return self._batch_sharded(len(data_shape))

    def get_variable_layout(self, variable):
        own = getattr(variable, "_layout", None)
        if own is not None:
            return own
        mapped = self._layout_map[variable.path]
        if mapped is not None:
            return mapped
        return TensorLayout((None,) * len(variable.shape), self._device_mesh)

    def get_tensor_layout(self, path):
        return self._layout_map[path]

    def shard_variable_init(self, variable, initializer):
        """Initialise only this rank's shard of ``variable`` (values equal the unsharded init)."""
        from keras_b200.parallel import tensor_parallel

        return tensor_parallel.shard_variable_init(self, variable, initializer)


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
