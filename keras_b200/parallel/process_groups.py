"""Process bootstrap: one process per GPU, NCCL for device traffic, gloo for host-side control.

Counterpart of keras/src/backend/torch/distribution_lib.py:109-128 (``initialize``) and :186-212
(mesh → ``torch.distributed.DeviceMesh``).  Rendezvous uses ``MASTER_ADDR``/``MASTER_PORT`` (default
``127.0.0.1:29500``); ``job_addresses`` may carry ``host:port`` of the coordinator.
"""

import datetime
import os

import numpy as np
import torch
import torch.distributed as dist

_STATE = {"host_group": None, "initialized_here": False}


def is_initialized():
    return dist.is_available() and dist.is_initialized()


def world_size():
    return dist.get_world_size() if is_initialized() else 1


def rank():
    return dist.get_rank() if is_initialized() else 0


def local_rank():
    return int(os.environ.get("LOCAL_RANK", rank() % max(torch.cuda.device_count(), 1) if torch.cuda.is_available() else 0))


def initialize(job_addresses=None, num_processes=None, process_id=None, backend=None, timeout_s=None):
    """Join the job.  No-op when ``torch.distributed`` is already initialised or the job has one process."""
    if is_initialized():
        _ensure_host_group()
        return
    if job_addresses:
        first = job_addresses.split(",")[0]
        if ":" in first:
            host, port = first.rsplit(":", 1)
            os.environ.setdefault("MASTER_ADDR", host)
            os.environ.setdefault("MASTER_PORT", port)
        else:
            os.environ.setdefault("MASTER_ADDR", first)
    if num_processes is None:
        num_processes = int(os.environ.get("WORLD_SIZE", "1"))
    if process_id is None:
        process_id = int(os.environ.get("RANK", "0"))
    if num_processes <= 1:
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    kwargs = {}
    if use_cuda:
        lr = int(os.environ.get("LOCAL_RANK", process_id % torch.cuda.device_count()))
        torch.cuda.set_device(lr)
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", lr)
    if timeout_s is None:
        timeout_s = float(os.environ.get("KERAS_B200_PG_TIMEOUT_S", "600"))
    dist.init_process_group(backend=backend, rank=process_id, world_size=num_processes, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    _STATE["initialized_here"] = True
    _ensure_host_group()
    _agree_on_seed()


def _ensure_host_group():
    if _STATE["host_group"] is None and is_initialized():
        if dist.get_backend() == "gloo":
            _STATE["host_group"] = dist.group.WORLD
        else:
            _STATE["host_group"] = dist.new_group(backend="gloo")
    return _STATE["host_group"]


def host_group():
    """gloo group over all processes: barriers, object exchange, checkpoints, heartbeats."""
    return _ensure_host_group()


def _agree_on_seed():
    """All processes adopt rank 0's global seed so that replicated variables initialise identically
    (the reference does the same with a ``psum`` over devices, keras/src/backend/jax/distribution_lib.py:109-135)."""
    from keras_b200.random import seed_generator
    from keras_b200.utils import misc_utils

    seed = misc_utils.get_random_seed()
    if seed is None:
        seed = seed_generator.make_default_seed()
    payload = [int(seed)]
    dist.broadcast_object_list(payload, src=0, group=host_group())
    misc_utils.set_random_seed(payload[0])


def shutdown():
    if is_initialized() and _STATE["initialized_here"]:
        dist.destroy_process_group()
        _STATE["host_group"] = None
        _STATE["initialized_here"] = False


class MeshGroups:
    """Process groups of a ``DeviceMesh``: one group per (axis, position along the other axes).

    ``get_group(axis_name)`` returns the group of this process along that axis, like
    ``torch.distributed.DeviceMesh.get_group``.  Device ``"gpu:i"`` / ``"cpu:i"`` is process ``i``.
    """

    def __init__(self, mesh):
        self.mesh = mesh
        self.axis_names = list(mesh.axis_names)
        ids = np.array([int(str(d).split(":")[-1]) for d in np.ravel(mesh.devices)], dtype=np.int64).reshape(mesh.devices.shape)
        self.ranks = ids
        self._groups = {}
        self._members = {}
        me = rank()
        pos = np.argwhere(ids == me)
        self.coords = tuple(int(c) for c in pos[0]) if len(pos) else None
        ws = world_size()
        for ax, name in enumerate(self.axis_names):
            moved = np.moveaxis(ids, ax, -1).reshape(-1, ids.shape[ax])
            for row in moved:
                members = [int(r) for r in row]
                if ws > 1 and len(members) > 1 and max(members) < ws:
                    g = dist.new_group(ranks=members) if len(members) < ws else dist.group.WORLD
                else:
                    g = None
                if me in members:
                    self._groups[name] = g
                    self._members[name] = members

    def get_group(self, axis_name):
        return self._groups.get(axis_name)

    def members(self, axis_name):
        return self._members.get(axis_name, [rank()])

    def size(self, axis_name):
        return len(self.members(axis_name))

    def index(self, axis_name):
        m = self.members(axis_name)
        return m.index(rank()) if rank() in m else 0
