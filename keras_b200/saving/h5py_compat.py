"""A stand-in for the ``h5py`` module, served by this package's own HDF5 reader and writer (``saving/hdf5.py``).

Programs written against ``h5py`` (the reference's loader, keras/src/saving/saving_lib.py:1190-1483, is one) can open
``.weights.h5`` files and the weight member of ``.keras`` archives on machines without h5py / libhdf5:

    from keras_b200.saving import h5py_compat
    h5py_compat.install()          # registers this module as ``h5py`` if no real h5py can be imported
    import h5py                    # -> this module

Covered: ``File`` (path, bytes or file object, mode "r"), ``Group`` (mapping protocol, ``attrs``, ``get`` with
``getclass`` / ``getlink``, ``visititems``), ``Dataset`` (``shape``, ``dtype``, ``attrs``, indexing, ``__array__``,
``external``, ``is_virtual``, ``id.get_storage_size()``), the link classes.  The files this package reads contain hard
links only, so ``getlink=True`` always answers ``HardLink``.  ``File(target, "w")`` offers ``create_group``,
``create_dataset(name, data=...)``, item assignment and ``attrs`` and writes the file on ``close``: what the reference's
saver (keras/src/saving/saving_lib.py:1425-1478) uses.
"""

import sys

import numpy as np

from keras_b200.saving import hdf5 as _hdf5

__version__ = "3.0.0"


class HardLink:
    pass


class SoftLink:
    def __init__(self, path=None):
        self.path = path


class ExternalLink:
    def __init__(self, filename=None, path=None):
        self.filename, self.path = filename, path


class _DatasetId:
    def __init__(self, dataset):
        self._dataset = dataset

    def get_storage_size(self):
        """Bytes the values occupy in the file (contiguous and compact layouts store them unpacked)."""
        info = self._dataset._info
        stored = info.get("stored_bytes")
        if stored is not None:
            return int(stored)
        return int(np.prod(self._dataset.shape, dtype=np.int64)) * np.dtype(self._dataset.dtype).itemsize


class Dataset(_hdf5.Dataset):
    external = None
    is_virtual = False

    @property
    def id(self):
        return _DatasetId(self)


def _adopt(node):
    """Re-class a node of the native reader so that ``isinstance(node, h5py.Group / h5py.Dataset)`` holds."""
    if isinstance(node, _hdf5.Dataset) and not isinstance(node, Dataset):
        node.__class__ = Dataset
    elif isinstance(node, _hdf5.Group) and not isinstance(node, (Group, File)):
        node.__class__ = Group
    return node


class Group(_hdf5.Group):
    def __getitem__(self, path):
        return _adopt(_hdf5.Group.__getitem__(self, path))

    def get(self, name, default=None, getclass=False, getlink=False):
        if name not in self:
            return default
        if getlink:
            return HardLink if getclass else HardLink()
        node = self[name]
        return type(node) if getclass else node

    def items(self):
        return [(k, self[k]) for k in self.keys()]

    def values(self):
        return [self[k] for k in self.keys()]

    def visititems(self, fn, _prefix=""):
        return _hdf5.Group.visititems(self, lambda name, node: fn(name, _adopt(node)), _prefix)


class _Attributes(dict):
    """``.attrs`` of a node being written: a dict that writes through to the writer's node."""


class _WriteDataset:
    """A dataset of a file opened for writing: just enough to attach attributes and read the value back."""

    def __init__(self, node):
        self._node = node
        self.attrs = node.attrs

    @property
    def shape(self):
        return tuple(self._node.array.shape)

    @property
    def dtype(self):
        return self._node.array.dtype

    def __array__(self, dtype=None, copy=None):
        arr = self._node.array
        return arr if dtype is None else arr.astype(dtype)

    def __getitem__(self, index):
        return self._node.array[index]


class _WriteGroup:
    """A group of a file opened for writing: ``create_group``, ``create_dataset(name, data=...)``, item assignment, ``attrs``."""

    def __init__(self, writer, path):
        self._writer, self._path = writer, path.strip("/")
        self._node = writer._group(self._path)
        self.attrs = self._node.attrs

    def _join(self, name):
        return f"{self._path}/{name}".strip("/")

    def create_group(self, name):
        if name.strip("/").split("/")[0] in self._node.children and self._join(name) and name in self:
            raise ValueError(f"Unable to create group (name already exists): {name}")
        return _WriteGroup(self._writer, self._join(name))

    def require_group(self, name):
        return _WriteGroup(self._writer, self._join(name))

    def create_dataset(self, name, data=None, shape=None, dtype=None, **kwargs):
        if data is None:
            data = np.zeros(shape or (), dtype=dtype or "float32")
        elif dtype is not None:
            data = np.asarray(data).astype(dtype)
        return _WriteDataset(self._writer.create_dataset(self._join(name), data))

    def __setitem__(self, name, value):
        self.create_dataset(name, data=value)

    def __getitem__(self, name):
        node = self._node
        for part in [p for p in name.split("/") if p]:
            node = node.children[part]
        return _WriteDataset(node) if hasattr(node, "array") else _WriteGroup(self._writer, self._join(name))

    def __delitem__(self, name):
        parts = [p for p in name.split("/") if p]
        node = self._node
        for part in parts[:-1]:
            node = node.children[part]
        del node.children[parts[-1]]

    def __contains__(self, name):
        node = self._node
        for part in [p for p in name.split("/") if p]:
            children = getattr(node, "children", None)
            if children is None or part not in children:
                return False
            node = children[part]
        return True

    def keys(self):
        return list(self._node.children.keys())

    def __iter__(self):
        return iter(self.keys())

    def __len__(self):
        return len(self._node.children)

    def __bool__(self):
        return True


class _WriteFile(_WriteGroup):
    """``h5py.File(target, "w")``: the tree is collected in memory and written to the path or file object on ``close``."""

    def __init__(self, target):
        self._target = target
        self._closed = False
        _WriteGroup.__init__(self, _hdf5.Writer(), "")

    def flush(self):
        pass

    def close(self):
        if self._closed:
            return
        self._closed = True
        data = self._writer.tobytes()
        if hasattr(self._target, "write"):
            self._target.write(data)
        else:
            with open(self._target, "wb") as f:
                f.write(data)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    @property
    def filename(self):
        return getattr(self._target, "name", self._target if isinstance(self._target, str) else "<memory>")


class File(Group, _hdf5.File):
    """``h5py.File``: mode "r" reads through this package's reader; mode "w" collects groups, datasets and attributes and writes
    them through this package's writer when the file is closed (mode "a" and "r+" are not offered)."""

    def __new__(cls, name=None, mode="r", **kwargs):
        if mode in ("w", "w-", "x"):
            return _WriteFile(name)
        return super().__new__(cls)

    def __init__(self, name, mode="r", **kwargs):
        if mode != "r":
            raise OSError("h5py_compat opens files for reading (\"r\") or writes new ones (\"w\"); appending is not offered")
        _hdf5.File.__init__(self, name, "r")

    @property
    def filename(self):
        return getattr(getattr(self, "_fh", None), "name", "<memory>")


def is_hdf5(path):
    try:
        with open(path, "rb") as f:
            return f.read(8) == b"\x89HDF\r\n\x1a\n"
    except OSError:
        return False


def install(force=False):
    """Make ``import h5py`` resolve to this module.  A real h5py wins unless ``force`` is set.  Returns the module that
    ``h5py`` now names."""
    if not force:
        try:
            import h5py  # noqa: F401

            return sys.modules["h5py"]
        except ImportError:
            pass
    sys.modules["h5py"] = sys.modules[__name__]
    return sys.modules[__name__]
