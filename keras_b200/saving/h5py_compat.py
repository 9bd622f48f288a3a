"""A read-only stand-in for the ``h5py`` module, served by this package's own HDF5 reader (``saving/hdf5.py``).

Programs written against ``h5py`` (the reference's loader, keras/src/saving/saving_lib.py:1190-1483, is one) can open
``.weights.h5`` files and the weight member of ``.keras`` archives on machines without h5py / libhdf5:

    from keras_b200.saving import h5py_compat
    h5py_compat.install()          # registers this module as ``h5py`` if no real h5py can be imported
    import h5py                    # -> this module

Covered: ``File`` (path, bytes or file object, mode "r"), ``Group`` (mapping protocol, ``attrs``, ``get`` with
``getclass`` / ``getlink``, ``visititems``), ``Dataset`` (``shape``, ``dtype``, ``attrs``, indexing, ``__array__``,
``external``, ``is_virtual``, ``id.get_storage_size()``), the link classes.  The files this package reads contain hard
links only, so ``getlink=True`` always answers ``HardLink``.  Writing is not offered here: use ``hdf5.Writer``.
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


class File(Group, _hdf5.File):
    def __init__(self, name, mode="r", **kwargs):
        if mode not in ("r", "r+") or mode == "r+":
            raise OSError("h5py_compat opens files read-only; write with keras_b200.saving.hdf5.Writer")
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
