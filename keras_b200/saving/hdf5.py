"""Minimal HDF5 reader and writer (no ``h5py`` / libhdf5 dependency).

Covers what Keras weight files use (keras/src/saving/saving_lib.py:1289-1483): nested groups,
N-d numeric datasets, string attributes.

Reader: superblock v0-v3; v1 and v2 object headers with continuation blocks; old-style groups
(symbol table = v1 B-tree + local heap + SNOD) and new-style compact link messages; contiguous,
compact and chunked (v1 B-tree index, optional deflate/shuffle) layouts; fixed-point, float,
string, opaque, enum (bool) datatypes; fixed and variable-length string attributes (global heap).

Writer: emits the "earliest" file format that libhdf5 / h5py read back: superblock v0, v1 object
headers, symbol-table groups with multi-level B-trees, contiguous little-endian datasets,
variable-length UTF-8 string attributes stored in global heap collections (the form h5py writes
for ``attrs["name"] = "dense"``), 2-byte opaque datasets plus a ``dtype="bfloat16"`` attribute
for bfloat16 payloads, and an ``int8`` enum for booleans.
"""

import struct
import zlib

import numpy as np

SIGNATURE = b"\x89HDF\r\n\x1a\n"
UNDEF = 0xFFFFFFFFFFFFFFFF


# ==================================================================================== reader
class _Reader:
    def __init__(self, buf):
        self.buf = buf
        self.base = 0
        self._parse_superblock()
        self._gheaps = {}

    def u(self, off, n):
        return int.from_bytes(self.buf[off:off + n], "little")

    def _parse_superblock(self):
        b = self.buf
        start = 0
        while b[start:start + 8] != SIGNATURE:
            start = 512 if start == 0 else start * 2
            if start >= len(b):
                raise ValueError("Not an HDF5 file (signature not found).")
        self.sb_start = start
        version = b[start + 8]
        self.sb_version = version
        if version in (0, 1):
            self.size_offsets = b[start + 13]
            self.size_lengths = b[start + 14]
            p = start + 16
            self.leaf_k = self.u(p, 2)
            self.internal_k = self.u(p + 2, 2)
            p += 8
            if version == 1:
                p += 4
            so = self.size_offsets
            self.base = self.u(p, so)
            p += so * 4
            # root symbol table entry
            self.root_header = self.u(p + so, so)
        elif version in (2, 3):
            self.size_offsets = b[start + 9]
            self.size_lengths = b[start + 10]
            so = self.size_offsets
            p = start + 12
            self.base = self.u(p, so)
            self.root_header = self.u(p + 3 * so, so)
            self.leaf_k, self.internal_k = 4, 16
        else:
            raise ValueError(f"Unsupported HDF5 superblock version {version}.")
        if self.size_offsets != 8 or self.size_lengths != 8:
            raise ValueError("Only HDF5 files with 8-byte offsets and lengths are supported.")

    # ---- object headers -----------------------------------------------------------------
    def messages(self, addr):
        """Yield (type, flags, data bytes) for every header message of the object at ``addr``."""
        addr += self.base
        b = self.buf
        if b[addr:addr + 4] == b"OHDR":
            yield from self._messages_v2(addr)
            return
        version = b[addr]
        if version != 1:
            raise ValueError(f"Unsupported object header version {version} at {addr}.")
        nmsgs = self.u(addr + 2, 2)
        size = self.u(addr + 8, 4)
        blocks = [(addr + 16, size)]
        count = 0
        while blocks and count < nmsgs:
            p, remaining = blocks.pop(0)
            end = p + remaining
            while p + 8 <= end and count < nmsgs:
                mtype = self.u(p, 2)
                msize = self.u(p + 2, 2)
                flags = b[p + 4]
                data = b[p + 8:p + 8 + msize]
                p += 8 + msize
                count += 1
                if mtype == 0x10:
                    blocks.append((self.u_bytes(data, 0, 8) + self.base, self.u_bytes(data, 8, 8)))
                else:
                    yield mtype, flags, data

    @staticmethod
    def u_bytes(data, off, n):
        return int.from_bytes(data[off:off + n], "little")

    def _messages_v2(self, addr):
        b = self.buf
        flags = b[addr + 5]
        p = addr + 6
        if flags & 0x20:
            p += 16
        if flags & 0x10:
            p += 4
        size_field = 1 << (flags & 0x3)
        chunk_size = self.u(p, size_field)
        p += size_field
        track_order = bool(flags & 0x04)
        blocks = [(p, chunk_size)]
        while blocks:
            p, remaining = blocks.pop(0)
            end = p + remaining
            while p + 4 <= end:
                mtype = b[p]
                msize = self.u(p + 1, 2)
                mflags = b[p + 3]
                p += 4
                if track_order:
                    p += 2
                data = b[p:p + msize]
                p += msize
                if mtype == 0x10:
                    caddr = self.u_bytes(data, 0, 8) + self.base
                    clen = self.u_bytes(data, 8, 8)
                    blocks.append((caddr + 4, clen - 8))  # skip "OCHK", drop checksum
                elif mtype != 0:
                    yield mtype, mflags, data

    # ---- groups -------------------------------------------------------------------------
    def links(self, addr):
        """Ordered dict name -> object header address for the group at ``addr``."""
        out = {}
        for mtype, _, data in self.messages(addr):
            if mtype == 0x11:
                btree = self.u_bytes(data, 0, 8)
                heap = self.u_bytes(data, 8, 8)
                self._walk_group_btree(btree + self.base, self._heap_data(heap + self.base), out)
            elif mtype == 0x06:
                name, target = self._parse_link(data)
                if target is not None:
                    out[name] = target
            elif mtype == 0x02:
                # link info: dense storage is not supported (never produced for small groups
                # unless link count > 8; handled via fractal heap walk below when present)
                fheap = self.u_bytes(data, 2 + (8 if data[1] & 1 else 0), 8)
                if fheap != UNDEF:
                    self._walk_dense_links(data, out)
        return out

    def _heap_data(self, addr):
        b = self.buf
        if b[addr:addr + 4] != b"HEAP":
            raise ValueError("Corrupt HDF5 file: local heap signature missing.")
        size = self.u(addr + 8, 8)
        data_addr = self.u(addr + 24, 8) + self.base
        return bytes(b[data_addr:data_addr + size])

    def _walk_group_btree(self, addr, heap, out):
        b = self.buf
        if b[addr:addr + 4] != b"TREE":
            raise ValueError("Corrupt HDF5 file: B-tree signature missing.")
        level = b[addr + 5]
        used = self.u(addr + 6, 2)
        p = addr + 24
        children = []
        for _ in range(used):
            p += 8  # key
            children.append(self.u(p, 8) + self.base)
            p += 8
        for child in children:
            if level > 0:
                self._walk_group_btree(child, heap, out)
            else:
                if b[child:child + 4] != b"SNOD":
                    raise ValueError("Corrupt HDF5 file: symbol node signature missing.")
                n = self.u(child + 6, 2)
                q = child + 8
                for _ in range(n):
                    name_off = self.u(q, 8)
                    header = self.u(q + 8, 8)
                    end = heap.index(b"\x00", name_off)
                    out[bytes(heap[name_off:end]).decode("utf-8")] = header
                    q += 40

    def _parse_link(self, data):
        flags = data[1]
        p = 2
        ltype = 0
        if flags & 0x08:
            ltype = data[p]
            p += 1
        if flags & 0x04:
            p += 8
        if flags & 0x10:
            p += 1
        nlen_size = 1 << (flags & 0x3)
        nlen = self.u_bytes(data, p, nlen_size)
        p += nlen_size
        name = bytes(data[p:p + nlen]).decode("utf-8")
        p += nlen
        if ltype == 0:
            return name, self.u_bytes(data, p, 8)
        return name, None

    def _walk_dense_links(self, data, out):
        raise NotImplementedError(
            "This HDF5 file stores group links in a fractal heap (dense link storage), which this reader does not "
            "support. Re-save the file with h5py's default (earliest) format or fewer than ~8 links per new-style group."
        )

    # ---- datasets / attributes ------------------------------------------------------------
    def object_info(self, addr):
        """Return dict(kind='group'|'dataset', attrs={...}, [shape, dtype info, layout])."""
        info = {"attrs": {}, "kind": "group"}
        for mtype, _, data in self.messages(addr):
            if mtype == 0x01:
                info["shape"] = self._parse_dataspace(data)
            elif mtype == 0x03:
                info["dtype"] = self._parse_datatype(data, 0)[0]
            elif mtype == 0x08:
                info["layout"] = bytes(data)
                info["kind"] = "dataset"
            elif mtype == 0x0B:
                info["filters"] = self._parse_filters(data)
            elif mtype == 0x0C:
                try:
                    name, value = self._parse_attribute(data)
                    info["attrs"][name] = value
                except Exception:
                    pass
        return info

    def _parse_dataspace(self, data):
        version = data[0]
        rank = data[1]
        if version == 1:
            p = 8
        else:
            p = 4
            if data[3] == 2:  # null dataspace
                return None
        return tuple(self.u_bytes(data, p + 8 * i, 8) for i in range(rank))

    def _parse_datatype(self, data, p):
        """Return (descriptor dict, bytes consumed)."""
        cls = data[p] & 0x0F
        version = data[p] >> 4
        bits = data[p + 1:p + 4]
        size = self.u_bytes(data, p + 4, 4)
        q = p + 8
        if cls == 0:
            signed = bool(bits[0] & 0x08)
            big = bool(bits[0] & 1)
            return {"np": np.dtype(f"{'>' if big else '<'}{'i' if signed else 'u'}{size}")}, q + 4 - p
        if cls == 1:
            big = bool(bits[0] & 1)
            exp_size, mant_size = data[q + 5], data[q + 7]
            if size == 2 and exp_size == 8 and mant_size == 7:
                return {"np": np.dtype("<u2"), "bfloat16": True}, q + 12 - p
            return {"np": np.dtype(f"{'>' if big else '<'}f{size}")}, q + 12 - p
        if cls == 3:
            return {"np": np.dtype(f"S{size}"), "string": True, "utf8": (bits[0] >> 4) == 1}, q - p
        if cls == 5:
            taglen = bits[0]
            tag = bytes(data[q:q + taglen]).split(b"\x00")[0].decode("ascii", "ignore")
            padded = (taglen + 7) // 8 * 8
            return {"np": np.dtype(f"V{size}"), "opaque": True, "tag": tag, "size": size}, q + padded - p
        if cls == 8:
            n = self.u_bytes(bits, 0, 2)
            base, used = self._parse_datatype(data, q)
            q += used
            names = []
            for _ in range(n):
                end = bytes(data).index(b"\x00", q)
                names.append(bytes(data[q:end]).decode())
                ln = end - q + 1
                q += (ln + 7) // 8 * 8 if version < 3 else ln
            q += n * base["np"].itemsize
            is_bool = sorted(names) == ["FALSE", "TRUE"]
            return {"np": base["np"], "bool": is_bool}, q - p
        if cls == 9:
            vtype = bits[0] & 0x0F
            base, used = self._parse_datatype(data, q)
            return {"vlen": True, "vlen_string": vtype == 1, "base": base, "np": np.dtype("V16")}, q + used - p
        if cls == 10:
            rank = data[q]
            q += 1
            if version < 4 and version == 2:
                q += 3
            dims = [self.u_bytes(data, q + 4 * i, 4) for i in range(rank)]
            q += 4 * rank
            if version == 2:
                q += 4 * rank
            base, used = self._parse_datatype(data, q)
            return {"np": np.dtype((base["np"], tuple(dims)))}, q + used - p
        raise NotImplementedError(f"HDF5 datatype class {cls} is not supported.")

    def _parse_filters(self, data):
        version = data[0]
        n = data[1]
        p = 8 if version == 1 else 2
        out = []
        for _ in range(n):
            fid = self.u_bytes(data, p, 2)
            p += 2
            if version == 1 or fid >= 256:
                nlen = self.u_bytes(data, p, 2)
                p += 2
            else:
                nlen = 0
            p += 2  # flags
            ncd = self.u_bytes(data, p, 2)
            p += 2
            if nlen:
                p += (nlen + 7) // 8 * 8 if version == 1 else nlen
            cd = [self.u_bytes(data, p + 4 * i, 4) for i in range(ncd)]
            p += 4 * ncd
            if version == 1 and ncd % 2:
                p += 4
            out.append((fid, cd))
        return out

    def _parse_attribute(self, data):
        version = data[0]
        name_size = self.u_bytes(data, 2, 2)
        dt_size = self.u_bytes(data, 4, 2)
        ds_size = self.u_bytes(data, 6, 2)
        p = 8
        if version == 3:
            p += 1
        pad = (lambda n: (n + 7) // 8 * 8) if version == 1 else (lambda n: n)
        name = bytes(data[p:p + name_size]).split(b"\x00")[0].decode("utf-8")
        p += pad(name_size)
        dtype, _ = self._parse_datatype(data, p)
        p += pad(dt_size)
        shape = self._parse_dataspace(data[p:p + ds_size])
        p += pad(ds_size)
        raw = bytes(data[p:])
        return name, self._decode_values(raw, dtype, shape or ())

    def _decode_values(self, raw, dtype, shape):
        count = int(np.prod(shape)) if shape else 1
        if dtype.get("vlen"):
            vals = []
            for i in range(count):
                ln = self.u_bytes(raw, 16 * i, 4)
                heap = self.u_bytes(raw, 16 * i + 4, 8)
                idx = self.u_bytes(raw, 16 * i + 12, 4)
                payload = self._gheap_object(heap, idx)
                if dtype.get("vlen_string"):
                    vals.append(payload[:ln].decode("utf-8", "replace"))
                else:
                    vals.append(np.frombuffer(payload[: ln * dtype["base"]["np"].itemsize], dtype=dtype["base"]["np"]))
            if not shape:
                return vals[0]
            return np.array(vals, dtype=object).reshape(shape)
        npd = dtype["np"]
        arr = np.frombuffer(raw[: count * npd.itemsize], dtype=npd)
        if dtype.get("string"):
            vals = [v.split(b"\x00")[0].decode("utf-8", "replace") for v in arr.tolist()]
            return vals[0] if not shape else np.array(vals, dtype=object).reshape(shape)
        if dtype.get("bool"):
            arr = arr.astype(bool)
        arr = arr.reshape(shape) if shape else arr.reshape(())
        if not shape:
            return arr[()]
        return arr

    def _gheap_object(self, addr, index):
        addr += self.base
        objs = self._gheaps.get(addr)
        if objs is None:
            b = self.buf
            if b[addr:addr + 4] != b"GCOL":
                raise ValueError("Corrupt HDF5 file: global heap signature missing.")
            size = self.u(addr + 8, 8)
            objs = {}
            p = addr + 16
            end = addr + size
            while p + 16 <= end:
                idx = self.u(p, 2)
                osize = self.u(p + 8, 8)
                if idx == 0:
                    break
                objs[idx] = bytes(b[p + 16:p + 16 + osize])
                p += 16 + (osize + 7) // 8 * 8
            self._gheaps[addr] = objs
        return objs[index]

    def read_dataset(self, info):
        shape = info.get("shape")
        dtype = info["dtype"]
        if shape is None:
            return np.zeros((0,), dtype=dtype["np"])
        layout = info["layout"]
        npd = dtype["np"]
        count = int(np.prod(shape)) if shape else 1
        nbytes = count * npd.itemsize
        version = layout[0]
        if version == 3:
            cls = layout[1]
            if cls == 1:
                addr = self.u_bytes(layout, 2, 8)
                if addr == UNDEF:
                    raw = bytes(nbytes)
                else:
                    raw = self.buf[addr + self.base: addr + self.base + nbytes]
            elif cls == 0:
                size = self.u_bytes(layout, 2, 2)
                raw = layout[4:4 + size]
            elif cls == 2:
                rank = layout[2]
                btree = self.u_bytes(layout, 3, 8)
                chunk = [self.u_bytes(layout, 11 + 4 * i, 4) for i in range(rank)]
                raw = self._read_chunked(btree, chunk[:-1], shape, npd, info.get("filters") or [])
            else:
                raise NotImplementedError(f"HDF5 layout class {cls} is not supported.")
        elif version in (1, 2):
            rank = layout[1]
            cls = layout[2]
            p = 8
            addr = None
            if cls != 0:
                addr = self.u_bytes(layout, p, 8)
                p += 8
            dims = [self.u_bytes(layout, p + 4 * i, 4) for i in range(rank)]
            p += 4 * rank
            if cls == 1:
                raw = self.buf[addr + self.base: addr + self.base + nbytes]
            elif cls == 0:
                size = self.u_bytes(layout, p, 4)
                raw = layout[p + 4:p + 4 + size]
            else:
                raw = self._read_chunked(addr, dims[:-1], shape, npd, info.get("filters") or [])
        else:
            raise NotImplementedError(f"HDF5 data layout version {version} is not supported.")
        if isinstance(raw, np.ndarray):
            arr = raw
        else:
            arr = np.frombuffer(raw, dtype=npd, count=count)
        arr = arr.reshape(shape)
        if dtype.get("bool"):
            arr = arr.astype(bool)
        if dtype.get("string"):
            arr = np.array([v.split(b"\x00")[0].decode("utf-8", "replace") for v in arr.reshape(-1).tolist()], dtype=object).reshape(shape)
        if dtype.get("bfloat16"):
            import ml_dtypes

            arr = arr.view(ml_dtypes.bfloat16)
        if dtype.get("vlen"):
            arr = self._decode_values(bytes(raw), dtype, shape)
        return arr

    def _read_chunked(self, btree, chunk, shape, npd, filters):
        out = np.zeros(shape, dtype=npd)
        if btree == UNDEF:
            return out
        rank = len(shape)

        def walk(addr):
            b = self.buf
            if b[addr:addr + 4] != b"TREE":
                raise ValueError("Corrupt HDF5 file: chunk B-tree signature missing.")
            level = b[addr + 5]
            used = self.u(addr + 6, 2)
            p = addr + 24
            key_size = 8 + 8 * (rank + 1)
            for _ in range(used):
                csize = self.u(p, 4)
                fmask = self.u(p + 4, 4)
                offs = [self.u(p + 8 + 8 * i, 8) for i in range(rank)]
                child = self.u(p + key_size, 8) + self.base
                p += key_size + 8
                if level > 0:
                    walk(child)
                    continue
                raw = bytes(b[child:child + csize])
                for k, (fid, cd) in reversed(list(enumerate(filters))):
                    if fmask & (1 << k):
                        continue
                    if fid == 1:
                        raw = zlib.decompress(raw)
                    elif fid == 2:
                        es = cd[0] if cd else npd.itemsize
                        a = np.frombuffer(raw, dtype=np.uint8)
                        n = len(a) // es
                        raw = a[: n * es].reshape(es, n).T.tobytes() + a[n * es:].tobytes()
                    elif fid == 3:
                        raw = raw[:-4]
                    else:
                        raise NotImplementedError(f"HDF5 filter id {fid} is not supported.")
                block = np.frombuffer(raw, dtype=npd, count=int(np.prod(chunk))).reshape(chunk)
                sel_out = tuple(slice(o, min(o + c, s)) for o, c, s in zip(offs, chunk, shape))
                sel_in = tuple(slice(0, s.stop - s.start) for s in sel_out)
                out[sel_out] = block[sel_in]

        walk(btree + self.base)
        return out


class Dataset:
    def __init__(self, reader, addr, info, name):
        self._r, self._addr, self._info, self.name = reader, addr, info, name
        self.attrs = info["attrs"]

    @property
    def shape(self):
        return tuple(self._info.get("shape") or ())

    @property
    def dtype(self):
        d = self._info["dtype"]
        if d.get("bool"):
            return np.dtype(bool)
        return d["np"]

    def __array__(self, dtype=None, copy=None):
        a = self[()]
        return a.astype(dtype) if dtype is not None else a

    def __getitem__(self, key):
        arr = self._r.read_dataset(self._info)
        if self._info["dtype"].get("opaque") and self.attrs.get("dtype") == "bfloat16":
            import ml_dtypes

            arr = arr.view(np.uint16).view(ml_dtypes.bfloat16) if arr.dtype.itemsize == 2 else arr
        if key == () or key is Ellipsis:
            return arr
        return arr[key]

    def __len__(self):
        return self.shape[0]


class Group:
    def __init__(self, reader, addr, name="/", info=None):
        self._r, self._addr, self.name = reader, addr, name
        self._links = None
        self._info = info

    @property
    def attrs(self):
        if self._info is None:
            self._info = self._r.object_info(self._addr)
        return self._info["attrs"]

    def _get_links(self):
        if self._links is None:
            self._links = self._r.links(self._addr)
        return self._links

    def keys(self):
        return list(self._get_links().keys())

    def __iter__(self):
        return iter(self.keys())

    def __len__(self):
        return len(self._get_links())

    def __contains__(self, name):
        try:
            self[name]
            return True
        except KeyError:
            return False

    def items(self):
        return [(k, self[k]) for k in self.keys()]

    def values(self):
        return [self[k] for k in self.keys()]

    def get(self, name, default=None):
        try:
            return self[name]
        except KeyError:
            return default

    def __getitem__(self, path):
        node = self
        parts = [p for p in path.split("/") if p]
        if path.startswith("/") and self.name != "/":
            node = Group(self._r, self._r.root_header, "/")
        for i, part in enumerate(parts):
            if not isinstance(node, Group):
                raise KeyError(path)
            links = node._get_links()
            if part not in links:
                raise KeyError(f"Unable to open object '{path}' (component '{part}' not found)")
            addr = links[part]
            info = node._r.object_info(addr)
            full = (node.name.rstrip("/") + "/" + part)
            if info["kind"] == "dataset":
                node = Dataset(node._r, addr, info, full)
            else:
                node = Group(node._r, addr, full, info)
        return node

    def visititems(self, fn, _prefix=""):
        for k in self.keys():
            obj = self[k]
            name = f"{_prefix}{k}"
            r = fn(name, obj)
            if r is not None:
                return r
            if isinstance(obj, Group):
                r = obj.visititems(fn, name + "/")
                if r is not None:
                    return r


class File(Group):
    """Read-only view of an HDF5 file: ``File(path_or_bytes_or_fileobj)``."""

    def __init__(self, source, mode="r"):
        if mode != "r":
            raise ValueError("hdf5.File only reads; use hdf5.Writer to create files.")
        self._mmap = None
        if isinstance(source, (bytes, bytearray, memoryview)):
            buf = memoryview(source)
        elif isinstance(source, str) or hasattr(source, "__fspath__"):
            import mmap

            self._fh = open(source, "rb")
            try:
                self._mmap = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
                buf = memoryview(self._mmap)
            except ValueError:
                buf = memoryview(self._fh.read())
        else:
            buf = memoryview(source.read())
        reader = _Reader(buf)
        super().__init__(reader, reader.root_header, "/")

    def __bool__(self):
        """True while the file is open (h5py's convention; a Group would otherwise be falsy when it has no members)."""
        return not getattr(self, "_closed", False)

    def close(self):
        self._links = None
        self._closed = True
        if self._mmap is not None:
            try:
                self._r.buf.release()
                self._mmap.close()
                self._fh.close()
            except Exception:
                pass
            self._mmap = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


# ==================================================================================== writer
def _pad8(b):
    return b + b"\x00" * ((-len(b)) % 8)


def _datatype_message(dtype_name):
    """Datatype message bytes for a numpy dtype name / 'bfloat16' / 'bool' / 'vlen_str'."""
    def fixed(size, signed):
        return struct.pack("<B3BI", 0x10 | 0, 0x08 if signed else 0x00, 0, 0, size) + struct.pack("<HH", 0, size * 8)

    def flt(size, exp_loc, exp_size, mant_size, bias):
        return struct.pack("<B3BI", 0x10 | 1, 0x20, size * 8 - 1, 0, size) + struct.pack("<HHBBBBI", 0, size * 8, exp_loc, exp_size, 0, mant_size, bias)

    table = {
        "float16": lambda: flt(2, 10, 5, 10, 15), "float32": lambda: flt(4, 23, 8, 23, 127), "float64": lambda: flt(8, 52, 11, 52, 1023),
        "int8": lambda: fixed(1, True), "int16": lambda: fixed(2, True), "int32": lambda: fixed(4, True), "int64": lambda: fixed(8, True),
        "uint8": lambda: fixed(1, False), "uint16": lambda: fixed(2, False), "uint32": lambda: fixed(4, False), "uint64": lambda: fixed(8, False),
    }
    if dtype_name in table:
        return table[dtype_name]()
    if dtype_name == "bfloat16":
        # opaque, 2 bytes, empty tag (what h5py emits for a 2-byte void dtype)
        return struct.pack("<B3BI", 0x10 | 5, 0, 0, 0, 2)
    if dtype_name == "bool":
        base = fixed(1, True)
        names = _pad8(b"FALSE\x00") + _pad8(b"TRUE\x00")
        return struct.pack("<B3BI", 0x10 | 8, 2, 0, 0, 1) + base + names + bytes([0, 1])
    if dtype_name == "vlen_str":
        base = struct.pack("<B3BI", 0x10 | 3, 0x00, 0, 0, 1)
        return struct.pack("<B3BI", 0x10 | 9, 0x01, 0x01, 0, 16) + base
    if dtype_name.startswith("S"):
        return struct.pack("<B3BI", 0x10 | 3, 0x00, 0, 0, int(dtype_name[1:]))
    raise ValueError(f"Cannot store dtype {dtype_name} in an HDF5 file.")


def _dataspace_message(shape):
    if shape is None:
        shape = ()
    return struct.pack("<BBBB4x", 1, len(shape), 0, 0) + b"".join(struct.pack("<Q", d) for d in shape)


def _message(mtype, data, flags=0):
    data = _pad8(data)
    return struct.pack("<HHB3x", mtype, len(data), flags) + data


class _GroupNode:
    def __init__(self):
        self.children = {}
        self.attrs = {}


class _DatasetNode:
    def __init__(self, array, dtype_name):
        self.array = array
        self.dtype_name = dtype_name
        self.attrs = {}


class Writer:
    """Collects a tree of groups / datasets / attributes, then serialises it in one pass."""

    def __init__(self):
        self.root = _GroupNode()

    def _group(self, path, create=True):
        node = self.root
        for part in [p for p in path.split("/") if p]:
            nxt = node.children.get(part)
            if nxt is None:
                if not create:
                    raise KeyError(path)
                nxt = _GroupNode()
                node.children[part] = nxt
            if not isinstance(nxt, _GroupNode):
                raise ValueError(f"'{part}' in path '{path}' is a dataset, not a group.")
            node = nxt
        return node

    def create_group(self, path, attrs=None):
        g = self._group(path)
        if attrs:
            g.attrs.update(attrs)
        return g

    def create_dataset(self, path, array, attrs=None):
        parts = [p for p in path.split("/") if p]
        parent = self._group("/".join(parts[:-1]))
        arr = np.asarray(array)
        name = arr.dtype.name
        if name == "bfloat16":
            arr = arr.view(np.uint16)
            attrs = dict(attrs or {}, dtype="bfloat16")
        elif name == "bool":
            arr = arr.astype(np.int8)
        elif name.startswith("float8"):
            attrs = dict(attrs or {}, dtype=name)
            arr = arr.view(np.uint8)
            name = "uint8"
        elif arr.dtype.kind in "US":
            raise ValueError("String datasets are not supported by this writer.")
        if arr.dtype.byteorder == ">":
            arr = arr.astype(arr.dtype.newbyteorder("<"))
        node = _DatasetNode(arr if arr.ndim == 0 else np.ascontiguousarray(arr), name)
        if attrs:
            node.attrs.update(attrs)
        parent.children[parts[-1]] = node
        return node

    def set_attr(self, path, key, value):
        parts = [p for p in path.split("/") if p]
        node = self.root
        for p in parts:
            node = node.children[p]
        node.attrs[key] = value

    # ---- serialisation ------------------------------------------------------------------
    def tobytes(self):
        out = bytearray(96)

        def alloc(data, align=8):
            while len(out) % align:
                out.append(0)
            addr = len(out)
            out.extend(data)
            return addr

        gheap_objects = []   # (placeholder position in `out`, payload)

        def attribute_messages(attrs):
            msgs = []
            for key, value in attrs.items():
                name = key.encode("utf-8") + b"\x00"
                if isinstance(value, (str, bytes)):
                    payload = value.encode("utf-8") if isinstance(value, str) else value
                    dt = _datatype_message("vlen_str")
                    ds = _dataspace_message(())
                    data = struct.pack("<IQI", len(payload), 0, 0)
                    body = struct.pack("<BxHHH", 1, len(name), len(dt), len(ds)) + _pad8(name) + _pad8(dt) + _pad8(ds)
                    msgs.append(("vlen", body, data, payload))
                else:
                    arr = np.asarray(value)
                    if arr.dtype.kind in "UO" and arr.size and all(isinstance(v, (str, bytes)) for v in arr.reshape(-1).tolist()):
                        enc = [v.encode("utf-8") if isinstance(v, str) else v for v in arr.reshape(-1).tolist()]
                        arr = np.array(enc, dtype=f"S{max(1, max(len(e) for e in enc))}").reshape(arr.shape)
                    elif arr.dtype.kind in "UO" and arr.size == 0:
                        arr = np.zeros(arr.shape, dtype="S1")
                    if arr.dtype.kind == "S":
                        dt = _datatype_message(f"S{arr.dtype.itemsize}")
                        ds = _dataspace_message(arr.shape)
                        body = struct.pack("<BxHHH", 1, len(name), len(dt), len(ds)) + _pad8(name) + _pad8(dt) + _pad8(ds)
                        msgs.append(("plain", body, arr.tobytes(), None))
                        continue
                    dname = arr.dtype.name
                    if dname == "bool":
                        arr = arr.astype(np.int8)
                    dt = _datatype_message(dname)
                    ds = _dataspace_message(arr.shape)
                    body = struct.pack("<BxHHH", 1, len(name), len(dt), len(ds)) + _pad8(name) + _pad8(dt) + _pad8(ds)
                    msgs.append(("plain", body, arr.tobytes(), None))
            return msgs

        def write_object_header(messages, attrs):
            """messages: list of raw message bytes. Returns header address."""
            attr_msgs = attribute_messages(attrs)
            blobs = list(messages)
            fixups = []
            for kind, body, data, payload in attr_msgs:
                raw = _message(0x0C, body + data)
                if kind == "vlen":
                    fixups.append((len(b"".join(blobs)) + 8 + len(body), payload))
                blobs.append(raw)
            body_bytes = b"".join(blobs)
            header = struct.pack("<BxHII4x", 1, len(blobs), 1, len(body_bytes))
            addr = alloc(header + body_bytes)
            for off, payload in fixups:
                gheap_objects.append((addr + 16 + off, payload))
            return addr

        def write_dataset(node):
            arr = node.array
            data_addr = alloc(arr.tobytes()) if arr.size else UNDEF
            layout = struct.pack("<BBQQ", 3, 1, data_addr, arr.nbytes)
            fill = struct.pack("<BBBBI", 2, 2, 2, 1, 0)
            msgs = [
                _message(0x01, _dataspace_message(arr.shape)),
                _message(0x03, _datatype_message(node.dtype_name), flags=1),
                _message(0x05, fill, flags=1),
                _message(0x08, layout),
            ]
            return write_object_header(msgs, node.attrs)

        LEAF_K, INTERNAL_K = 4, 16

        def write_group(node):
            child_addrs = {}
            for name, child in node.children.items():
                child_addrs[name] = write_group(child) if isinstance(child, _GroupNode) else write_dataset(child)
            # local heap: offset 0 holds the empty string
            names = sorted(child_addrs, key=lambda s: s.encode("utf-8"))
            heap = bytearray(8)
            offsets = {}
            for n in names:
                offsets[n] = len(heap)
                heap.extend(_pad8(n.encode("utf-8") + b"\x00"))
            free_off = len(heap)
            # keep a free block at the end, as libhdf5 does (>= 16 bytes: next-free + size)
            heap.extend(struct.pack("<QQ", 1, 16))
            heap_data_addr = alloc(bytes(heap))
            heap_addr = alloc(b"HEAP" + struct.pack("<B3xQQQ", 0, len(heap), free_off, heap_data_addr))
            # symbol nodes
            per = 2 * LEAF_K
            snods = []
            for i in range(0, max(len(names), 1), per):
                chunk = names[i:i + per]
                body = bytearray(b"SNOD" + struct.pack("<BxH", 1, len(chunk)))
                for n in chunk:
                    child = node.children[n]
                    if isinstance(child, _GroupNode):
                        body.extend(struct.pack("<QQII", offsets[n], child_addrs[n], 1, 0) + struct.pack("<QQ", *child._btree_heap))
                    else:
                        body.extend(struct.pack("<QQII16x", offsets[n], child_addrs[n], 0, 0))
                body.extend(bytes(8 + per * 40 - len(body)))
                last = offsets[chunk[-1]] if chunk else 0
                snods.append((alloc(bytes(body)), last))
            # B-tree levels
            level = 0
            entries = snods
            while True:
                per_node = 2 * INTERNAL_K
                groups = [entries[i:i + per_node] for i in range(0, len(entries), per_node)]
                node_size = 24 + (2 * per_node + 1) * 8
                addrs = []
                base = alloc(bytes(node_size * len(groups)))
                prev_key = 0
                new_entries = []
                for gi, grp in enumerate(groups):
                    addr = base + gi * node_size
                    left = base + (gi - 1) * node_size if gi > 0 else UNDEF
                    right = base + (gi + 1) * node_size if gi + 1 < len(groups) else UNDEF
                    body = bytearray(b"TREE" + struct.pack("<BBHQQ", 0, level, len(grp), left, right))
                    body.extend(struct.pack("<Q", prev_key))
                    for child_addr, last_key in grp:
                        body.extend(struct.pack("<QQ", child_addr, last_key))
                        prev_key = last_key
                    body.extend(bytes(node_size - len(body)))
                    out[addr:addr + node_size] = body
                    new_entries.append((addr, grp[-1][1]))
                entries = new_entries
                if len(entries) == 1:
                    break
                level += 1
            btree_addr = entries[0][0]
            node._btree_heap = (btree_addr, heap_addr)
            stab = _message(0x11, struct.pack("<QQ", btree_addr, heap_addr))
            return write_object_header([stab], node.attrs)

        root_addr = write_group(self.root)
        # global heap collection(s) for variable-length strings
        if gheap_objects:
            MAX = 60000
            batch, batches, size = [], [], 0
            for item in gheap_objects:
                need = 16 + (len(item[1]) + 7) // 8 * 8
                if batch and (size + need > MAX or len(batch) >= 65000):
                    batches.append(batch)
                    batch, size = [], 0
                batch.append(item)
                size += need
            batches.append(batch)
            for batch in batches:
                body = bytearray()
                for i, (_, payload) in enumerate(batch, start=1):
                    body.extend(struct.pack("<HH4xQ", i, 1, len(payload)) + _pad8(payload))
                total = max(4096, 16 + len(body) + 16)
                free = total - 16 - len(body)
                body.extend(struct.pack("<HH4xQ", 0, 0, free - 16) + bytes(free - 16))
                addr = alloc(b"GCOL" + struct.pack("<B3xQ", 1, total) + bytes(body))
                for i, (pos, payload) in enumerate(batch, start=1):
                    out[pos:pos + 16] = struct.pack("<IQI", len(payload), addr, i)
        while len(out) % 8:
            out.append(0)
        eof = len(out)
        sb = SIGNATURE + struct.pack("<BBBBBBBBHHI", 0, 0, 0, 0, 0, 8, 8, 0, LEAF_K, INTERNAL_K, 0)
        sb += struct.pack("<QQQQ", 0, UNDEF, eof, UNDEF)
        sb += struct.pack("<QQII", 0, root_addr, 1, 0) + struct.pack("<QQ", *self.root._btree_heap)
        out[0:96] = sb
        return bytes(out)

    def save(self, target):
        data = self.tobytes()
        if isinstance(target, str) or hasattr(target, "__fspath__"):
            with open(target, "wb") as f:
                f.write(data)
        else:
            target.write(data)
