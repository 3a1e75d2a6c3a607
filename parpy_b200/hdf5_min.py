"""Minimal pure-Python reader for the subset of HDF5 the HMM model and signal
files use, for environments without h5py / libhdf5 (the reference's loaders,
benchmarks/forward.py:40-55, use h5py). It understands exactly what
the nanopore model / signal files need: superblock version 0, version-1 object
headers (with continuation blocks), old-style groups (symbol table message ->
v1 B-tree -> symbol nodes -> local heap), simple dataspaces, fixed-point and
IEEE float datatypes, contiguous layout, and single-level chunked layout with
the shuffle + deflate filter pair. Anything else raises ``NotImplementedError``.

Layout facts follow the public "HDF5 File Format Specification Version 2.0".
"""
import struct
import zlib

import numpy as np

_SIG = b"\x89HDF\r\n\x1a\n"
_UNDEF = 0xFFFFFFFFFFFFFFFF


class _Obj:
    def __init__(self):
        self.msgs = []  # (type, bytes)


class H5File:
    def __init__(self, path):
        with open(path, "rb") as f:
            self.b = f.read()
        if self.b[:8] != _SIG:
            raise ValueError("not an HDF5 file")
        ver = self.b[8]
        if ver != 0:
            raise NotImplementedError(f"superblock version {ver}")
        so, sl = self.b[13], self.b[14]
        if (so, sl) != (8, 8):
            raise NotImplementedError("only 8-byte offsets/lengths")
        # 8 sig + 8 version bytes + 2+2 K values + 4 flags = 24, then 4 addresses
        self.base = struct.unpack_from("<Q", self.b, 24)[0]
        root_entry = 24 + 4 * 8
        self.root_addr = struct.unpack_from("<Q", self.b, root_entry + 8)[0]
        self.root = Group(self, self.root_addr)

    # -- object headers ----------------------------------------------------
    def read_header(self, addr):
        b = self.b
        ver, _, nmsg, _refc, hsize = struct.unpack_from("<BBHII", b, addr)
        if ver != 1:
            raise NotImplementedError(f"object header version {ver}")
        obj = _Obj()
        blocks = [(addr + 16, hsize)]
        while blocks and len(obj.msgs) < nmsg:
            pos, size = blocks.pop(0)
            end = pos + size
            while pos + 8 <= end and len(obj.msgs) < nmsg:
                mtype, msize, _flags = struct.unpack_from("<HHB", b, pos)
                data = b[pos + 8:pos + 8 + msize]
                pos += 8 + msize
                if mtype == 0x10:
                    coff, clen = struct.unpack_from("<QQ", data, 0)
                    blocks.append((coff, clen))
                obj.msgs.append((mtype, data))
        return obj

    def __getitem__(self, key):
        return self.root[key]

    def keys(self):
        return self.root.keys()


def _parse_dataspace(d):
    ver, rank, flags = d[0], d[1], d[2]
    if ver == 1:
        off = 8
    elif ver == 2:
        off = 4
        if d[3] == 2:  # null dataspace: no elements
            return None
    else:
        raise NotImplementedError(f"dataspace version {ver}")
    return tuple(struct.unpack_from("<Q", d, off + 8 * i)[0] for i in range(rank))


def _parse_datatype(d):
    cls = d[0] & 0x0F
    bits0 = d[1]
    size = struct.unpack_from("<I", d, 4)[0]
    if cls in (0, 1) and (bits0 & 1):
        raise NotImplementedError("big-endian data")
    if cls == 0:
        signed = bool(bits0 & 0x08)
        return np.dtype(("<i" if signed else "<u") + str(size))
    if cls == 1:
        return np.dtype("<f" + str(size))
    if cls == 3:
        return np.dtype("S" + str(size))
    raise NotImplementedError(f"datatype class {cls}")


def _pad8(n):
    return (n + 7) & ~7


def _parse_attrs(obj):
    out = {}
    for mtype, d in obj.msgs:
        if mtype != 0x0C:
            continue
        ver = d[0]
        if ver != 1:
            raise NotImplementedError(f"attribute message version {ver}")
        nsz, tsz, ssz = struct.unpack_from("<HHH", d, 2)
        pos = 8
        name = d[pos:pos + nsz].split(b"\0")[0].decode()
        pos += _pad8(nsz)
        try:
            dt = _parse_datatype(d[pos:pos + tsz])
        except NotImplementedError:
            out[name] = None  # e.g. variable-length strings: not needed here
            continue
        pos += _pad8(tsz)
        shape = _parse_dataspace(d[pos:pos + ssz])
        pos += _pad8(ssz)
        if shape is None:
            out[name] = None
            continue
        n = int(np.prod(shape)) if shape else 1
        arr = np.frombuffer(d, dtype=dt, count=n, offset=pos).reshape(shape)
        out[name] = arr[()] if shape == () else arr.copy()
    return out


class Group:
    def __init__(self, f, addr):
        self.f = f
        self.obj = f.read_header(addr)
        self._links = None
        self.attrs = _parse_attrs(self.obj)

    def _load(self):
        if self._links is not None:
            return
        self._links = {}
        stab = [d for t, d in self.obj.msgs if t == 0x11]
        if not stab:
            raise NotImplementedError("group without a symbol table message")
        btree, heap = struct.unpack_from("<QQ", stab[0], 0)
        b = self.f.b
        if b[heap:heap + 4] != b"HEAP":
            raise ValueError("bad local heap")
        heap_data = struct.unpack_from("<Q", b, heap + 8 + 16)[0]
        self._walk(btree, heap_data)

    def _walk(self, node, heap_data):
        b = self.f.b
        if b[node:node + 4] != b"TREE":
            raise ValueError("bad B-tree node")
        _ntype, level, used = struct.unpack_from("<BBH", b, node + 4)
        pos = node + 8 + 16
        for i in range(used):
            child = struct.unpack_from("<Q", b, pos + 8)[0]
            pos += 16
            if level > 0:
                self._walk(child, heap_data)
            else:
                self._snod(child, heap_data)

    def _snod(self, addr, heap_data):
        b = self.f.b
        if b[addr:addr + 4] != b"SNOD":
            raise ValueError("bad symbol node")
        nsym = struct.unpack_from("<H", b, addr + 6)[0]
        pos = addr + 8
        for _ in range(nsym):
            name_off, ohdr = struct.unpack_from("<QQ", b, pos)
            pos += 40
            s = heap_data + name_off
            e = b.index(b"\0", s)
            self._links[b[s:e].decode()] = ohdr

    def keys(self):
        self._load()
        return sorted(self._links)

    def __getitem__(self, key):
        self._load()
        node = self
        parts = [p for p in key.split("/") if p]
        addr = node._links[parts[0]]
        obj = self.f.read_header(addr)
        is_group = any(t == 0x11 for t, _ in obj.msgs)
        child = Group(self.f, addr) if is_group else Dataset(self.f, addr)
        if len(parts) > 1:
            return child["/".join(parts[1:])]
        return child


class Dataset:
    def __init__(self, f, addr):
        self.f = f
        self.obj = f.read_header(addr)
        self.attrs = _parse_attrs(self.obj)
        m = dict((t, d) for t, d in self.obj.msgs)
        self.shape = _parse_dataspace(m[0x01])
        self.dtype = _parse_datatype(m[0x03])
        self.layout = m[0x08]
        self.filters = self._parse_filters(m.get(0x0B))

    @staticmethod
    def _parse_filters(d):
        if d is None:
            return []
        ver, nf = d[0], d[1]
        if ver != 1:
            raise NotImplementedError(f"filter pipeline version {ver}")
        pos = 8
        out = []
        for _ in range(nf):
            fid, nlen, _flags, ncd = struct.unpack_from("<HHHH", d, pos)
            pos += 8 + _pad8(nlen)
            cd = struct.unpack_from("<" + "I" * ncd, d, pos)
            pos += 4 * ncd + (4 if ncd % 2 else 0)
            out.append((fid, cd))
        return out

    def read(self):
        d = self.layout
        ver, cls = d[0], d[1]
        if ver != 3:
            raise NotImplementedError(f"layout version {ver}")
        n = int(np.prod(self.shape)) if self.shape else 1
        if cls == 1:
            addr, _size = struct.unpack_from("<QQ", d, 2)
            return np.frombuffer(self.f.b, dtype=self.dtype, count=n,
                                 offset=addr).reshape(self.shape).copy()
        if cls == 2:
            ndim = d[2]
            btree = struct.unpack_from("<Q", d, 3)[0]
            cdims = struct.unpack_from("<" + "I" * ndim, d, 11)
            if len(self.shape) != 1:
                raise NotImplementedError("chunked data with rank != 1")
            out = np.empty(self.shape, dtype=self.dtype)
            self._chunks(btree, ndim, cdims, out)
            return out
        raise NotImplementedError(f"layout class {cls}")

    def _chunks(self, node, ndim, cdims, out):
        b = self.f.b
        if b[node:node + 4] != b"TREE":
            raise ValueError("bad chunk B-tree node")
        ntype, level, used = struct.unpack_from("<BBH", b, node + 4)
        if ntype != 1:
            raise ValueError("not a chunk B-tree")
        pos = node + 8 + 16
        keysz = 8 + 8 * ndim
        for _ in range(used):
            csize, _mask = struct.unpack_from("<II", b, pos)
            offs = struct.unpack_from("<" + "Q" * ndim, b, pos + 8)
            child = struct.unpack_from("<Q", b, pos + keysz)[0]
            pos += keysz + 8
            if level > 0:
                self._chunks(child, ndim, cdims, out)
                continue
            raw = b[child:child + csize]
            for fid, cd in reversed(self.filters):
                if fid == 1:
                    raw = zlib.decompress(raw)
                elif fid == 2:
                    es = cd[0]
                    a = np.frombuffer(raw, dtype=np.uint8)
                    raw = a.reshape(es, -1).T.tobytes()
                else:
                    raise NotImplementedError(f"filter id {fid}")
            chunk = np.frombuffer(raw, dtype=self.dtype, count=cdims[0])
            lo = offs[0]
            hi = min(lo + cdims[0], out.shape[0])
            out[lo:hi] = chunk[:hi - lo]
