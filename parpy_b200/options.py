"""Value types of the call surface: element types, loop-parallelism hints and
compile options. They mirror the reference's pyo3 classes so that call sites
written against it run unchanged (src/par.rs:9-68, src/option.rs:8-131,
src/buffer.rs:17-128). Nothing here compiles anything: the kernels are prebuilt,
so most options are accepted and recorded, and only ``backend`` and the
package's own ``b200`` dictionary change behaviour.
"""
import ctypes
import enum

import numpy as np

DEFAULT_TPB = 1024


class CompileBackend(enum.Enum):
    Auto = 0
    Cuda = 1
    Metal = 2


class Target(enum.Enum):
    Host = 0
    Device = 1


class ElemSize(enum.Enum):
    """Scalar element types, named as in the reference (src/buffer.rs:17-30)."""
    Bool = "b1"
    I8 = "i1"
    I16 = "i2"
    I32 = "i4"
    I64 = "i8"
    U8 = "u1"
    U16 = "u2"
    U32 = "u4"
    U64 = "u8"
    F16 = "f2"
    F32 = "f4"
    F64 = "f8"

    def __str__(self):
        return self.value

    def size(self):
        return int(self.value[1])

    def is_integer(self):
        return self.value[0] in "iu"

    def is_signed_integer(self):
        return self.value[0] == "i"

    def is_unsigned_integer(self):
        return self.value[0] == "u"

    def is_floating_point(self):
        return self.value[0] == "f"

    def to_numpy(self):
        return {"b1": np.bool_, "i1": np.int8, "i2": np.int16, "i4": np.int32, "i8": np.int64,
                "u1": np.uint8, "u2": np.uint16, "u4": np.uint32, "u8": np.uint64,
                "f2": np.float16, "f4": np.float32, "f8": np.float64}[self.value]

    def to_torch(self):
        # Unsigned 16/32/64-bit map to the signed torch dtype of the same width,
        # as in the reference (src/buffer.rs:93-109).
        import torch
        return {"b1": torch.bool, "i1": torch.int8, "i2": torch.int16, "i4": torch.int32,
                "i8": torch.int64, "u1": torch.uint8, "u2": torch.int16, "u4": torch.int32,
                "u8": torch.int64, "f2": torch.float16, "f4": torch.float32,
                "f8": torch.float64}[self.value]

    def to_ctype(self):
        return {"b1": ctypes.c_bool, "i1": ctypes.c_int8, "i2": ctypes.c_int16,
                "i4": ctypes.c_int32, "i8": ctypes.c_int64, "u1": ctypes.c_uint8,
                "u2": ctypes.c_uint16, "u4": ctypes.c_uint32, "u8": ctypes.c_uint64,
                "f2": ctypes.c_uint16, "f4": ctypes.c_float, "f8": ctypes.c_double}[self.value]


class DataType:
    """An array-interface typestr (``'<f4'``) with its element type."""

    def __init__(self, typestr):
        if isinstance(typestr, DataType):
            typestr = str(typestr)
        if len(typestr) != 3 or typestr[0] not in "<|=":
            raise RuntimeError(f"Unsupported array typestr {typestr!r}")
        try:
            self.sz = ElemSize(typestr[1:])
        except ValueError:
            raise RuntimeError(f"Unknown type identifier {typestr[1:]}")
        self.typestr = typestr

    @staticmethod
    def from_elem_size(sz):
        return DataType(("|" if sz.size() == 1 else "<") + sz.value)

    def __str__(self):
        return self.typestr

    def __repr__(self):
        return f"DataType({self.typestr!r})"

    def __eq__(self, other):
        return isinstance(other, DataType) and other.sz == self.sz

    def __hash__(self):
        return hash(self.sz)

    def size(self):
        return self.sz.size()

    def is_integer(self):
        return self.sz.is_integer()

    def is_floating_point(self):
        return self.sz.is_floating_point()

    def to_numpy(self):
        return self.sz.to_numpy()

    def to_torch(self):
        return self.sz.to_torch()

    def to_ctype(self):
        return self.sz.to_ctype()


class ExtType:
    """Pointer-to-element type used by external declarations (types.pointer)."""

    def __init__(self, elem):
        self.elem = elem

    @staticmethod
    def Pointer(elem):
        return ExtType(elem)

    def __eq__(self, other):
        return isinstance(other, ExtType) and other.elem == self.elem

    def __hash__(self):
        return hash(("ptr", self.elem))


class LoopPar:
    """Parallelism hint attached to a label (src/par.rs:9-68). Immutable:
    every modifier returns a new object."""

    def __init__(self, nthreads=0, reduction=False, tpb=DEFAULT_TPB):
        self.nthreads = int(nthreads)
        self.reduction = bool(reduction)
        self._tpb = int(tpb)

    def __repr__(self):
        return (f"LoopPar {{ nthreads: {self.nthreads}, reduction: "
                f"{str(self.reduction).lower()}, tpb: {self._tpb} }}")

    __str__ = __repr__

    def __eq__(self, other):
        return (isinstance(other, LoopPar) and self.nthreads == other.nthreads and
                self.reduction == other.reduction and self._tpb == other._tpb)

    def is_parallel(self):
        return self.nthreads > 0

    def threads(self, nthreads):
        if self.nthreads != 0:
            raise RuntimeError("The number of threads can only be set once")
        return LoopPar(int(nthreads), self.reduction, self._tpb)

    def reduce(self):
        return LoopPar(self.nthreads, True, self._tpb)

    def tpb(self, tpb):
        tpb = int(tpb)
        if tpb <= 0 or tpb % 32 != 0:
            raise RuntimeError("The number of threads per block must be a positive "
                               "integer divisible by 32.")
        return LoopPar(self.nthreads, self.reduction, tpb)


class CompileOptions:
    """Options object passed as ``opts=`` (src/option.rs:14-131). Attribute
    names and defaults are the reference's; ``b200`` is this package's own
    extension: a dict of per-operator switches, e.g.
    ``{"forward": "five_term", "write_alpha": True}``."""

    def __init__(self):
        self.parallelize = {}
        self.verbose_backend_resolution = False
        self.debug_print = False
        self.write_output = False
        self.backend = CompileBackend.Auto
        self.use_cuda_thread_block_clusters = False
        self._max_thread_blocks_per_cluster = 8
        self.use_cuda_graphs = False
        self._force_int_size = None
        self._force_float_size = None
        self.includes = []
        self.libs = []
        self.extra_flags = []
        self.b200 = {}

    @property
    def max_thread_blocks_per_cluster(self):
        return self._max_thread_blocks_per_cluster

    @max_thread_blocks_per_cluster.setter
    def max_thread_blocks_per_cluster(self, n):
        if n > 0 and (n & (n - 1)) == 0:
            self._max_thread_blocks_per_cluster = int(n)
        else:
            raise RuntimeError("The number of thread blocks per cluster must be a power of two.")

    @property
    def force_int_size(self):
        return self._force_int_size

    @force_int_size.setter
    def force_int_size(self, sz):
        if not (isinstance(sz, ElemSize) and sz.is_integer()):
            raise RuntimeError("Cannot use a non integer type for integer scalars.")
        self._force_int_size = sz

    @property
    def force_float_size(self):
        return self._force_float_size

    @force_float_size.setter
    def force_float_size(self, sz):
        if not (isinstance(sz, ElemSize) and sz.is_floating_point()):
            raise RuntimeError("Cannot use a non floating-point type for floating-point scalars.")
        self._force_float_size = sz

    def __str__(self):
        par = ", ".join(f"{k!r}: {v}" for k, v in sorted(self.parallelize.items()))
        return (f"CompileOptions {{ parallelize: {{{par}}}, backend: {self.backend.name}, "
                f"use_cuda_thread_block_clusters: {self.use_cuda_thread_block_clusters}, "
                f"max_thread_blocks_per_cluster: {self._max_thread_blocks_per_cluster}, "
                f"use_cuda_graphs: {self.use_cuda_graphs}, b200: {self.b200} }}")


def par(p):
    """Default options carrying the given label -> LoopPar mapping
    (src/option.rs:133-139)."""
    if not isinstance(p, dict):
        raise TypeError("par expects a dict mapping labels to LoopPar objects")
    for k, v in p.items():
        if not isinstance(k, str) or not isinstance(v, LoopPar):
            raise TypeError("par expects a dict mapping str labels to LoopPar objects")
    opts = CompileOptions()
    opts.parallelize = dict(p)
    return opts
