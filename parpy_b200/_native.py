"""ctypes binding of ``libparpy_b200.so`` (the C ABI declared in
``include/parpy_b200.h``).

The library is built in-tree by :mod:`parpy_b200.csrc.build`. There is no CPU
or PyTorch fallback: if the shared object is missing or cannot be loaded,
:func:`lib` raises and every operator of the package fails loudly.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libparpy_b200.so")

_lock = threading.Lock()
_lib = None

c_f32 = ctypes.c_float
c_f64 = ctypes.c_double
c_i32 = ctypes.c_int32
c_i64 = ctypes.c_int64
c_u32 = ctypes.c_uint32
c_ptr = ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/parpy_b200.h one to one.
SIGNATURES = {
    "parpy_init": (None, [c_i64]),
    "parpy_sync": (c_i32, []),
    "parpy_alloc_buffer": (c_ptr, [c_i64]),
    "parpy_memcpy": (c_i32, [c_ptr, c_ptr, c_i64, c_i64]),
    "parpy_memset": (c_i32, [c_ptr, c_i64, ctypes.c_int8]),
    "parpy_free_buffer": (c_i32, [c_ptr]),
    "parpy_get_error_message": (ctypes.c_char_p, []),
    "parpy_b200_device_summary": (c_i32, [c_ptr, c_ptr, c_ptr]),
    "forward_kernel": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_f32, c_ptr, c_ptr, c_ptr, c_ptr,
                               c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "forward_kernel_scratch_first": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_f32, c_ptr, c_ptr,
                                             c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "parpy_b200_forward": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_f32, c_ptr, c_ptr, c_ptr, c_ptr,
                                   c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_u32, c_ptr]),
    "parpy_b200_forward_ex": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_i64, c_f32, c_ptr, c_ptr, c_ptr, c_ptr,
                                      c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_u32, c_ptr]),
    "parpy_b200_forward_schedule": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr]),
    "parpy_b200_forward_noalloc": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_f32, c_ptr, c_ptr, c_ptr, c_ptr,
                                           c_i64, c_i64, c_ptr, c_ptr]),
    "parpy_b200_forward_plan": (c_i32, [c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_ptr]),
    "parpy_b200_forward_status": (c_i32, [c_ptr]),
    "softmax": (c_i32, [c_ptr, c_i64, c_i64, c_ptr]),
    "parpy_b200_softmax": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr]),
    "parpy_b200_reduce_rows": (c_i32, [c_i32, c_ptr, c_ptr, c_i64, c_i64, c_ptr]),
    "parpy_b200_sum_max": (c_i32, [c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "spmv_row": (c_i32, [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr]),
    "parpy_b200_spmv": (c_i32, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "parpy_sddmm_decompress_csr": (c_i32, [c_ptr, c_ptr, c_i64]),
    "parpy_b200_sddmm_decompress_csr": (c_i32, [c_ptr, c_ptr, c_i64, c_ptr]),
    "parpy_b200_sddmm_csr": (c_i32, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i64,
                                     c_i64, c_i64, c_f64, c_f64, c_ptr]),
    "parpy_b200_sddmm_coo": (c_i32, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64,
                                     c_f64, c_f64, c_ptr]),
    "normalize_rows": (c_i32, [c_ptr, c_i64, c_i64]),
    "parpy_b200_normalize_rows": (c_i32, [c_ptr, c_i64, c_i64, c_ptr]),
    "parpy_b200_sum_exp_rows": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr]),
    "spmm_cell": (c_i32, [c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr]),
    "parpy_b200_spmm": (c_i32, [c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_ptr]),
    "parpy_b200_hmm_prepare_tables": (c_i32, [c_ptr, c_ptr, c_ptr, c_i32, c_i32, c_i64, c_ptr, c_ptr, c_ptr,
                                              c_ptr, c_ptr]),
    "parpy_b200_hmm_pad_signals": (c_i32, [c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_ptr]),
    "parpy_b200_viterbi": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_f32, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i64,
                                   c_i64, c_i64, c_ptr, c_i64, c_ptr]),
    "parpy_b200_viterbi_ex": (c_i32, [c_f32, c_ptr, c_i64, c_ptr, c_i64, c_f32, c_ptr, c_ptr, c_ptr, c_ptr, c_i64,
                                      c_i64, c_i64, c_i64, c_ptr, c_i64, c_ptr]),
    "parpy_b200_viterbi_status": (c_i32, [c_ptr]),
    "parpy_b200_viterbi_wait_probe": (c_i32, [c_i32, c_ptr]),
    "parpy_b200_forward_wait_probe": (c_i32, [c_i32, c_ptr]),
}

REDUCE_SUM, REDUCE_PROD, REDUCE_MAX, REDUCE_MIN = 0, 1, 2, 3

NOALLOC_MAX_SEQUENCES = 16384

FWD_AUTO = 0
FWD_STREAMING = 1
FWD_WRITE_ALPHA = 2
FWD_FIVE_TERM = 4
FWD_SCALED = 8
FWD_LOG_SPACE = 16


class NativeLibraryMissing(RuntimeError):
    pass


def lib():
    """Returns the loaded library, loading it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise NativeLibraryMissing(
                    f"{LIB_PATH} is missing: build it with "
                    "`python -m parpy_b200.csrc.build` (needs nvcc); "
                    "parpy_b200 has no CPU fallback")
            handle = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype = res
                fn.argtypes = args
            _lib = handle
    return _lib


def error_message():
    return lib().parpy_get_error_message().decode("ascii", "replace")


def check(status, what="native call"):
    """Raises RuntimeError with the library's error text on a non-zero status
    (the reference's convention, python/parpy/compile.py:178-182)."""
    if status != 0:
        raise RuntimeError(f"{what}: {error_message()} (code={status})")
