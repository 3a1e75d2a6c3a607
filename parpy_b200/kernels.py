"""The reduction-heavy functions of the reference's tests and benchmarks, bound
to their native kernels under the reference's names and signatures: ``softmax``
(test/test_softmax.py:11-26), the twelve row / axis / full reductions
(test/test_reduce.py:12-70), ``spmv_row`` (test/test_spmv.py:12-18) and the
SDDMM kernels (benchmarks/sddmm.py:21-41,63-70). All take ``opts=`` and write
their outputs in place. ``sum_max`` is this package's fused one-pass sum + max
of a long vector."""
from . import jit


@jit
def softmax(x, N, M, out):
    """out[i,:] = softmax(x[i,:])"""


def _bind_reduce(name):
    def template(x, out, N):
        pass
    template.__name__ = name
    template.__qualname__ = name
    return jit(template)


sum_rows, prod_rows, max_rows, min_rows = (_bind_reduce(f"{o}_rows") for o in ("sum", "prod", "max", "min"))
sum_axis, prod_axis, max_axis, min_axis = (_bind_reduce(f"{o}_axis") for o in ("sum", "prod", "max", "min"))
sum_2d, prod_2d, max_2d, min_2d = (_bind_reduce(f"{o}_2d") for o in ("sum", "prod", "max", "min"))


@jit
def spmv_row(A, x, y):
    """y[row] += sum(A.values[i] * x[A.cols[i]]) over the row's non-zeros"""


@jit
def parpy_sddmm_decompress_csr(C_crows, C_rows, N):
    """C_rows[i] = row of non-zero i"""


@jit
def parpy_sddmm_csr_kernel(A, B, C, D, N, alpha, beta):
    """D[i] = alpha * dot(A[row_i,:], B[:,col_i]) + beta * C.values[i]; fills C.rows"""


@jit
def parpy_sddmm_coo_kernel(A, B, C, D, alpha, beta):
    """D[i] = alpha * dot(A[C.rows[i],:], B[:,C.cols[i]]) + beta * C.values[i]"""


def sum_max(x):
    """(sum, max) of a float32 CUDA tensor of any shape in one pass over it;
    returns a 2-element CUDA tensor."""
    import ctypes
    import torch
    from . import _native
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
        raise TypeError("sum_max expects a contiguous float32 CUDA tensor")
    out = torch.empty(2, dtype=torch.float32, device=x.device)
    P = ctypes.c_void_p
    rc = _native.lib().parpy_b200_sum_max(P(x.data_ptr()), x.numel(), P(out.data_ptr()),
                                          P(out.data_ptr() + 4), P(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "sum_max")
    return out


@jit
def normalize_rows(t, nrows, ncols):
    """t[i,:] /= sum(t[i,:]), in place"""


@jit
def sum_exp_3d(x, N, M, out):
    """x = exp(x) in place; out[i,j] = sum(x[i,j,:])"""


@jit
def spmm_cell(A, B, C):
    """C[i,j] += sum over row i's non-zeros of A.values[a] * B.values[A.cols[a], j]"""
