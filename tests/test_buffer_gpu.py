"""Device buffers, written the way the reference's test/test_buffer.py is (CUDA backend only)."""
import numpy as np
import pytest
import torch

import parpy_b200 as parpy

pytestmark = pytest.mark.gpu
CUDA = parpy.CompileBackend.Cuda


def test_empty_zeros_and_like():
    shape = (20, 10, 32)
    b = parpy.buffer.empty(shape, parpy.types.F32, CUDA)
    assert b.numpy().shape == shape
    b2 = parpy.buffer.empty_like(b)
    assert b.shape == b2.shape and b._get_ptr() != b2._get_ptr()
    z = parpy.buffer.zeros(shape, parpy.types.F32, CUDA)
    assert np.allclose(z.numpy(), np.zeros(shape, dtype=np.float32))
    z2 = parpy.buffer.zeros_like(b)
    assert z2.shape == shape and z2._get_ptr() != b._get_ptr() and not z2.numpy().any()


def test_from_numpy_scalars_size_and_views():
    a = np.ndarray((20, 10, 32), dtype=np.float32)
    b = parpy.buffer.from_array(a, CUDA)
    assert b.shape == a.shape and b.src is a
    assert b.dtype == parpy.buffer.DataType.from_elem_size(parpy.types.F32)
    assert float(parpy.buffer.from_array(np.array(2.5, dtype=np.float32), CUDA)) == 2.5
    assert int(parpy.buffer.from_array(np.array(2, dtype=np.int32), CUDA)) == 2
    assert bool(parpy.buffer.from_array(torch.tensor(True, dtype=torch.bool), CUDA))
    i16 = parpy.buffer.zeros((20, 10, 32), parpy.types.I16, CUDA)
    assert parpy.types.I16.size() == 2 and i16.size() == 20 * 10 * 32 * 2
    assert i16.numpy().dtype == np.int16 and i16.torch().dtype == torch.int16
    assert i16.torch().device == torch.device("cuda", torch.cuda.current_device())


def test_reshape_refcount_and_type_views():
    shape = (20, 10, 32)
    b1 = parpy.buffer.zeros(shape, parpy.types.F32, CUDA)
    assert b1.refcount[0] == 1
    b2 = b1.reshape(200, 32)
    assert b1.shape == shape and b2.shape == (200, 32)
    assert b1.refcount[0] == 2 and b2.refcount[0] == 2
    del b2
    assert b1.refcount[0] == 1
    with pytest.raises(ValueError, match="Cannot reshape buffer of shape.*to.*"):
        b1.reshape(20, 10, 32, 2)
    i = parpy.buffer.zeros(shape, parpy.types.I32, CUDA)
    u = i.with_type(parpy.types.U32)
    assert u.dtype == parpy.buffer.DataType.from_elem_size(parpy.types.U32) and i._get_ptr() == u._get_ptr()
    f = i.with_type(parpy.types.F64)
    assert f.dtype == parpy.buffer.DataType.from_elem_size(parpy.types.F64) and i._get_ptr() != f._get_ptr()


def test_round_trip_and_write_back_on_release():
    a = np.random.randn(20, 10, 32)
    b = parpy.buffer.from_array(a, CUDA)
    assert np.allclose(a, b.numpy())
    # a buffer staged from a host array writes the device contents back when it goes
    host = np.zeros(8, dtype=np.float32)
    buf = parpy.buffer.from_array(host, CUDA)
    buf.torch().fill_(3.0)
    del buf
    assert np.array_equal(host, np.full(8, 3.0, dtype=np.float32))
    parpy.sync(CUDA)


class ForeignDeviceArray:
    """A device array that is not a torch tensor: only ``__cuda_array_interface__``
    (version 3), the way a CuPy array presents itself (test/test_cupy.py). Backed
    by a torch allocation that it keeps alive."""

    def __init__(self, tensor, readonly=False, strides=None):
        self._keep = tensor
        typestr = {torch.float32: "<f4", torch.int64: "<i8", torch.int8: "|i1"}[tensor.dtype]
        self.__cuda_array_interface__ = {
            "shape": tuple(tensor.shape), "typestr": typestr, "data": (tensor.data_ptr(), readonly),
            "strides": strides, "version": 3,
        }


def test_foreign_cuda_array_interface_is_used_without_a_copy():
    # the reference's add(a, b, c, N) test with CuPy arrays (test/test_cupy.py:9-24), on this
    # package's row-sum kernel: inputs and output are foreign device arrays
    base = torch.randn(64, 96, device="cuda")
    out = torch.zeros(64, device="cuda")
    x, o = ForeignDeviceArray(base), ForeignDeviceArray(out)
    buf = parpy.buffer.from_array(x, CUDA)
    assert buf._get_ptr() == base.data_ptr() and buf.src is None and buf.shape == (64, 96)
    from parpy_b200 import kernels
    kernels.sum_rows(x, o, 64, opts=parpy.par({"N": parpy.threads(64)}))
    torch.cuda.synchronize()
    assert torch.allclose(out, base.sum(dim=1), atol=1e-4)          # written in place, no staging
    # read-only and strided memory are rejected as the reference does (python/parpy/buffer.py:15-31)
    with pytest.raises(ValueError, match="read-only"):
        parpy.buffer.from_array(ForeignDeviceArray(base, readonly=True), CUDA)
    with pytest.raises(ValueError, match="contiguous"):
        parpy.buffer.from_array(ForeignDeviceArray(base.t(), strides=(4, 384)), CUDA)


def test_forward_accepts_foreign_device_arrays():
    from parpy_b200 import hmm as hmm_mod, synthetic
    hmm, seqs = synthetic.hmm_model(4, seed=3), synthetic.hmm_sequences(6, 3, 40, seed=4)
    dh, ds = hmm_mod.to_device(hmm), hmm_mod.to_device(seqs)
    want = hmm_mod.forward_parpy(dh, ds)
    wrap = lambda d: {k: (ForeignDeviceArray(v) if isinstance(v, torch.Tensor) and v.dim() > 0 else v)
                      for k, v in d.items()}
    result = torch.zeros(6, device="cuda")
    hmm_mod.forward_kernel(wrap(dh), wrap(ds), ForeignDeviceArray(result), None, None,
                           opts=parpy.par({"inst": parpy.threads(6)}))
    assert torch.equal(result, want)
