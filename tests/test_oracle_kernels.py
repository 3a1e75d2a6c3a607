"""Pins the CPU oracles of the surrounding kernels to the same references the
reference's own tests use (torch / NumPy on the CPU). No GPU needed."""
import warnings

import numpy as np
import torch

from oracle import oracle
from parpy_b200 import synthetic


def test_softmax_oracle_matches_torch():
    # test/test_softmax.py:35-40
    torch.manual_seed(1234)
    x = torch.randn((256, 512), dtype=torch.float32)
    assert torch.allclose(torch.softmax(x, 1), torch.from_numpy(oracle.softmax(x)), atol=1e-5)


def test_reduce_oracle_matches_numpy():
    # test/test_reduce.py:82-85
    np.random.seed(1234)
    x = np.random.randn(100, 50).astype(np.float32)
    for op, fn in (("sum", np.sum), ("prod", np.prod), ("max", np.max), ("min", np.min)):
        assert np.allclose(fn(x, axis=1), oracle.reduce_rows(op, x), atol=1e-4)


def test_spmv_oracle_matches_torch_csr_matmul():
    # test/test_spmv.py:46-53
    A = synthetic.zipf_csr(512, 4096, mean_nnz=40, cap=600, seed=5)
    x = torch.randn(4096, generator=torch.Generator().manual_seed(1))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        t = torch.sparse_csr_tensor(A["rows"], A["cols"], A["values"], (512, 4096))
        expect = t.matmul(x).numpy()
    got = oracle.spmv(A, x, np.zeros(512, dtype=np.float32))
    assert np.allclose(got, expect, atol=1e-4, rtol=1e-5)
    # accumulates into y
    y0 = np.arange(512, dtype=np.float32)
    assert np.allclose(oracle.spmv(A, x, y0), expect + y0, atol=1e-4, rtol=1e-5)


def test_sddmm_oracle_matches_dense_restatement():
    # benchmarks/sddmm.py:18-19 computes alpha * (A @ B)[mask] + beta * C
    C = synthetic.uniform_csr(96, 160, 0.05, seed=9)
    rows = oracle.sddmm_decompress(C["crows"])
    assert np.array_equal(rows, np.repeat(np.arange(96), 8))
    g = torch.Generator().manual_seed(42)
    A, B = torch.randn(96, 64, generator=g), torch.randn(64, 160, generator=g)
    for alpha, beta in ((1.0, 0.0), (1.5, 2.0)):
        dense = (A.double() @ B.double()).numpy()
        expect = alpha * dense[rows, C["cols"].numpy()] + beta * C["values"].double().numpy()
        got = oracle.sddmm(A, B, rows, C["cols"], C["values"], alpha, beta)
        assert np.allclose(got, expect, atol=1e-5, rtol=1e-5)


def test_zipf_csr_generator_shape():
    A = synthetic.zipf_csr(200000, 200000, mean_nnz=32, cap=4096, seed=1)
    lens = np.diff(A["rows"].numpy())
    assert lens.max() <= 4096 and abs(lens.mean() - 32) < 1.0
    assert (lens >= 1024).sum() > 0 and np.median(lens) < 16    # heavy tail next to short rows
    assert A["cols"].min() >= 0 and A["cols"].max() < 200000


def test_normalize_sum_exp_and_spmm_oracles():
    # test/test_normalize.py:26-31, test/test_sync.py:71-80, test/test_spmm.py:80-87
    t = torch.rand((17, 100), generator=torch.Generator().manual_seed(3)) + 0.1
    assert torch.allclose(torch.nn.functional.normalize(t, p=1, dim=1), torch.from_numpy(oracle.normalize_rows(t)), 1e-5)
    x = np.random.RandomState(5).randn(10 * 20, 30).astype(np.float32)
    ex, sums = oracle.sum_exp_rows(x)
    assert np.allclose(ex, np.exp(x), rtol=1e-6) and np.allclose(sums, np.exp(x).sum(axis=1), atol=1e-5, rtol=1e-6)
    A = synthetic.zipf_csr(64, 48, mean_nnz=3, cap=20, seed=8)
    B = torch.randn(48, 40, generator=torch.Generator().manual_seed(2))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        dense = torch.sparse_csr_tensor(A["rows"], A["cols"], A["values"], (64, 48)).to_dense()
    assert np.allclose(oracle.spmm(A, B, np.zeros((64, 40), np.float32)), (dense @ B).numpy(), atol=1e-5)
