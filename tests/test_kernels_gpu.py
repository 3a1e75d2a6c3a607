"""Parity of the softmax / reduction / SpMV / SDDMM kernels with the CPU oracle
and with the references the reference's own tests use, through the Python call
surface (host and device arrays) and through the C ABI. Tolerance: max relative
error <= 1e-4 for fp32 values (plus the reference tests' own atol where they
state one); integer outputs are compared bit for bit."""
import ctypes
import warnings

import numpy as np
import pytest
import torch

import parpy_b200 as parpy
from conftest import max_rel
from parpy_b200 import kernels, synthetic

pytestmark = pytest.mark.gpu
P = ctypes.c_void_p


@pytest.fixture(scope="module")
def oracle_mod():
    from oracle import oracle
    return oracle


def opts(**labels):
    return parpy.par({k: v for k, v in labels.items()})


# ---- softmax ---------------------------------------------------------------------------------
def test_softmax_like_reference_test():
    # test/test_softmax.py:28-40,48-54: host tensors, N:256 M:128 threads
    torch.manual_seed(1234)
    N, M = 256, 512
    x = torch.randn((N, M), dtype=torch.float32)
    out = torch.zeros_like(x)
    kernels.softmax(x, N, M, out, opts=opts(N=parpy.threads(256), M=parpy.threads(128)))
    assert torch.allclose(torch.softmax(x, 1), out, atol=1e-5)


@pytest.mark.parametrize("shape", [(256, 1024), (3, 4), (5, 1), (7, 1023), (33, 2048), (9, 2052),
                                   (4, 5000), (3, 49152), (2, 70001), (1, 8), (1000, 36)])
def test_softmax_shapes_against_oracle(native, oracle_mod, shape):
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    xd = x.cuda()
    out = torch.empty_like(xd)
    rc = native.lib().parpy_b200_softmax(P(xd.data_ptr()), shape[0], shape[1], P(out.data_ptr()),
                                         P(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, native.error_message()
    exp = oracle_mod.softmax(x)
    got = out.cpu().numpy()
    assert max_rel(got, exp) <= 1e-4
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("shape", [(9000, 1024), (33007, 512), (40003, 260), (2100, 4096), (601, 16384), (1003, 9000)])
def test_large_row_maps(native, oracle_mod, shape):
    # Inputs of 32 MiB and more (several waves of CTAs): short rows, one per warp, with a last
    # CTA that is not full; long rows, one per CTA, with the last float4 slots of a thread
    # unused; softmax, in-place normalisation, exp + row sums.
    g = torch.Generator().manual_seed(77)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    xd = x.cuda()
    out = torch.empty_like(xd)
    stream = P(torch.cuda.current_stream().cuda_stream)
    rc = native.lib().parpy_b200_softmax(P(xd.data_ptr()), shape[0], shape[1], P(out.data_ptr()), stream)
    assert rc == 0, native.error_message()
    got = out.cpu().numpy()
    assert max_rel(got, oracle_mod.softmax(x)) <= 1e-4
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)
    pos = (torch.rand(shape, generator=g) + 0.05)
    pd = pos.cuda()
    rc = native.lib().parpy_b200_normalize_rows(P(pd.data_ptr()), shape[0], shape[1], stream)
    assert rc == 0, native.error_message()
    assert max_rel(pd.cpu().numpy(), oracle_mod.normalize_rows(pos)) <= 1e-5
    small = (x * 0.25).contiguous()
    sd = small.cuda()
    sums = torch.empty(shape[0], device="cuda")
    rc = native.lib().parpy_b200_sum_exp_rows(P(sd.data_ptr()), shape[0], shape[1], P(sums.data_ptr()), stream)
    assert rc == 0, native.error_message()
    ref_x, ref_sums = oracle_mod.sum_exp_rows(small.numpy().copy())
    assert max_rel(sd.cpu().numpy(), ref_x) <= 1e-5
    assert np.allclose(sums.cpu().numpy(), ref_sums, rtol=1e-5)


def test_softmax_reference_shaped_entry_and_extremes(native):
    x = torch.tensor([[1e4, 1e4 - 1, -1e4, 0.0], [-3e38, -3e38, -3e38, -3e38]], device="cuda")
    out = torch.empty_like(x)
    rc = native.lib().softmax(P(x.data_ptr()), 2, 4, P(out.data_ptr()))
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.allclose(out.cpu(), torch.softmax(x.cpu(), 1), atol=1e-6)
    rc = native.lib().softmax(None, 2, 4, P(out.data_ptr()))
    assert rc != 0 and "null" in native.error_message()


# ---- reductions ------------------------------------------------------------------------------------
NP_OPS = {"sum": np.sum, "prod": np.prod, "max": np.max, "min": np.min}


@pytest.mark.parametrize("op", ["sum", "prod", "max", "min"])
@pytest.mark.parametrize("kind", ["rows", "axis", "2d"])
def test_reduce_like_reference_test(op, kind):
    # test/test_reduce.py:72-85,103-126: NumPy host arrays, N=100, M=50, atol 1e-4
    np.random.seed(1234)
    N, M = 100, 50
    x = np.random.randn(N, M).astype(np.float32)
    out = np.zeros(N, dtype=np.float32)
    fn = getattr(kernels, f"{op}_{kind}")
    fn(x, out, N, opts=opts(outer=parpy.threads(N), inner=parpy.threads(128)))
    if kind == "2d":
        expected = np.zeros(N, dtype=np.float32)
        expected[0] = NP_OPS[op](x)
    else:
        expected = NP_OPS[op](x, axis=1)
    assert np.allclose(expected, out, atol=1e-4), f"{expected}\n{out}"


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (64, 1024), (2000, 300), (8, 100003), (3, 1 << 20),
                                   (1, (1 << 22) + 3), (5, 0)])
@pytest.mark.parametrize("op", [0, 2, 3])
def test_reduce_shapes_against_oracle(native, oracle_mod, shape, op):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    xd = x.cuda()
    out = torch.full((shape[0],), 123.0, device="cuda")
    for _ in range(2):          # twice: the scratch tickets must be left reusable
        rc = native.lib().parpy_b200_reduce_rows(op, P(xd.data_ptr()), P(out.data_ptr()), shape[0], shape[1],
                                                 P(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, native.error_message()
    exp = oracle_mod.reduce_rows(["sum", "prod", "max", "min"][op], x.numpy())
    got = out.cpu().numpy()
    if op == 0:
        # sums of N(0,1) values: compare against the double-precision oracle relative to sqrt(M)
        assert np.all(np.abs(got - exp) <= 1e-4 * max(1.0, np.sqrt(shape[1])))
    else:
        assert np.array_equal(got, exp)


def test_prod_rows_against_oracle(native, oracle_mod):
    g = torch.Generator().manual_seed(3)
    x = (1.0 + 0.01 * torch.randn((37, 4099), generator=g)).float()
    out = torch.empty(37, device="cuda")
    xd = x.cuda()
    rc = native.lib().parpy_b200_reduce_rows(1, P(xd.data_ptr()), P(out.data_ptr()), 37, 4099, None)
    torch.cuda.synchronize()
    assert rc == 0 and max_rel(out.cpu().numpy(), oracle_mod.reduce_rows("prod", x.numpy())) <= 1e-4


def test_fused_sum_max():
    g = torch.Generator().manual_seed(11)
    for n in (1, 5, 1 << 20, (1 << 24) + 5):
        x = torch.randn(n, generator=g, dtype=torch.float32).cuda()
        r1 = kernels.sum_max(x).cpu().numpy()
        r2 = kernels.sum_max(x).cpu().numpy()
        assert np.array_equal(r1, r2)                      # deterministic
        assert r1[1] == float(x.max())
        assert abs(r1[0] - float(x.double().sum())) <= 1e-4 * max(1.0, np.sqrt(n))


# ---- SpMV -----------------------------------------------------------------------------------------------
def uniform_random_csr_f32_i64(N, M, d):
    # test/test_spmv.py:31-44
    nnz = int(N * M * d)
    s = set()
    while len(s) < nnz:
        s.update(np.random.randint(0, N * M, nnz - len(s)))
    flat = np.array(list(s), dtype=np.int64)
    rows, cols = np.divmod(flat, M)
    values = torch.randn(nnz, dtype=torch.float32)
    A = torch.sparse_coo_tensor(np.array((rows, cols)), values)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return A.to_sparse_csr()


def test_spmv_like_reference_test():
    # test/test_spmv.py:20-29,46-53,62-71: host tensors, compare with torch CSR matmul, atol 1e-5
    torch.manual_seed(1234)
    np.random.seed(1234)
    N, M = 256, 4096
    A = uniform_random_csr_f32_i64(N, M, 0.01)
    x = torch.randn(M, dtype=torch.float32)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        y1 = A.matmul(x)
        Ad = {"values": A.values(), "rows": A.crow_indices(), "cols": A.col_indices(), "nrows": N}
    y2 = torch.zeros((N,), dtype=x.dtype)
    kernels.spmv_row(Ad, x, y2, opts=opts(row=parpy.threads(N), i=parpy.threads(128).reduce()))
    assert torch.allclose(y1, y2, atol=1e-5)


@pytest.mark.parametrize("nrows,ncols,mean,cap", [(1, 10, 3, 8), (5000, 5000, 2, 16), (20000, 30000, 32, 4096),
                                                   (300, 1000, 900, 4096), (100000, 100000, 8, 64)])
def test_spmv_power_law_against_oracle(native, oracle_mod, nrows, ncols, mean, cap):
    A = synthetic.zipf_csr(nrows, ncols, mean_nnz=mean, cap=min(cap, ncols), seed=nrows)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(ncols, generator=g)
    y0 = torch.randn(nrows, generator=g)          # y is accumulated into
    exp = oracle_mod.spmv(A, x, y0.numpy())
    d = {k: v.cuda() for k, v in A.items() if isinstance(v, torch.Tensor)}
    xd, yd = x.cuda(), y0.cuda()
    rc = native.lib().parpy_b200_spmv(P(d["values"].data_ptr()), P(d["rows"].data_ptr()), P(d["cols"].data_ptr()),
                                      nrows, d["values"].numel(), P(xd.data_ptr()), P(yd.data_ptr()),
                                      P(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, native.error_message()
    got = yd.cpu().numpy()
    scale = np.maximum(np.abs(exp), np.sqrt(np.maximum(np.diff(A["rows"].numpy()), 1)))
    assert np.all(np.abs(got - exp) <= 1e-4 * scale)
    empty = np.diff(A["rows"].numpy()) == 0
    assert np.array_equal(got[empty], y0.numpy()[empty])       # empty rows untouched, bit for bit


def test_spmv_reference_shaped_entry(native, oracle_mod):
    A = synthetic.zipf_csr(4000, 4000, mean_nnz=20, cap=500, seed=12)
    x = torch.randn(4000, generator=torch.Generator().manual_seed(5))
    d = {k: v.cuda() for k, v in A.items() if isinstance(v, torch.Tensor)}
    xd, yd = x.cuda(), torch.zeros(4000, device="cuda")
    torch.cuda.synchronize()
    rc = native.lib().spmv_row(P(d["cols"].data_ptr()), 4000, P(d["rows"].data_ptr()), P(d["values"].data_ptr()),
                               P(xd.data_ptr()), P(yd.data_ptr()))
    torch.cuda.synchronize()
    assert rc == 0, native.error_message()
    exp = oracle_mod.spmv(A, x, np.zeros(4000, dtype=np.float32))
    assert np.allclose(yd.cpu().numpy(), exp, atol=1e-4, rtol=1e-4)


# ---- SDDMM ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (1.5, 2.0)])
@pytest.mark.parametrize("N,ncols,K,density", [(512, 768, 64, 0.02), (100, 333, 30, 0.05), (64, 64, 1024, 0.1),
                                               (128, 200, 256, 0.05), (96, 150, 512, 0.07), (300, 4000, 1024, 0.01)])
def test_sddmm_csr_and_coo_against_oracle(oracle_mod, alpha, beta, N, ncols, K, density):
    # benchmarks/sddmm.py:43-61,72-84 call shapes; validation rule of :86-103 is atol=rtol=1e-5
    C = synthetic.uniform_csr(N, ncols, density, seed=N + K)
    g = torch.Generator().manual_seed(42)
    A, B = torch.randn(N, K, generator=g), torch.randn(K, ncols, generator=g)
    exp_rows = oracle_mod.sddmm_decompress(C["crows"])
    exp = oracle_mod.sddmm(A, B, exp_rows, C["cols"], C["values"], alpha, beta)
    nnz = C["nnz"]
    # CSR entry, device tensors
    Cd = {"crows": C["crows"].cuda(), "rows": torch.empty(nnz, dtype=torch.int64, device="cuda"),
          "cols": C["cols"].cuda(), "values": C["values"].cuda(), "nnz": nnz}
    D = torch.empty(nnz, device="cuda")
    p = {"N": parpy.threads(N), "M": parpy.threads(32), "nnz": parpy.threads(nnz)}
    kernels.parpy_sddmm_csr_kernel(A.cuda(), B.cuda(), Cd, D, N, alpha, beta, opts=parpy.par(p))
    assert np.array_equal(Cd["rows"].cpu().numpy(), exp_rows)                  # index output: bit exact
    got = D.cpu().numpy()
    # fp32 dot products of K terms in different summation orders: absolute slack grows with K
    assert np.all(np.abs(got - exp) <= 1e-5 + 2e-7 * K + 1e-4 * np.abs(exp)), max_rel(got, exp)
    # COO entry, host arrays
    Ch = {"rows": exp_rows, "cols": C["cols"].numpy(), "values": C["values"].numpy(), "nnz": nnz}
    Dh = np.zeros(nnz, dtype=np.float32)
    kernels.parpy_sddmm_coo_kernel(A.numpy(), B.numpy(), Ch, Dh, alpha, beta, opts=parpy.par({"nnz": parpy.threads(nnz)}))
    assert np.array_equal(Dh, got)
    # COO entries in any order (the long-dot-product kernel caches the A row of a run of equal rows,
    # and must not depend on the runs being long)
    perm = np.random.default_rng(N).permutation(nnz)
    Cp = {"rows": exp_rows[perm].copy(), "cols": C["cols"].numpy()[perm].copy(), "values": C["values"].numpy()[perm].copy(),
          "nnz": nnz}
    Dp = np.zeros(nnz, dtype=np.float32)
    kernels.parpy_sddmm_coo_kernel(A.numpy(), B.numpy(), Cp, Dp, alpha, beta, opts=parpy.par({"nnz": parpy.threads(nnz)}))
    assert np.array_equal(Dp, got[perm])


def test_sddmm_decompress_entry(native, oracle_mod):
    C = synthetic.uniform_csr(1000, 2000, 0.01, seed=4)
    crows = C["crows"].cuda()
    rows = torch.full((C["nnz"],), -1, dtype=torch.int64, device="cuda")
    rc = native.lib().parpy_sddmm_decompress_csr(P(crows.data_ptr()), P(rows.data_ptr()), 1000)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(rows.cpu().numpy(), oracle_mod.sddmm_decompress(C["crows"]))
    rows_h = np.zeros(C["nnz"], dtype=np.int64)
    kernels.parpy_sddmm_decompress_csr(C["crows"].numpy(), rows_h, 1000, opts=parpy.par({}))
    assert np.array_equal(rows_h, oracle_mod.sddmm_decompress(C["crows"]))


# ---- normalize_rows, sum_exp_3d, spmm_cell ----------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 1024), (256, 1024), (7, 33), (5, 4100), (3, 40000), (2, 70001)])
def test_normalize_rows_like_reference_test(oracle_mod, shape):
    # test/test_normalize.py:17-45: ones (and positive random rows), compared with L1 normalisation
    t = torch.ones(shape, dtype=torch.float32)
    out = t.clone()
    kernels.normalize_rows(out, shape[0], shape[1], opts=opts(i=parpy.threads(256), j1=parpy.threads(128).reduce()))
    assert torch.allclose(torch.nn.functional.normalize(t, p=1, dim=1), out, 1e-5)
    r = torch.rand(shape, generator=torch.Generator().manual_seed(9)) + 0.05
    dev = r.cuda()
    kernels.normalize_rows(dev, shape[0], shape[1], opts=parpy.par({}))
    assert max_rel(dev.cpu().numpy(), oracle_mod.normalize_rows(r)) <= 1e-5


@pytest.mark.parametrize("dims", [(10, 20, 30), (4, 8, 1024), (3, 5, 8192), (2, 2, 50000)])
def test_sum_exp_3d_like_reference_test(oracle_mod, dims):
    # test/test_sync.py:71-80
    N, M, K = dims
    x = np.random.RandomState(1).randn(N, M, K).astype(np.float32)
    ref_x, ref_out = oracle_mod.sum_exp_rows(x.reshape(N * M, K))
    out = np.zeros((N, M), dtype=np.float32)
    kernels.sum_exp_3d(x, N, M, out, opts=opts(N=parpy.threads(N), M=parpy.threads(M), K_1=parpy.threads(32),
                                               K_2=parpy.threads(64)))
    assert np.allclose(out.reshape(-1), ref_out, atol=1e-5, rtol=1e-5)
    assert max_rel(x.reshape(N * M, K), ref_x) <= 1e-5          # x was exponentiated in place


@pytest.mark.parametrize("N,M,K", [(1024, 256, 512), (100, 77, 33), (5, 9, 4), (300, 500, 64), (257, 300, 100),
                                   (70000, 900, 16), (64, 200, 8), (33, 100, 32)])
def test_spmm_like_reference_test(native, oracle_mod, N, M, K):
    # test/test_spmm.py:53-87: uniform random CSR at 1 % (denser for the tiny cases), dense B
    A = synthetic.zipf_csr(N, M, mean_nnz=max(2, M // 100), cap=M, seed=N)
    B = torch.randn(M, K, generator=torch.Generator().manual_seed(4))
    C0 = torch.randn(N, K, generator=torch.Generator().manual_seed(5))      # C is accumulated into
    exp = oracle_mod.spmm(A, B, C0.numpy())
    Ad = {"values": A["values"], "rows": A["rows"], "cols": A["cols"], "nrows": N}
    C = C0.clone()
    kernels.spmm_cell(Ad, {"values": B, "ncols": K}, C, opts=opts(i=parpy.threads(N), j=parpy.threads(K),
                                                                  aidx=parpy.threads(32).reduce()))
    assert np.allclose(C.numpy(), exp, atol=1e-5, rtol=1e-5)
    # reference-shaped C entry on device memory
    d = {k: v.cuda() for k, v in A.items() if isinstance(v, torch.Tensor)}
    Bd, Cd = B.cuda(), C0.cuda()
    rc = native.lib().spmm_cell(P(d["cols"].data_ptr()), N, P(d["rows"].data_ptr()), P(d["values"].data_ptr()), K,
                                P(Bd.data_ptr()), P(Cd.data_ptr()))
    torch.cuda.synchronize()
    assert rc == 0 and np.allclose(Cd.cpu().numpy(), exp, atol=1e-5, rtol=1e-5)


def test_compile_string_round_trip(oracle_mod, tmp_path, monkeypatch):
    # the reference's workflow: print the CUDA for a function, edit it, compile the string, call it
    monkeypatch.setenv("PARPY_B200_CACHE", str(tmp_path))
    src = parpy.print_compiled(kernels.softmax, [])
    edited = src.replace("// parpy_b200: amalgamated source", "// edited copy of the amalgamated source", 1)
    fn = parpy.compile_string("softmax", edited)
    x = torch.randn((64, 512), generator=torch.Generator().manual_seed(3))
    out = torch.zeros_like(x)
    fn(x, 64, 512, out)
    assert max_rel(out.numpy(), oracle_mod.softmax(x)) <= 1e-4
    # a small hand-written kernel with a dict argument, flattened in sorted-key order
    code = r"""
    #include <cstdint>
    __global__ void k(const float* a, float s, float* y, int64_t n) {
        int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
        if (i < n) y[i] = s * a[i] + y[i];
    }
    extern "C" int32_t scale_add(float* a, float s, float* y, int64_t n) {
        k<<<(unsigned)((n + 255) / 256), 256>>>(a, s, y, n);
        return (int32_t)cudaGetLastError();
    }
    """
    f2 = parpy.compile_string("scale_add", code)
    a = np.arange(1000, dtype=np.float32)
    y = np.ones(1000, dtype=np.float32)
    f2({"a": a, "s": np.array(2.0, dtype=np.float32)}, y, 1000)
    assert np.array_equal(y, 2.0 * a + 1.0)


# ---- row-block sharding on one GPU: the shards of every rank run one after another -------------------------
@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_block_shards_reassemble_the_unsharded_result(oracle_mod, world):
    # What each rank of an N-GPU job computes (parpy_b200.dist.shard_csr + the single-GPU kernel on
    # the block), run here shard after shard on one GPU and put together without the collective.
    from parpy_b200 import dist
    A = synthetic.zipf_csr(20000, 20000, mean_nnz=16, cap=1024, seed=9)
    g = torch.Generator().manual_seed(10)
    x = torch.randn(20000, generator=g)
    Ad = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in A.items()}
    xd = x.cuda()
    y_full = torch.zeros(20000, device="cuda")
    kernels.spmv_row(Ad, xd, y_full, opts=opts(row=parpy.threads(20000)))
    y_parts = torch.zeros(20000, device="cuda")
    for r in range(world):
        local, bounds = dist.shard_csr(Ad, r, world)
        assert int(local["rows"][0]) == 0 and int(local["rows"][-1]) == local["nnz"]
        y_local = y_parts[local["row_begin"]:local["row_end"]].clone()
        dist._default_spmv(local, xd, y_local)
        y_parts[local["row_begin"]:local["row_end"]] = y_local
    exp = oracle_mod.spmv(A, x, np.zeros(20000, dtype=np.float32))
    assert np.allclose(y_parts.cpu().numpy(), exp, atol=1e-4, rtol=1e-4)
    # rows are summed in chunks of non-zeros whose cuts move with the block's first non-zero
    assert np.allclose(y_parts.cpu().numpy(), y_full.cpu().numpy(), atol=1e-5, rtol=1e-5)

    # SDDMM: every non-zero is an independent dot product, so the shards agree bit for bit
    N, ncols, K = 1024, 1536, 64
    C = synthetic.uniform_csr(N, ncols, 0.02, seed=11)
    Am, Bm = torch.randn(N, K, generator=g).cuda(), torch.randn(K, ncols, generator=g).cuda()
    Cd = {"crows": C["crows"].cuda(), "rows": torch.zeros(C["nnz"], dtype=torch.int64, device="cuda"),
          "cols": C["cols"].cuda(), "values": C["values"].cuda(), "nnz": C["nnz"]}
    D_full = torch.empty(C["nnz"], device="cuda")
    kernels.parpy_sddmm_csr_kernel(Am, Bm, Cd, D_full, N, 1.5, 2.0, opts=opts(nnz=parpy.threads(C["nnz"])))
    D_parts = torch.zeros(C["nnz"], device="cuda")
    rows_parts = torch.zeros(C["nnz"], dtype=torch.int64, device="cuda")
    for r in range(world):
        local, bounds = dist.shard_csr(Cd, r, world, rows_key="crows")
        local["rows"] = torch.zeros(local["nnz"], dtype=torch.int64, device="cuda")
        D_local = torch.zeros(local["nnz"], device="cuda")
        dist._default_sddmm(Am[local["row_begin"]:local["row_end"]].contiguous(), Bm, local, D_local, 1.5, 2.0)
        D_parts[local["nnz_begin"]:local["nnz_end"]] = D_local
        rows_parts[local["nnz_begin"]:local["nnz_end"]] = local["rows"] + local["row_begin"]
    assert torch.equal(D_parts, D_full)
    assert torch.equal(rows_parts, Cd["rows"])

    # sum and max over slices: the maximum is exact, the sum agrees to fp32 summation order
    v = torch.randn(1 << 22, generator=g).cuda()
    whole = kernels.sum_max(v).cpu().numpy()
    sb = dist.slice_bounds(v.numel(), world)
    pairs = [kernels.sum_max(v[int(sb[r]):int(sb[r + 1])]).cpu().numpy() for r in range(world)]
    assert max(p[1] for p in pairs) == whole[1]
    assert abs(sum(float(p[0]) for p in pairs) - float(whole[0])) <= 1e-4 * float(v.abs().sum())


# ---- the benchmark workloads at full size ------------------------------------------------------------
def test_full_size_sddmm_config(oracle_mod):
    # CSR mask 8192 x 8192 at 1 % density, A [8192, 64], B [64, 8192]; (alpha, beta) = (1, 0) and (1.5, 2)
    N, K = 8192, 64
    C = synthetic.uniform_csr(N, N, 0.01, seed=1234)
    g = torch.Generator().manual_seed(1234)
    A, B = torch.randn(N, K, generator=g), torch.randn(K, N, generator=g)
    rows = oracle_mod.sddmm_decompress(C["crows"])
    Ad, Bd = A.cuda(), B.cuda()
    for alpha, beta in ((1.0, 0.0), (1.5, 2.0)):
        exp = oracle_mod.sddmm(A, B, rows, C["cols"], C["values"], alpha, beta)
        Cd = {"crows": C["crows"].cuda(), "rows": torch.empty(C["nnz"], dtype=torch.int64, device="cuda"),
              "cols": C["cols"].cuda(), "values": C["values"].cuda(), "nnz": C["nnz"]}
        D = torch.empty(C["nnz"], device="cuda")
        kernels.parpy_sddmm_csr_kernel(Ad, Bd, Cd, D, N, alpha, beta, opts=parpy.par({"nnz": parpy.threads(C["nnz"])}))
        assert np.array_equal(Cd["rows"].cpu().numpy(), rows)
        got = D.cpu().numpy()
        assert np.all(np.abs(got - exp) <= 1e-5 + 2e-7 * K + 1e-4 * np.abs(exp))


def test_full_size_spmv_config(native, oracle_mod):
    # 4,194,304 x 4,194,304 CSR, Zipf(1.5) row lengths with mean 32 capped at 4096, x ~ N(0,1)
    n = 1 << 22
    A = synthetic.zipf_csr(n, n, mean_nnz=32, cap=4096, seed=1234)
    x = torch.randn(n, generator=torch.Generator().manual_seed(1234))
    exp = oracle_mod.spmv(A, x, np.zeros(n, dtype=np.float32))
    d = {k: v.cuda() for k, v in A.items() if isinstance(v, torch.Tensor)}
    xd, yd = x.cuda(), torch.zeros(n, device="cuda")
    rc = native.lib().parpy_b200_spmv(P(d["values"].data_ptr()), P(d["rows"].data_ptr()), P(d["cols"].data_ptr()),
                                      n, d["values"].numel(), P(xd.data_ptr()), P(yd.data_ptr()),
                                      P(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, native.error_message()
    got = yd.cpu().numpy()
    lens = np.diff(A["rows"].numpy())
    assert np.all(np.abs(got - exp) <= 1e-4 * np.maximum(np.abs(exp), np.sqrt(np.maximum(lens, 1))))
    assert np.array_equal(got[lens == 0], np.zeros(int((lens == 0).sum()), dtype=np.float32))
    # linearity: A(2x) = 2 A(x) exactly in binary floating point
    y2 = torch.zeros(n, device="cuda")
    x2 = (2.0 * x).cuda()
    rc = native.lib().parpy_b200_spmv(P(d["values"].data_ptr()), P(d["rows"].data_ptr()), P(d["cols"].data_ptr()),
                                      n, d["values"].numel(), P(x2.data_ptr()), P(y2.data_ptr()),
                                      P(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    short = lens <= 64                      # rows summed by one thread in index order: bit-exact doubling
    assert np.array_equal(y2.cpu().numpy()[short], 2.0 * got[short])


def test_full_size_sum_and_max_over_2_to_30():
    n = 1 << 30
    v = torch.empty(n, dtype=torch.float32, device="cuda").normal_(generator=torch.Generator(device="cuda").manual_seed(1234))
    r = kernels.sum_max(v).cpu().numpy()
    assert r[1] == float(v.max())
    ref = float(v.sum(dtype=torch.float64))
    assert abs(r[0] - ref) <= 1e-4 * max(abs(ref), np.sqrt(n))
    out = np.zeros(1, dtype=np.float32)
    o = torch.zeros(1, device="cuda")
    kernels.max_2d(v.view(1 << 15, 1 << 15), o, 1 << 15, opts=parpy.par({"outer": parpy.threads(1024)}))
    assert float(o[0]) == r[1]
    kernels.min_2d(v.view(1 << 15, 1 << 15), o, 1 << 15, opts=parpy.par({"outer": parpy.threads(1024)}))
    assert float(o[0]) == float(v.min())
