"""Host-side behaviour of the call surface: option types, kernel resolution,
argument validation and the sharding helpers. No GPU needed."""
import os

import numpy as np
import pytest

import parpy_b200 as parpy
from parpy_b200 import buffer, dist, ops, synthetic
from parpy_b200.options import DataType


def test_looppar_rules():
    # src/par.rs:49-68
    p = parpy.threads(128)
    assert p.nthreads == 128 and p.is_parallel() and not p.reduction
    with pytest.raises(RuntimeError, match="number of threads"):
        p.threads(256)
    assert parpy.reduce().reduction
    with pytest.raises(RuntimeError, match="divisible by 32"):
        parpy.threads(4).tpb(16)
    assert parpy.threads(4).tpb(64)._tpb == 64


def test_compile_options_defaults_and_setters():
    # src/option.rs:90-131
    o = parpy.CompileOptions()
    assert o.backend == parpy.CompileBackend.Auto and o.max_thread_blocks_per_cluster == 8
    o.max_thread_blocks_per_cluster = 16
    with pytest.raises(RuntimeError, match="power of two"):
        o.max_thread_blocks_per_cluster = 12
    with pytest.raises(RuntimeError, match="non integer"):
        o.force_int_size = parpy.types.F32
    o.force_float_size = parpy.types.F32
    q = parpy.par({"inst": parpy.threads(10)})
    assert "inst" in q.parallelize and "inst" in str(q)


def test_elem_types_round_trip():
    for name in ("Bool", "I8", "I16", "I32", "I64", "U8", "U16", "U32", "U64", "F16", "F32", "F64"):
        e = getattr(parpy.types, name)
        assert np.dtype(e.to_numpy()).itemsize == e.size()
        assert DataType.from_elem_size(e).sz == e
    assert DataType("<f4").to_numpy() is np.float32


def test_jit_binds_known_functions_and_rejects_unknown():
    @parpy.jit
    def forward_kernel(hmm, seqs, result, alpha1, alpha2):
        pass

    @parpy.jit
    def forward_init_inst(hmm, seqs, alpha_src, inst):
        pass

    with pytest.raises(RuntimeError, match="only available inlined"):
        forward_init_inst(1, 2, 3, 4, opts=parpy.par({}))
    with pytest.raises(RuntimeError, match="no native kernel"):
        @parpy.jit
        def something_else(x, y):
            pass
    with pytest.raises(RuntimeError, match="no native kernel"):
        @parpy.jit
        def forward_kernel(a, b):  # right name, wrong parameters
            pass
    assert len(parpy.print_compiled(forward_kernel, [])) != 0


def test_opts_keyword_is_required_and_exclusive():
    # python/parpy/__init__.py:59-67,89-99
    from parpy_b200.hmm import forward_kernel
    with pytest.raises(RuntimeError, match="Missing required keyword argument opts"):
        forward_kernel(1, 2, 3, 4, 5)
    with pytest.raises(RuntimeError, match="should be of type"):
        forward_kernel(1, 2, 3, 4, 5, opts={"inst": 3})
    with pytest.raises(RuntimeError, match="unsupported keyword"):
        forward_kernel(1, 2, 3, 4, 5, opts=parpy.par({}), seq=True)


def test_metal_backend_is_refused():
    from parpy_b200.hmm import forward_kernel
    o = parpy.par({})
    o.backend = parpy.CompileBackend.Metal
    with pytest.raises(RuntimeError, match="not available"):
        forward_kernel(1, 2, 3, 4, 5, opts=o)


def test_array_interface_checks():
    # python/parpy/buffer.py:15-31
    a = np.zeros((4, 6), dtype=np.float32)
    shape, dtype, _ = buffer._extract_array_interface(a)
    assert shape == (4, 6) and str(dtype) == "<f4"
    with pytest.raises(ValueError, match="contiguous"):
        buffer._extract_array_interface(a[:, ::2])
    ro = np.zeros(3, dtype=np.float32)
    ro.setflags(write=False)
    with pytest.raises(ValueError, match="read-only"):
        buffer._extract_array_interface(ro)
    with pytest.raises(ValueError, match="Failed to extract"):
        buffer._extract_array_interface(object())


def test_forward_option_flags():
    from parpy_b200 import _native
    o = parpy.par({})
    assert ops._forward_flags(o) == _native.FWD_AUTO and not ops.forward_wants_alpha(o)
    o.b200 = {"forward": "five_term", "write_alpha": True}
    assert ops._forward_flags(o) == _native.FWD_FIVE_TERM | _native.FWD_WRITE_ALPHA
    assert ops.forward_wants_alpha(o)
    for mode, flag in (("log_space", _native.FWD_LOG_SPACE), ("scaled", _native.FWD_SCALED),
                       ("streaming", _native.FWD_STREAMING), ("auto", _native.FWD_AUTO)):
        o.b200 = {"forward": mode}
        assert ops._forward_flags(o) == flag
    # the values are the header's
    header = open(os.path.join(os.path.dirname(__file__), "..", "include", "parpy_b200.h")).read()
    for name, value in (("LOG_SPACE", _native.FWD_LOG_SPACE), ("SCALED", _native.FWD_SCALED),
                        ("FIVE_TERM", _native.FWD_FIVE_TERM), ("WRITE_ALPHA", _native.FWD_WRITE_ALPHA),
                        ("STREAMING", _native.FWD_STREAMING)):
        assert f"#define PARPY_B200_FWD_{name} {value}u" in header
    o.b200 = {"forward": "bogus"}
    with pytest.raises(RuntimeError, match="must be"):
        ops._forward_flags(o)


def test_lpt_partition_is_balanced_deterministic_and_complete():
    lens = synthetic.hmm_sequences(500, 1000, 4000)["lens"].numpy()
    for world in (1, 2, 4, 8):
        parts = dist.lpt_partition(lens, world)
        allidx = np.sort(np.concatenate(parts))
        assert np.array_equal(allidx, np.arange(500))
        loads = np.array([lens[p].sum() for p in parts])
        assert loads.max() - loads.min() <= lens.max()
        again = dist.lpt_partition(lens, world)
        assert all(np.array_equal(a, b) for a, b in zip(parts, again))
    assert dist.lpt_partition(np.array([], dtype=np.int64), 2)[0].size == 0


def test_shard_sequences_trims_to_local_maxlen():
    seqs = synthetic.hmm_sequences(16, 10, 50, seed=5)
    for rank in range(3):
        local, idx = dist.shard_sequences(seqs, rank, 3)
        assert int(local["maxlen"]) == int(seqs["lens"][idx].max())
        for j, i in enumerate(idx):
            n = int(seqs["lens"][i])
            assert np.array_equal(local["data"][j, :n].numpy(), seqs["data"][i, :n].numpy())


def test_row_block_partition_balances_nnz():
    csr = synthetic.zipf_csr(10000, 10000, mean_nnz=16, cap=512, seed=3)
    cuts = dist.row_block_partition(csr["rows"].numpy(), 4)
    assert cuts[0] == 0 and cuts[-1] == 10000 and np.all(np.diff(cuts) >= 0)
    nnz = np.diff(csr["rows"].numpy()[cuts])
    assert nnz.max() - nnz.min() <= 2 * 512


def test_synthetic_generators_are_seeded_and_shaped():
    h1, h2 = synthetic.hmm_model(5), synthetic.hmm_model(5)
    assert all((h1[k] == h2[k]).all() for k in h1)
    assert tuple(h1["trans1"].shape) == (1024, 4) and tuple(h1["output_prob"].shape) == (101, 1024)
    assert int(h1["num_states"]) == 16384
    s = synthetic.hmm_sequences(100, 2000, 2000)
    assert tuple(s["data"].shape) == (100, 2000) and s["data"].min() >= 0 and s["data"].max() <= 100
    r = synthetic.hmm_sequences(50, 10, 40)
    lens = r["lens"]
    assert lens.min() >= 10 and lens.max() <= 40 and int(r["maxlen"]) == int(lens.max())
    assert synthetic.state_steps(h1, s) == 16384 * 200000


def test_print_compiled_returns_a_self_contained_translation_unit(tmp_path, monkeypatch):
    # python/parpy/__init__.py:177-199; test/test_softmax.py:57-66 asserts len(s) != 0
    import shutil
    from parpy_b200 import kernels, source
    src = parpy.print_compiled(kernels.softmax, [])
    assert len(src) != 0 and "rowmap_warp_rows" in src and 'extern "C"' in src
    assert '#include "' not in src                      # local includes are inlined
    for op in ("forward_kernel", "spmv_row", "sum_rows", "parpy_sddmm_coo_kernel", "spmm_cell"):
        assert len(source.kernel_source(op)) > 1000
    if shutil.which("nvcc"):
        monkeypatch.setenv("PARPY_B200_CACHE", str(tmp_path))
        lib = source.compile_source(src)                # cross-compiles without a GPU
        import ctypes
        assert hasattr(ctypes.CDLL(lib), "softmax")
        assert source.compile_source(src) == lib        # cached by content
        with pytest.raises(RuntimeError, match="Compilation of CUDA source failed"):
            source.compile_source("this is not CUDA")


def test_hdf5_reader_reproduces_the_committed_fixtures():
    # the minimal HDF5 reader + the loader steps of benchmarks/forward.py:40-56 against tests/golden/*.npz
    import os
    import sys
    from oracle import build as oracle_build
    ref = oracle_build.reference_root()
    if not ref or not os.path.isdir(os.path.join(ref, "test", "data")):
        pytest.skip("reference checkout with test/data not present")
    from conftest import GOLDEN
    sys.path.insert(0, GOLDEN)
    import make_golden
    for name in ("3mer", "5mer"):
        built = make_golden.build_model(os.path.join(ref, "test", "data", f"{name}-model.hdf5"))
        stored = np.load(os.path.join(GOLDEN, f"hmm_{name}.npz"))
        for key in stored.files:
            assert np.array_equal(np.asarray(built[key]), stored[key], equal_nan=True), (name, key)
    sig = make_golden.build_signals(os.path.join(ref, "test", "data", "signals.hdf5"))
    stored = np.load(os.path.join(GOLDEN, "signals.npz"))
    assert np.array_equal(sig["data"], stored["data"]) and np.array_equal(sig["lens"], stored["lens"])


def test_buffer_module_without_a_device():
    # test/test_buffer.py:59-73
    a = np.ndarray((20, 10, 32), dtype=np.float32)
    b = parpy.buffer.from_array(a, None)
    assert b.shape == (20, 10, 32)
    assert b.dtype == parpy.buffer.DataType.from_elem_size(parpy.types.F32)
    with pytest.raises(ValueError, match="Cannot convert to buffer of unknown backend 5"):
        parpy.buffer.from_array(np.ndarray((10,), dtype=np.float32), 5)
    with pytest.raises(RuntimeError, match="Metal"):
        parpy.buffer.from_array(a, parpy.CompileBackend.Metal)
