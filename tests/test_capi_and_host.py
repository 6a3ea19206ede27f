"""The C-ABI library builds, loads and exports what the header declares; host-side logic of
the Python layer that needs no device."""
import ctypes
import os
import re

import numpy as np
import pytest
import scipy.sparse as sp

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "featgraph_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fg_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from featgraph_b200 import _native, build
    path = build.build_cuda()
    assert os.path.exists(path)
    L = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(L, name), "library lacks %s" % name
    assert sorted(_native.SIGNATURES) == declared, "python binding table and header disagree"


def test_version_and_error_text_without_a_device():
    from featgraph_b200 import _native
    L = _native.lib()
    assert L.fg_version() >= 100
    assert isinstance(L.fg_last_error(), bytes)


def test_argument_errors_are_reported_not_raised_as_faults():
    """Host-side validation happens before any CUDA call, so it can be exercised here."""
    from featgraph_b200 import _native
    L = _native.lib()
    rc = L.fg_spmm_csr_f32(None, None, None, None, None, 0, None, 0, 4, 4, 0, 0, 0, None)
    assert rc == 1 and b"bad sizes" in L.fg_last_error()
    rc = L.fg_spmm_csr_f32(None, None, None, None, None, 0, None, 0, 4, 4, 0, 8, 48, None)
    assert rc == 1 and b"feat_tile" in L.fg_last_error()
    rc = L.fg_sddmm_coo_f32(None, None, None, 0, None, 0, None, 4, 4, 5, 8, 0, 0, 0, None)
    assert rc == 1 and b"NULL" in L.fg_last_error()
    assert L.fg_sddmm_coo_f32(None, None, None, 0, None, 0, None, 4, 4, 0, 8, 0, 0, 0, None) == 0
    rc = L.fg_spmm_csr_f32(None, None, None, None, None, 4, None, 0, 4, 4, 0, 8, 0, None)
    assert rc == 1 and b"row strides" in L.fg_last_error()
    with pytest.raises(_native.FeatGraphError):
        _native.check(rc)


def test_modules_refuse_to_run_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from featgraph.module import VanillaSDDMMcuda, VanillaSpMMcuda, VanillaSpMMx86
    adj = sp.random(8, 8, density=0.5, format="csr", random_state=0).astype("float32")
    for make in (lambda: VanillaSpMMcuda(adj), lambda: VanillaSpMMx86(adj, 2),
                 lambda: VanillaSDDMMcuda(adj.tocoo().astype("int32"))):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            make()


def test_reference_import_paths_and_op_names():
    import featgraph.module as m
    import featgraph.op as op
    import featgraph.util as u
    for name in ("VanillaSpMMx86", "VanillaSpMMcuda", "VanillaSDDMMx86", "VanillaSDDMMcuda"):
        assert hasattr(m, name)
    assert m.VanillaSpMM is m.VanillaSpMMcuda and m.VanillaSDDMM is m.VanillaSDDMMcuda
    for name in ("util_convert_csr_to_dds", "util_partition_adj_coo_2d"):
        assert hasattr(u, name)
    # python/featgraph/op/__init__.py:1-5
    for name in ("vanilla_sddmm", "schedule_vanilla_sddmm_x86", "schedule_vanilla_sddmm_cuda_tree_reduce",
                 "schedule_vanilla_sddmm_cuda_single_thread_reduce", "vanilla_spmm_csr_x86",
                 "schedule_vanilla_spmm_csr_x86", "vanilla_spmm_dds_x86", "schedule_vanilla_spmm_dds_x86",
                 "vanilla_spmm_csr_cuda", "schedule_vanilla_spmm_csr_cuda"):
        assert callable(getattr(op, name))
    from featgraph import placeholder
    spec = op.vanilla_sddmm(placeholder((9, 16)), placeholder((7, 16)), placeholder((30,), "int32"),
                            placeholder((30,), "int32"))
    assert spec.shape == (30,)
    with pytest.raises(AssertionError):
        op.schedule_vanilla_sddmm_cuda_tree_reduce(spec, num_cuda_blocks=31)


def test_graph_generators_are_deterministic_and_well_formed():
    from featgraph_b200 import graphgen as g
    a = g.fixed_degree_graph(500, 20, seed=1)
    b = g.fixed_degree_graph(500, 20, seed=1)
    assert np.array_equal(a.indices, b.indices) and a.indices.dtype == np.int32
    assert np.all(np.diff(a.indptr) == 20) and np.all(a.data == 1.0) and a.data.dtype == np.float32
    for r in range(500):
        row = a.indices[a.indptr[r]:a.indptr[r + 1]]
        assert np.all(np.diff(row) > 0) and row.min() >= 0 and row.max() < 500
    assert not np.array_equal(a.indices, g.fixed_degree_graph(500, 20, seed=2).indices)

    p = g.power_law_graph(2000, 100_000, seed=3, kmax=400)
    deg = np.diff(p.indptr)
    assert p.nnz == 100_000 and deg.min() >= 1 and deg.max() <= 400
    assert np.median(deg) < deg.mean()  # heavy tail
    for r in (0, 7, 1999):
        row = p.indices[p.indptr[r]:p.indptr[r + 1]]
        assert np.all(np.diff(row) > 0)

    r = g.rmat_graph(10, 8, seed=4)
    assert r.shape == (1024, 1024) and 0 < r.nnz <= 8 * 1024
    coo = r.tocoo()
    assert np.all(coo.row != coo.col)
    keys = coo.row.astype(np.int64) * 1024 + coo.col
    assert np.all(np.diff(keys) > 0)  # sorted, no duplicates

    x = g.uniform_features((64, 8), seed=5)
    assert x.dtype == np.float32 and x.min() >= -1.0 and x.max() < 1.0
    assert np.array_equal(x, g.uniform_features((64, 8), seed=5))


def test_loading_the_library_rebuilds_it_when_a_source_is_newer(monkeypatch):
    """An edited kernel must never be tested against a stale binary: lib() asks build_cuda() to bring the
    library up to date, and build_cuda() compiles exactly when a source or header is newer than the .so."""
    import time
    from featgraph_b200 import _native, build
    build.build_cuda()
    assert not build.cuda_stale()
    src = os.path.join(build.CSRC, "validate.cu")
    st = os.stat(src)
    try:
        os.utime(src, (time.time() + 60, time.time() + 60))
        assert build.cuda_stale()
        # what lib() does on first use: it must reach the compiler for a stale library
        asked = []
        monkeypatch.setattr(build, "build_cuda", lambda force=False, **kw: asked.append(force) or build.CUDA_LIB)
        monkeypatch.setattr(_native, "_lib", None)
        _native.lib()
        assert asked == [False]
    finally:
        os.utime(src, (st.st_atime, st.st_mtime))
    assert not build.cuda_stale()
    # a library named by FEATGRAPH_B200_LIB is loaded as it is, without a build
    asked.clear()
    monkeypatch.setenv("FEATGRAPH_B200_LIB", build.CUDA_LIB)
    monkeypatch.setattr(_native, "_lib", None)
    _native.lib()
    assert asked == []


def test_ncu_traffic_table_is_tied_to_the_kernel_signature():
    """bench.py trusts profiles/ncu_traffic.json only while the loaded library reports the kernel shapes the
    table was captured from; any other signature makes the table 'stale' instead of silently wrong."""
    import importlib.util
    import json
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    rec = json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json")))
    assert sorted((c["op"], c["d"]) for c in rec["calls"]) == sorted(
        (op, d) for op in ("spmm", "sddmm") for d in (32, 64, 128, 256, 512))
    table, note = bench.load_ncu_traffic(rec["kernel_signature"])
    assert len(table) == 10 and all(v > 0 for v in table.values()) and "stale" not in note
    table, note = bench.load_ncu_traffic(rec["kernel_signature"] + "+changed")
    assert table == {} and "stale" in note
    from featgraph_b200 import _native
    assert _native.lib().fg_kernel_signature().decode() == rec["kernel_signature"], \
        "kernel shapes changed since profiles/ncu_traffic.json was captured: re-capture it " \
        "(python -m featgraph_b200.benchmark.ncu_traffic)"


def test_header_is_plain_c():
    """The boundary is a C ABI: include/featgraph_b200.h must compile as C99 on its own."""
    import shutil
    import subprocess
    import tempfile
    cc = shutil.which("gcc") or shutil.which("cc")
    if not cc:
        pytest.skip("no C compiler")
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "use_header.c")
        open(src, "w").write('#include "featgraph_b200.h"\nint main(void) { return FG_OK; }\n')
        r = subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                            "-fsyntax-only", src], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
