import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# Tolerance the hot path is held to against the CPU oracle for floating point
# (SDDMM; SpMM is compared bit for bit).
RTOL = 1e-5
ATOL = 1e-4


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def numeric_golden():
    return dict(np.load(os.path.join(GOLDEN, "numeric_cases.npz")))


@pytest.fixture(scope="session")
def partition_golden():
    return dict(np.load(os.path.join(GOLDEN, "partition_cases.npz")))


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle
    _oracle.lib()
    return _oracle


def reference_util_or_skip():
    """The reference's own partitioners, loaded by file path, or skip where the checkout is absent."""
    import importlib.util
    root = os.environ.get("FEATGRAPH_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))
    path = os.path.join(root, "python", "featgraph", "util", "adj_partitioning.py")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present on this machine")
    spec = importlib.util.spec_from_file_location("reference_adj_partitioning", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sddmm_reference_cases():
    """(name, row, col, src, dst, num_feat_partitions, reference_output) for every case of
    tests/golden/sddmm_reference_tvm.npz (outputs of the reference's own SDDMM definition compiled by a
    TVM build; inputs are re-created from their seeds by the generating script's own functions)."""
    import importlib.util
    path = os.path.join(GOLDEN, "make_sddmm_reference_golden.py")
    spec = importlib.util.spec_from_file_location("make_sddmm_reference_golden", path)
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    fixture = np.load(os.path.join(GOLDEN, "sddmm_reference_tvm.npz"))
    for name, n_rows, n_cols, d, nfp, seed in gen.cases():
        row, col, src, dst = gen.inputs(n_rows, n_cols, d, seed)
        yield name, row, col, src, dst, nfp, fixture[name]


def spmm_reference_cases():
    """(name, kind, adj, x, num_feat_partitions, num_col_partitions, reference_output) for every case of
    tests/golden/spmm_reference_tvm.npz (outputs of the reference's own SpMM definitions compiled by a TVM
    build; inputs are re-created from their seeds by the generating script's own functions)."""
    import importlib.util
    path = os.path.join(GOLDEN, "make_spmm_reference_golden.py")
    spec = importlib.util.spec_from_file_location("make_spmm_reference_golden", path)
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    fixture = np.load(os.path.join(GOLDEN, "spmm_reference_tvm.npz"))
    for name, n_rows, n_cols, d, kind, nfp, ncp, seed, density in gen.cases():
        adj, x = gen.inputs(n_rows, n_cols, d, seed, density)
        yield name, kind, adj, x, nfp, ncp, fixture[name]
