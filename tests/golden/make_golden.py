"""Regenerates the golden fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py [path-to-reference-checkout]

Needs the reference checkout (default: ``reference`` under the home directory) only for the partition cases: its
``python/featgraph/util/adj_partitioning.py`` is loaded by file path (it depends on numpy and
scipy alone) and run on seeded random matrices.  The SpMM / SDDMM cases store what the
reference's own tests compare against - ``adj.dot(X)`` (tests/test_module_spmm.py:29) and
``(Src[col] * Dst[row]).sum(-1)`` (tests/test_module_sddmm.py:34-36) - on the reference's test
shape (127 x 255, density 0.1, feat_len 128), with seeded inputs so that the files reproduce.
"""
import importlib.util
import os
import sys

import numpy as np
import scipy.sparse as sp

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_util(ref_root):
    path = os.path.join(ref_root, "python", "featgraph", "util", "adj_partitioning.py")
    spec = importlib.util.spec_from_file_location("reference_adj_partitioning", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def partition_cases(ref):
    rng = np.random.default_rng(20200)
    out = {}
    shapes = [(5, 5, 0.4), (127, 255, 0.1), (64, 17, 0.3), (1, 40, 0.5), (33, 1, 0.6), (50, 50, 0.0)]
    for i, (n, m, dens) in enumerate(shapes):
        seed = int(rng.integers(1 << 30))
        csr = sp.random(n, m, density=dens, format="csr", random_state=seed).astype("float32")
        coo = sp.random(n, m, density=dens, format="coo", random_state=seed + 1).astype("int32")
        out["c%d_shape" % i] = np.array([n, m], dtype=np.int64)
        out["c%d_csr_indptr" % i] = csr.indptr
        out["c%d_csr_indices" % i] = csr.indices
        out["c%d_csr_data" % i] = csr.data
        out["c%d_coo_row" % i] = coo.row
        out["c%d_coo_col" % i] = coo.col
        for P in (1, 2, 3, 4, 7):
            s1_pos, s1_idx, vals = ref.util_convert_csr_to_dds(csr, P)
            out["c%d_dds%d_pos" % (i, P)] = s1_pos
            out["c%d_dds%d_idx" % (i, P)] = s1_idx
            out["c%d_dds%d_vals" % (i, P)] = vals
        for Pr, Pc in ((1, 1), (2, 2), (4, 4), (3, 5), (8, 1)):
            ids, r, c = ref.util_partition_adj_coo_2d(coo.copy(), Pr, Pc)
            out["c%d_p2d%dx%d_ids" % (i, Pr, Pc)] = ids
            out["c%d_p2d%dx%d_row" % (i, Pr, Pc)] = r
            out["c%d_p2d%dx%d_col" % (i, Pr, Pc)] = c
    out["num_cases"] = np.array(len(shapes))
    return out


def numeric_cases():
    n, m, d = 127, 255, 128
    csr = sp.random(n, m, density=0.1, format="csr", random_state=127255).astype("float32")
    rng = np.random.default_rng(128)
    x = rng.random((m, d), dtype=np.float32)          # U[0,1) as in the reference's tests
    y = rng.random((n, d), dtype=np.float32)
    coo = sp.random(n, m, density=0.1, format="coo", random_state=255127).astype("int32")
    return dict(
        csr_indptr=csr.indptr, csr_indices=csr.indices, csr_data=csr.data, x=x, y=y,
        spmm_scipy=csr.dot(x).astype(np.float32),
        coo_row=coo.row, coo_col=coo.col,
        sddmm_numpy=(x[coo.col] * y[coo.row]).sum(axis=-1).astype(np.float32),
    )


if __name__ == "__main__":
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.expanduser("~"), "reference")
    ref = load_reference_util(ref_root)
    np.savez_compressed(os.path.join(HERE, "partition_cases.npz"), **partition_cases(ref))
    np.savez_compressed(os.path.join(HERE, "numeric_cases.npz"), **numeric_cases())
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
