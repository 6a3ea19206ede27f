"""Regenerates sddmm_reference_tvm.npz: outputs of the REFERENCE'S OWN SDDMM compute definition.

The reference describes SDDMM to Apache TVM (python/featgraph/op/vanilla_sddmm.py:6-63).  The TVM
release it was written for is not installable here, but the TVM fork bundled with the `tilelang`
package (0.23.dev0) can lower that compute definition with te.create_prim_func and compile it with the
C backend (default loop nest: edge outer, k ascending inner - the order of the reference's x86
schedule, which for num_feat_partitions > 1 only hoists the outer part of k, op/vanilla_sddmm.py:66-74).
This script loads the reference file by path, runs it on seeded inputs and stores inputs' seeds and
outputs.  (The SpMM definitions need one repair before that fork compiles them; their fixture is made by
make_spmm_reference_golden.py beside this file.)

    python tests/golden/make_sddmm_reference_golden.py [path-to-reference-checkout]
"""
import importlib.util
import os
import sys

import numpy as np
import scipy.sparse as sp

HERE = os.path.dirname(os.path.abspath(__file__))


def cases():
    """(name, n_rows, n_cols, d, num_feat_partitions, seed): the reference's test shape and two more."""
    return [("t127x255_d128_p1", 127, 255, 128, 1, 11), ("t127x255_d128_p4", 127, 255, 128, 4, 12),
            ("t64x300_d36_p1", 64, 300, 36, 1, 13), ("t500x40_d512_p8", 500, 40, 512, 8, 14)]


def inputs(n_rows, n_cols, d, seed):
    coo = sp.random(n_rows, n_cols, density=0.1, format="coo", random_state=seed)
    rng = np.random.default_rng(seed)
    src = (rng.random((n_cols, d), dtype=np.float32) * 2 - 1).astype(np.float32)
    dst = (rng.random((n_rows, d), dtype=np.float32) * 2 - 1).astype(np.float32)
    return coo.row.astype(np.int32), coo.col.astype(np.int32), src, dst


if __name__ == "__main__":
    import tilelang  # noqa: F401  (puts its TVM fork on the import path)
    import tvm
    from tvm import te

    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.expanduser("~"), "reference")
    path = os.path.join(ref_root, "python", "featgraph", "op", "vanilla_sddmm.py")
    spec = importlib.util.spec_from_file_location("reference_vanilla_sddmm", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {"tvm_version": np.array(tvm.__version__)}
    dev = tvm.cpu(0)
    for name, n_rows, n_cols, d, nfp, seed in cases():
        row, col, src, dst = inputs(n_rows, n_cols, d, seed)
        Src = te.placeholder((n_cols, d), name="SrcFeat")
        Dst = te.placeholder((n_rows, d), name="DstFeat")
        R = te.placeholder((len(row),), dtype="int32", name="Adj_row_indices")
        C = te.placeholder((len(row),), dtype="int32", name="Adj_col_indices")
        Out = ref.vanilla_sddmm(Src, Dst, R, C, num_feat_partitions=nfp)
        lib = tvm.compile(tvm.IRModule({"main": te.create_prim_func([Src, Dst, R, C, Out])}), target="c")
        args = [tvm.runtime.tensor(a, dev) for a in (src, dst, row, col, np.zeros(len(row), np.float32))]
        lib["main"](*args)
        out[name] = args[-1].numpy()
        print(name, out[name].shape, float(np.abs(out[name]).max()))
    np.savez_compressed(os.path.join(HERE, "sddmm_reference_tvm.npz"), **out)
