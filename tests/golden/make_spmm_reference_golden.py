"""Regenerates spmm_reference_tvm.npz: outputs of the REFERENCE'S OWN SpMM compute definitions.

Same route as make_sddmm_reference_golden.py: the reference's python/featgraph/op/vanilla_spmm.py is
loaded by file path and its compute definitions - vanilla_spmm_csr_x86 (:6-62), vanilla_spmm_csr_cuda
(:83-125), vanilla_spmm_dds_x86 (:149-224) - are lowered with te.create_prim_func and compiled with
the C backend of the TVM fork bundled in the `tilelang` package (0.23.dev0).  One repair is needed for
that fork to compile them: the data-dependent reduce extent (indptr[row+1] - indptr[row]) is left in
the lowered function as a load from the tensor-expression placeholder, which later passes cannot hash;
`as_buffer_loads` rewrites those loads into loads from the function's own buffer of the same name.
Nothing about the arithmetic or the loop order is touched.  The default (schedule-less) loop nest adds
a row's nonzeros in storage order, as the reference's x86 schedule does (:73).

The DDS inputs come from the reference's own util_convert_csr_to_dds, also loaded by path.

    python tests/golden/make_spmm_reference_golden.py [path-to-reference-checkout]
"""
import importlib.util
import os
import sys

import numpy as np
import scipy.sparse as sp

HERE = os.path.dirname(os.path.abspath(__file__))


def cases():
    """(name, n_rows, n_cols, d, kind, num_feat_partitions, num_col_partitions, seed, density).

    The DDS cases are dense enough that no (column partition, row) segment is empty: the fork's
    lowering runs a reduction's init inside its loop, so a zero-length segment would leave the
    (uninitialised) intermediate untouched.  For the same reason the output array is zero-filled
    before each call, which is also what the reference's module does (module/spmm.py:110-111)."""
    return [("csr_x86_127x255_d128_p1", 127, 255, 128, "csr_x86", 1, 1, 21, 0.1),
            ("csr_x86_127x255_d128_p4", 127, 255, 128, "csr_x86", 4, 1, 22, 0.1),
            ("csr_cuda_127x255_d128", 127, 255, 128, "csr_cuda", 1, 1, 23, 0.1),
            ("csr_x86_300x90_d36_p1", 300, 90, 36, "csr_x86", 1, 1, 24, 0.1),
            ("dds_x86_127x255_d128_c4_p1", 127, 255, 128, "dds_x86", 1, 4, 25, 0.3),
            ("dds_x86_127x255_d128_c4_p4", 127, 255, 128, "dds_x86", 4, 4, 26, 0.3),
            ("dds_x86_60x77_d64_c7_p2", 60, 77, 64, "dds_x86", 2, 7, 27, 0.8)]


def inputs(n_rows, n_cols, d, seed, density):
    """Random CSR with non-unit values in [-1, 1) and features in [-1, 1)."""
    adj = sp.random(n_rows, n_cols, density=density, format="csr", random_state=seed).astype(np.float32)
    rng = np.random.default_rng(seed)
    adj.data = (rng.random(adj.nnz, dtype=np.float32) * 2 - 1).astype(np.float32)
    x = (rng.random((n_cols, d), dtype=np.float32) * 2 - 1).astype(np.float32)
    return adj, x


def _load(ref_root, rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    import tilelang  # noqa: F401  (puts its TVM fork on the import path)
    import tvm
    from tvm import te, tir

    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.expanduser("~"), "reference")
    ref_op = _load(ref_root, "python/featgraph/op/vanilla_spmm.py", "reference_vanilla_spmm")
    ref_util = _load(ref_root, "python/featgraph/util/adj_partitioning.py", "reference_adj_partitioning")

    def as_buffer_loads(func):
        buffers = {b.name: b for b in func.buffer_map.values()}

        def post(expr):
            if isinstance(expr, tir.ProducerLoad):
                return tir.BufferLoad(buffers[expr.producer.name], list(expr.indices))
            return None

        return func.with_body(tir.stmt_functor.ir_transform(func.body, None, post, ["tir.ProducerLoad"]))

    dev = tvm.cpu(0)
    out = {"tvm_version": np.array(tvm.__version__)}
    for name, n_rows, n_cols, d, kind, nfp, ncp, seed, density in cases():
        adj, x = inputs(n_rows, n_cols, d, seed, density)
        X = te.placeholder((n_cols, d), name="SrcFeat")
        if kind == "dds_x86":
            s1_pos, s1_idx, vals = ref_util.util_convert_csr_to_dds(adj, ncp)
            seg = np.diff(s1_pos.reshape(ncp, n_rows + 1), axis=1)
            assert seg.min() > 0, "case %s has an empty (partition, row) segment" % name
            arrays = (s1_pos, s1_idx, vals)
            P = te.placeholder(s1_pos.shape, dtype="int32", name="Adj_s1_pos")
            I = te.placeholder(s1_idx.shape, dtype="int32", name="Adj_s1_idx")
            V = te.placeholder(vals.shape, dtype="float32", name="Adj_vals")
            Out = ref_op.vanilla_spmm_dds_x86(X, P, I, V, ncp, n_rows + 1, num_feat_partitions=nfp)
        else:
            arrays = (adj.indptr, adj.indices, adj.data)
            P = te.placeholder(adj.indptr.shape, dtype="int32", name="Adj_indptr")
            I = te.placeholder(adj.indices.shape, dtype="int32", name="Adj_indices")
            V = te.placeholder(adj.data.shape, dtype="float32", name="Adj_vals")
            if kind == "csr_x86":
                Out = ref_op.vanilla_spmm_csr_x86(X, P, I, V, num_feat_partitions=nfp)
            else:
                Out = ref_op.vanilla_spmm_csr_cuda(X, P, I, V)
        func = as_buffer_loads(te.create_prim_func([X, P, I, V, Out]))
        lib = tvm.compile(tvm.IRModule({"main": func}), target="c")
        args = [tvm.runtime.tensor(a, dev) for a in (x, *arrays, np.zeros((n_rows, d), np.float32))]
        lib["main"](*args)
        out[name] = args[-1].numpy()
        print(name, out[name].shape, float(np.abs(out[name]).max()))
    np.savez_compressed(os.path.join(HERE, "spmm_reference_tvm.npz"), **out)
