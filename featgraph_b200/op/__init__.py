"""Names of the reference's ``featgraph.op`` (python/featgraph/op/__init__.py:1-5).

In the reference these functions describe a computation and a loop schedule to a code
generator.  There is no code generator here: each compute function returns an ``OpSpec``
naming the C-ABI entry point that implements the same math, and each schedule function
returns the spec with its knobs recorded (they never change a result).  The module
classes do not go through these; they exist so that code which imports the names still
loads and can inspect what would run.
"""
from ..placeholder import static_shape


class OpSpec:
    def __init__(self, kind, entry_point, out_shape, **knobs):
        self.kind = kind
        self.entry_point = entry_point
        self.shape = tuple(out_shape)
        self.dtype = "float32"
        self.knobs = dict(knobs)

    def with_knobs(self, **knobs):
        merged = dict(self.knobs)
        merged.update({k: v for k, v in knobs.items() if v is not None})
        return OpSpec(self.kind, self.entry_point, self.shape, **merged)

    def __repr__(self):
        return "OpSpec(%s -> %s, shape=%s, knobs=%s)" % (self.kind, self.entry_point, self.shape, self.knobs)


def _feat(SrcFeat, num_feat_partitions):
    n, d = static_shape(SrcFeat)
    assert d % num_feat_partitions == 0, "feat_len must be divisible by num_feat_partitions"
    return n, d


def vanilla_spmm_csr_x86(SrcFeat, Adj_indptr, Adj_indices, Adj_vals, num_feat_partitions=1):
    """python/featgraph/op/vanilla_spmm.py:6-62."""
    assert static_shape(Adj_indices)[0] == static_shape(Adj_vals)[0]
    _, d = _feat(SrcFeat, num_feat_partitions)
    return OpSpec("spmm_csr", "fg_spmm_csr_f32", (static_shape(Adj_indptr)[0] - 1, d),
                  num_feat_partitions=num_feat_partitions)


def schedule_vanilla_spmm_csr_x86(Out):
    """python/featgraph/op/vanilla_spmm.py:65-80."""
    return Out


def vanilla_spmm_csr_cuda(SrcFeat, Adj_indptr, Adj_indices, Adj_vals):
    """python/featgraph/op/vanilla_spmm.py:83-125."""
    return vanilla_spmm_csr_x86(SrcFeat, Adj_indptr, Adj_indices, Adj_vals, 1)


def schedule_vanilla_spmm_csr_cuda(Out, num_cuda_blocks=None, num_threads_per_cuda_block=None):
    """python/featgraph/op/vanilla_spmm.py:128-146."""
    return Out.with_knobs(num_cuda_blocks=num_cuda_blocks,
                          num_threads_per_cuda_block=num_threads_per_cuda_block)


def vanilla_spmm_dds_x86(SrcFeat, Adj_s1_pos, Adj_s1_idx, Adj_vals, d1_size, d2_size,
                         num_feat_partitions=1):
    """python/featgraph/op/vanilla_spmm.py:149-224."""
    assert d1_size * d2_size == static_shape(Adj_s1_pos)[0]
    assert static_shape(Adj_s1_idx)[0] == static_shape(Adj_vals)[0]
    _, d = _feat(SrcFeat, num_feat_partitions)
    return OpSpec("spmm_dds", "fg_spmm_dds_f32", (d2_size - 1, d),
                  num_feat_partitions=num_feat_partitions, num_col_partitions=d1_size)


def schedule_vanilla_spmm_dds_x86(Out):
    """python/featgraph/op/vanilla_spmm.py:227-246."""
    return Out


def vanilla_sddmm(SrcFeat, DstFeat, Adj_row_indices, Adj_col_indices, num_feat_partitions=1):
    """python/featgraph/op/vanilla_sddmm.py:6-63."""
    d = static_shape(SrcFeat)[1]
    assert static_shape(DstFeat)[1] == d, "dimension mismatch"
    num_edges = static_shape(Adj_row_indices)[0]
    assert static_shape(Adj_col_indices)[0] == num_edges, "dimension mismatch"
    assert d % num_feat_partitions == 0
    return OpSpec("sddmm", "fg_sddmm_coo_f32", (num_edges,), num_feat_partitions=num_feat_partitions)


def schedule_vanilla_sddmm_x86(Out, num_feat_partitions=1):
    """python/featgraph/op/vanilla_sddmm.py:66-74."""
    return Out.with_knobs(num_feat_partitions=num_feat_partitions)


def schedule_vanilla_sddmm_cuda_tree_reduce(Out, num_feat_partitions=1, num_cuda_blocks=8192):
    """python/featgraph/op/vanilla_sddmm.py:77-89."""
    assert num_feat_partitions == 1, "cuda schedule for sddmm does not support feat dimension tiling, " \
                                     "which requires cross-cuda-block reduction and atomic operations."
    num_edges = Out.shape[0]
    assert num_cuda_blocks <= num_edges, "num_cuda_blocks must be smaller than num_edges, " \
                                         "which is {}.".format(num_edges)
    return Out.with_knobs(num_cuda_blocks=num_cuda_blocks, reduce="tree")


def schedule_vanilla_sddmm_cuda_single_thread_reduce(Out, num_feat_partitions=1,
                                                     num_threads_per_cuda_block=32):
    """python/featgraph/op/vanilla_sddmm.py:92-100."""
    assert num_feat_partitions == 1, "cuda schedule for sddmm does not support feat dimension tiling, " \
                                     "which requires cross-cuda-block reduction and atomic operations."
    return Out.with_knobs(num_threads_per_cuda_block=num_threads_per_cuda_block, reduce="single_thread")


__all__ = [
    "vanilla_sddmm", "schedule_vanilla_sddmm_x86", "schedule_vanilla_sddmm_cuda_tree_reduce",
    "schedule_vanilla_sddmm_cuda_single_thread_reduce", "vanilla_spmm_csr_x86",
    "schedule_vanilla_spmm_csr_x86", "vanilla_spmm_dds_x86", "schedule_vanilla_spmm_dds_x86",
    "vanilla_spmm_csr_cuda", "schedule_vanilla_spmm_csr_cuda", "OpSpec",
]
