"""One graph over several GPUs: rows sharded in nnz-balanced contiguous ranges, one process per
GPU (``torch.distributed``).  The reference is single-device (``tvm.gpu(0)`` is hard-wired,
python/featgraph/module/spmm.py:218); this layer is what spreads its two ops over a node.

SpMM: rank p owns rows ``[bounds[p], bounds[p+1])`` of the adjacency (column ids stay global)
and the same rows of the feature matrix.  A call all-gathers the feature rows into every
rank's own memory (the one exchange step the op has), then runs the single-GPU kernel on the
local rows; the output stays sharded.  No row is ever split, so each output element is summed
exactly as on one GPU.

SDDMM: rank p owns the edges of its rows (a contiguous range of the CSR-ordered edge list).  The
row-side features are local, the column-side features are all-gathered; the per-edge output
stays sharded (concatenating the ranks' outputs gives the single-GPU output).

The host-side bookkeeping (ranges, local CSR slices, the gather itself) runs unchanged on CPU
tensors with the gloo backend; only ``run`` needs a GPU.
"""
import numpy as np
import scipy.sparse
import torch
import torch.distributed as dist

from .util import nnz_balanced_row_ranges


def shard_csr_rows(adj_csr, bounds, rank):
    """Rows ``[bounds[rank], bounds[rank+1])`` of a CSR matrix as a CSR matrix of the same width:
    indptr rebased to start at 0, column ids untouched."""
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    e0, e1 = int(adj_csr.indptr[lo]), int(adj_csr.indptr[hi])
    indptr = (adj_csr.indptr[lo:hi + 1] - adj_csr.indptr[lo]).astype(adj_csr.indptr.dtype)
    local = scipy.sparse.csr_matrix((adj_csr.data[e0:e1], adj_csr.indices[e0:e1], indptr),
                                    shape=(hi - lo, adj_csr.shape[1]))
    return local


def all_gather_rows(full, local, bounds, group=None):
    """``full[bounds[p]:bounds[p+1]] = rank p's local`` on every rank.  Row counts differ between
    ranks.  NCCL does this as one grouped operation writing straight into ``full``; other
    backends get one broadcast per rank."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    if tuple(local.shape[1:]) != tuple(full.shape[1:]) or local.shape[0] != hi - lo:
        raise ValueError("local block has shape %s, rank %d owns rows [%d, %d)" % (tuple(local.shape), rank, lo, hi))
    if world == 1:
        full[lo:hi].copy_(local)
        return full
    views = [full[int(bounds[p]):int(bounds[p + 1])] for p in range(world)]
    if dist.get_backend(group) == "nccl":
        dist.all_gather(views, local.contiguous(), group=group)
    else:
        views[rank].copy_(local)
        for p in range(world):
            if views[p].numel():
                dist.broadcast(views[p], src=dist.get_global_rank(group, p) if group is not None else p,
                               group=group)
    return full


class _ShardedBase:
    def __init__(self, bounds, group, device):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.bounds = np.asarray(bounds, dtype=np.int64)
        assert self.bounds.shape[0] == self.world + 1
        self.row_lo, self.row_hi = int(self.bounds[self.rank]), int(self.bounds[self.rank + 1])
        self.device = device

    def _gather(self, full, local):
        if not dist.is_initialized():
            full[self.row_lo:self.row_hi].copy_(local)
            return full
        return all_gather_rows(full, local, self.bounds, self.group)


class ShardedSpMM(_ShardedBase):
    """Row-sharded SpMM for a square adjacency.

    ``local_adj``: this rank's rows (``shard_csr_rows``), ``bounds``: the row ranges of all ranks
    (``nnz_balanced_row_ranges`` of the whole graph's indptr)."""

    def __init__(self, local_adj, bounds, group=None, device=None):
        from .module import VanillaSpMMcuda
        super().__init__(bounds, group, device)
        assert local_adj.shape[0] == self.row_hi - self.row_lo
        assert local_adj.shape[1] == int(self.bounds[-1]), "square adjacency expected (features are row-sharded)"
        self.module = VanillaSpMMcuda(local_adj, device=device)
        self.device = self.module.ctx
        self.n = local_adj.shape[1]
        self.x_full = None

    def build(self, feat_len, feat_tile=0):
        from .placeholder import placeholder
        self.module.build([placeholder((self.n, feat_len))], {}, {"feat_tile": feat_tile})
        self.x_full = torch.empty((self.n, feat_len), dtype=torch.float32, device=self.device)

    def gather(self, x_local):
        """The exchange step alone: every rank's feature rows into this rank's ``x_full``."""
        return self._gather(self.x_full, x_local)

    def compute(self):
        """The local kernel alone, on the features gathered last."""
        return self.module.run([self.x_full])

    def run(self, x_local):
        """x_local: this rank's rows of the feature matrix.  Returns this rank's rows of A.X."""
        self.gather(x_local)
        return self.compute()


class ShardedSDDMM(_ShardedBase):
    """Edge-sharded SDDMM by the same row ranges (square adjacency)."""

    def __init__(self, local_adj, bounds, group=None, device=None):
        from .module import VanillaSDDMMcuda
        super().__init__(bounds, group, device)
        assert local_adj.shape[0] == self.row_hi - self.row_lo
        self.module = VanillaSDDMMcuda(local_adj.tocoo(), device=device)
        self.device = self.module.ctx
        self.n = local_adj.shape[1]
        self.src_full = None

    def build(self, feat_len):
        from .placeholder import placeholder
        self.module.build([placeholder((self.n, feat_len)), placeholder((self.row_hi - self.row_lo, feat_len))], {}, {})
        self.src_full = torch.empty((self.n, feat_len), dtype=torch.float32, device=self.device)

    def gather(self, src_local):
        return self._gather(self.src_full, src_local)

    def compute(self, dst_local):
        return self.module.run([self.src_full, dst_local])

    def run(self, src_local, dst_local):
        """src_local: this rank's rows of the column-side matrix (gathered from all ranks);
        dst_local: this rank's rows of the row-side matrix.  Returns this rank's edges' dots."""
        self.gather(src_local)
        return self.compute(dst_local)
