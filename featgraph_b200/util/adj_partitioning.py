"""Host-side adjacency re-layouts behind the ``num_col_partitions`` / ``num_row_partitions`` knobs.

Same names, arguments, return values and dtypes as the reference's
``python/featgraph/util/adj_partitioning.py`` (``util_convert_csr_to_dds`` :7-57,
``util_partition_adj_coo_2d`` :60-128), but computed with one stable sort over all
nonzeros instead of a Python loop of scipy sub-matrix slices, so a 10^8-edge graph
costs seconds.  Results are bit-identical to the reference's (pinned by its golden
vectors, tests/test_util.py:22-24,43, and by randomised comparison with the reference
functions themselves).

``nnz_balanced_row_ranges`` has no counterpart in the reference (which is single
device): it is the row sharding used when one graph is spread over several GPUs.
"""
import numpy as np
import scipy.sparse


def _ceil_div(a, b):
    return (a + b - 1) // b


def util_convert_csr_to_dds(adj_scipy_csr, num_col_partitions):
    """Column (source-vertex) partitioning: CSR -> dense-dense-sparse arrays.

    Column block k covers ``[k*w, (k+1)*w)`` with ``w = ceil(num_cols / num_col_partitions)``;
    the last block takes whatever is left (reference :42-47).  The output lists block
    0's nonzeros row by row, then block 1's, ...; inside a (block, row) segment the
    nonzeros keep their CSR storage order.  ``s1_pos`` holds, per block, the
    ``num_rows + 1`` segment boundaries as absolute positions (reference :50);
    ``s1_idx`` holds column ids relative to the block's first column.

    Returns ``(s1_pos, s1_idx, vals)`` with the dtypes of ``indptr``, ``indices``, ``data``.
    """
    num_rows, num_cols = adj_scipy_csr.shape
    indptr = np.asarray(adj_scipy_csr.indptr)
    indices = np.asarray(adj_scipy_csr.indices)
    data = np.asarray(adj_scipy_csr.data)
    nnz = indices.shape[0]
    P = int(num_col_partitions)
    d2 = indptr.shape[0]
    w = _ceil_div(num_cols, P)

    if nnz == 0:
        return (np.zeros(P * d2, dtype=indptr.dtype), np.zeros(0, dtype=indices.dtype),
                np.zeros(0, dtype=data.dtype))
    # block of every nonzero; columns past (P-1)*w all belong to the last block
    block = np.minimum(indices.astype(np.int64) // max(w, 1), P - 1)
    if w == 0:
        block[:] = P - 1
    rows = np.repeat(np.arange(num_rows, dtype=np.int64), np.diff(indptr).astype(np.int64))
    key = block * num_rows + rows
    order = np.argsort(key, kind="stable")
    s1_idx = (indices[order].astype(np.int64) - block[order] * w).astype(indices.dtype)
    vals = data[order]
    counts = np.bincount(key, minlength=P * num_rows).reshape(P, num_rows)
    seg_end = np.cumsum(counts.ravel()).reshape(P, num_rows)
    s1_pos = np.empty((P, d2), dtype=np.int64)
    s1_pos[:, 1:] = seg_end
    s1_pos[0, 0] = 0
    s1_pos[1:, 0] = seg_end[:-1, -1]
    return s1_pos.ravel().astype(indptr.dtype), s1_idx, vals


def util_partition_adj_coo_2d(adj_scipy_coo, num_row_partitions, num_col_partitions):
    """2-D partitioning of an edge list into row-block x column-block tiles.

    Row blocks are ``ceil(num_rows / num_row_partitions)`` tall, column blocks
    ``ceil(num_cols / num_col_partitions)`` wide, the last of each takes the rest
    (reference :100-101, :105-119).  Tiles are visited row-block-major (:103-104);
    inside a tile edges come in (row, column) order, because the reference slices a
    CSR matrix made with ``tocsr()``, which sorts each row's columns (:95).

    Returns ``(edge_ids, rows, cols)``: ``edge_ids`` are the 1-based positions of the
    edges in the input COO arrays (int32), ``rows`` / ``cols`` keep the input's index
    dtype.  As in the reference (:92) the input matrix's ``data`` is REPLACED by
    ``arange(1, nnz + 1, dtype=int32)``.

    Duplicate (row, col) entries raise ``ValueError``: the reference's ``tocsr()``
    would add their ids together and return arrays that describe no edge list.
    """
    num_rows, num_cols = adj_scipy_coo.shape
    row = np.asarray(adj_scipy_coo.row)
    col = np.asarray(adj_scipy_coo.col)
    nnz = row.shape[0]
    assert col.shape[0] == nnz, "length of adj_row_indices and that of adj_col_indices do not match"
    adj_scipy_coo.data = np.arange(1, 1 + nnz, dtype="int32")

    Pr, Pc = int(num_row_partitions), int(num_col_partitions)
    h = _ceil_div(num_rows, Pr)
    w = _ceil_div(num_cols, Pc)
    r64 = row.astype(np.int64)
    c64 = col.astype(np.int64)
    rb = np.minimum(r64 // max(h, 1), Pr - 1)
    cb = np.minimum(c64 // max(w, 1), Pc - 1)
    # one key, most significant first: row block, column block, row, column
    key = ((rb * Pc + cb) * max(num_rows, 1) + r64) * max(num_cols, 1) + c64
    order = np.argsort(key, kind="stable")
    if nnz > 1 and np.any(np.diff(key[order]) == 0):
        raise ValueError("util_partition_adj_coo_2d: duplicate (row, col) entries are not supported")
    edge_ids = (order + 1).astype(np.int32)
    return edge_ids, row[order], col[order]


def nnz_balanced_row_ranges(indptr, num_parts):
    """Split rows into ``num_parts`` contiguous ranges holding about equal nonzeros.

    ``bounds[p] = searchsorted(indptr, (p * nnz) // num_parts, side='left')`` with
    ``bounds[0] = 0`` and ``bounds[num_parts] = num_rows``; part ``p`` owns rows
    ``[bounds[p], bounds[p+1])``.  A row is never split, so per-row summation order is
    untouched.  Returns an int64 array of length ``num_parts + 1``.
    """
    indptr = np.asarray(indptr)
    n = indptr.shape[0] - 1
    nnz = int(indptr[-1])
    P = int(num_parts)
    assert P >= 1
    targets = (np.arange(P + 1, dtype=np.int64) * nnz) // P
    bounds = np.searchsorted(indptr, targets, side="left").astype(np.int64)
    bounds[0] = 0
    bounds[P] = n
    return np.minimum(np.maximum.accumulate(bounds), n)
