"""One graph over several GPUs: rows sharded in nnz-balanced contiguous ranges, one process per
GPU (``torch.distributed``).  The reference is single-device (``tvm.gpu(0)`` is hard-wired,
python/featgraph/module/spmm.py:218); this layer is what spreads its two ops over a node.

SpMM: rank p owns rows ``[bounds[p], bounds[p+1])`` of the adjacency and the same rows of the
feature matrix.  A call all-gathers the feature rows into every rank's own memory (the one
exchange step the op has), then runs the single-GPU kernel on the local rows; the output stays
sharded.  No row is ever split, so each output element is summed exactly as on one GPU.
Row blocks differ in size.  Where they differ little (a graph whose rows are of similar weight) the
gather runs over equal slots of a padded buffer (one plain all-gather) and each shard's column ids
are remapped once, at construction, to point into it.  Where they differ much (nnz-balanced ranges
of an R-MAT graph: a few hub rows on one rank, a million light rows on another) padding would
multiply the bytes exchanged, so the blocks are gathered at their own sizes into the plain matrix.

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


class ExchangeError(RuntimeError):
    """The feature all-gather failed or timed out (a peer rank is gone or stuck).  Raised on the host;
    nothing is left running on the GPU by this layer, and the local modules stay usable."""


def all_gather_rows(full, local, bounds, group=None, async_op=False):
    """``full[bounds[p]:bounds[p+1]] = rank p's local`` on every rank.  Row counts differ between
    ranks.  NCCL does this as one grouped operation writing straight into ``full``; other
    backends get one broadcast per rank.  ``async_op`` (NCCL only) returns the work handle."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    if tuple(local.shape[1:]) != tuple(full.shape[1:]) or local.shape[0] != hi - lo:
        raise ValueError("local block has shape %s, rank %d owns rows [%d, %d)" % (tuple(local.shape), rank, lo, hi))
    if world == 1:
        full[lo:hi].copy_(local)
        return full
    views = [full[int(bounds[p]):int(bounds[p + 1])] for p in range(world)]
    try:
        if dist.get_backend(group) == "nccl":
            work = dist.all_gather(views, local.contiguous(), group=group, async_op=async_op)
            if async_op:
                return work
        else:
            views[rank].copy_(local)
            for p in range(world):
                if views[p].numel():
                    dist.broadcast(views[p], src=dist.get_global_rank(group, p) if group is not None else p,
                                   group=group)
    except Exception as exc:  # the process group's timeout, a closed connection, an aborted communicator
        raise ExchangeError("rank %d of %d: feature all-gather failed: %s" % (rank, world, exc)) from exc
    return full


def padded_layout(bounds):
    """Equal-sized slots for an all-gather of unequal row blocks: rank p's rows sit at
    ``[p*slot, p*slot + rows_p)`` of a ``world*slot``-row buffer.  Returns ``(slot, shift)`` with
    ``shift[p] = p*slot - bounds[p]``, the amount to add to a global row id owned by rank p."""
    bounds = np.asarray(bounds, dtype=np.int64)
    world = bounds.shape[0] - 1
    slot = int(np.diff(bounds).max()) if world > 0 else 0
    shift = np.arange(world, dtype=np.int64) * slot - bounds[:-1]
    return slot, shift


def remap_columns_to_padded(adj_csr, bounds):
    """Copy of a CSR row shard whose column ids point into the padded gather buffer.  The map is
    increasing, so the order of a row's nonzeros (and with it every sum) is unchanged."""
    slot, shift = padded_layout(bounds)
    world = len(shift)
    owner = np.searchsorted(np.asarray(bounds[1:], dtype=np.int64), adj_csr.indices, side="right")
    new_cols = (adj_csr.indices.astype(np.int64) + shift[owner]).astype(adj_csr.indices.dtype)
    out = scipy.sparse.csr_matrix((adj_csr.data, new_cols, adj_csr.indptr), shape=(adj_csr.shape[0], world * slot))
    return out


def all_gather_padded(padded, local, bounds, group=None):
    """All-gather of unequal row blocks through equal slots: ``padded[p*slot : p*slot + rows_p] =
    rank p's local`` on every rank, as ONE equal-sized all-gather (in place: each rank first copies
    its block into its own slot)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    slot, _ = padded_layout(bounds)
    rows = int(bounds[rank + 1] - bounds[rank])
    if tuple(local.shape[1:]) != tuple(padded.shape[1:]) or local.shape[0] != rows:
        raise ValueError("local block has shape %s, rank %d owns %d rows" % (tuple(local.shape), rank, rows))
    if padded.shape[0] != world * slot:
        raise ValueError("padded buffer has %d rows, want %d" % (padded.shape[0], world * slot))
    mine = padded[rank * slot:(rank + 1) * slot]
    mine[:rows].copy_(local)
    if world > 1:
        try:
            if dist.get_backend(group) == "nccl":
                dist.all_gather_into_tensor(padded, mine, group=group)
            else:
                dist.all_gather([padded[p * slot:(p + 1) * slot] for p in range(world)], mine.clone(), group=group)
        except Exception as exc:  # the process group's timeout, a closed connection, an aborted communicator
            raise ExchangeError("rank %d of %d: feature all-gather failed: %s" % (rank, world, exc)) from exc
    return padded


# Padding is worth it while the padded buffer is at most this much larger than the matrix.
PADDED_LAYOUT_MAX_WASTE = 1.15


def use_padded_layout(bounds):
    """True where equal slots cost little: ``world * largest block <= 1.15 * rows``."""
    bounds = np.asarray(bounds, dtype=np.int64)
    world = bounds.shape[0] - 1
    slot, _ = padded_layout(bounds)
    return world * slot <= PADDED_LAYOUT_MAX_WASTE * max(int(bounds[-1]), 1)


def remap_columns(adj_csr, bounds):
    """The shard with column ids pointing into the gather buffer of the layout chosen for ``bounds``
    (unchanged in the plain layout)."""
    return remap_columns_to_padded(adj_csr, bounds) if use_padded_layout(bounds) else adj_csr


# ---- host-buffer steps -------------------------------------------------------------------------------
# The single-GPU modules pipeline host copies inside one call (run_host -> fg_*_host).  A sharded call has
# the exchange between copy-in and kernel, so here the three stages are spread over streams of this
# layer: copy-in (host -> this rank's rows on the device, then the exchange behind it), the caller's
# compute stream (kernels), copy-out (results -> host).  Calls only enqueue; ``host_sync`` waits.  With
# the next call's copy-in and exchange issued before the current call's kernels, a step costs about
# max(copies in, kernels, copies out) instead of their sum.
_copy_streams = {}


def copy_streams(device):
    """(copy-in, copy-out) streams of this layer on ``device`` (created once per device)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _copy_streams:
        _copy_streams[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _copy_streams[key]


def host_sync(device):
    """Wait until every host-buffer call issued so far on ``device`` has delivered its result."""
    s_in, s_out = copy_streams(device)
    s_in.synchronize()
    torch.cuda.current_stream(device).synchronize()
    s_out.synchronize()


def copy_out_async(result, out_host, device, holder):
    """Enqueue ``out_host <- result`` on the copy-out stream behind what the compute stream holds now.
    The event of the copy is kept on ``holder`` under the result buffer's address: the next kernel that
    overwrites that buffer waits for it (``wait_for_copy_out``)."""
    _, s_out = copy_streams(device)
    done = torch.cuda.current_stream(device).record_event()
    s_out.wait_event(done)
    with torch.cuda.stream(s_out):
        out_host.copy_(result, non_blocking=True)
        holder.__dict__.setdefault("_out_done", {})[result.data_ptr()] = s_out.record_event()
    return out_host


def wait_for_copy_out(buffer, device, holder):
    """Make the compute stream wait until the last copy-out of ``buffer`` (if any) has left the device."""
    if buffer is None:
        return
    ev = holder.__dict__.get("_out_done", {}).pop(buffer.data_ptr(), None)
    if ev is not None:
        torch.cuda.current_stream(device).wait_event(ev)


class _ShardedBase:
    def __init__(self, bounds, group, device):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.bounds = np.asarray(bounds, dtype=np.int64)
        assert self.bounds.shape[0] == self.world + 1
        self.row_lo, self.row_hi = int(self.bounds[self.rank]), int(self.bounds[self.rank + 1])
        self.device = device
        self.slot, self.shift = padded_layout(self.bounds)
        self.padded = use_padded_layout(self.bounds)
        # rows of the gather buffer every rank holds
        self.n = self.world * self.slot if self.padded else int(self.bounds[-1])

    def _gather(self, buf, local):
        if self.padded:
            return all_gather_padded(buf, local, self.bounds, self.group)
        return all_gather_rows(buf, local, self.bounds, self.group)

    def _gather_async(self, buf, local):
        """Start the exchange (NCCL); returns the work handle."""
        try:
            if self.padded:
                rows = self.row_hi - self.row_lo
                mine = buf[self.rank * self.slot:(self.rank + 1) * self.slot]
                mine[:rows].copy_(local)
                return dist.all_gather_into_tensor(buf, mine, group=self.group, async_op=True)
            return all_gather_rows(buf, local, self.bounds, self.group, async_op=True)
        except ExchangeError:
            raise
        except Exception as exc:
            raise ExchangeError("rank %d of %d: feature all-gather failed: %s" % (self.rank, self.world, exc)) from exc


class GatheredFeatures(_ShardedBase):
    """A row-sharded feature matrix all-gathered ONCE into this rank's memory, for several ops to
    read: SpMM and SDDMM of one GNN layer gather from the same matrix, and exchanging it per op
    would double the NVLink traffic.  ``gather(x_local)`` returns ``self``; pass it to
    ``ShardedSpMM.run`` / ``ShardedSDDMM.run`` in place of the local tensor."""

    def __init__(self, bounds, feat_len, group=None, device=None, peer_copy=False):
        super().__init__(bounds, group, device)
        self.feat_len = int(feat_len)
        self._peer = None
        if peer_copy and self.world > 1 and dist.get_backend(group) == "nccl":
            self._peer = PeerCopyExchange.create(self, group, device)
        if self._peer is not None:
            self.full = self._peer.full
        else:
            self.full = torch.zeros((self.n, self.feat_len), dtype=torch.float32, device=device)
        self._own_full = True

    @property
    def exchange(self):
        """'peer-copy' (copy engines over NVLink into the peers' buffers) or 'all-gather' (the backend's collective)."""
        return "peer-copy" if self._peer is not None else "all-gather"

    def _slot(self, p):
        """Rows of the gather buffer that hold rank p's block."""
        if self.padded:
            return p * self.slot, p * self.slot + int(self.bounds[p + 1] - self.bounds[p])
        return int(self.bounds[p]), int(self.bounds[p + 1])

    def gather(self, x_local):
        if self.world == 1:
            self.full = x_local  # nothing to exchange: the local rows are all rows
            self._own_full = False
        elif self._peer is not None:
            self.gather_async(x_local).wait()
        else:
            self._gather(self.full, x_local)
        return self

    def gather_async(self, x_local):
        """Start the exchange and return at once; ``wait()`` before the first op that reads it.  The
        collective starts after the work already enqueued on the current stream and runs beside
        what is enqueued afterwards, so a caller whose next feature matrix is already available can
        exchange it while the current ops compute (NCCL backend; otherwise this is ``gather``)."""
        self._work = None
        if self.world == 1 or dist.get_backend(self.group) != "nccl":
            return self.gather(x_local)
        if self._peer is not None:
            self._peer_done = self._peer.start(x_local)
            return self
        self._work = self._gather_async(self.full, x_local)
        return self

    def gather_from_host_async(self, x_host_local):
        """``gather_async`` for rows that live in (pinned) host memory: the copy to the device runs on this
        layer's copy-in stream and the exchange starts behind it, neither touching the compute stream
        until ``wait()``.  A call may be issued while earlier kernels still read this buffer's previous
        contents only if those kernels were enqueued through ``ShardedSpMM.run_host`` /
        ``ShardedSDDMM.run_host`` (they leave the event this call waits for)."""
        s_in, _ = copy_streams(self.device)
        rows = self.row_hi - self.row_lo
        if tuple(x_host_local.shape) != (rows, self.feat_len):
            raise ValueError("local block has shape %s, this rank owns %d rows of %d columns"
                             % (tuple(x_host_local.shape), rows, self.feat_len))
        self._work = None
        read_done = getattr(self, "_read_done", None)
        if read_done is not None:
            s_in.wait_event(read_done)  # the kernels that gathered from the previous contents
        with torch.cuda.stream(s_in):
            if self.world == 1:
                if self.full is None or tuple(self.full.shape) != (rows, self.feat_len) or not self._own_full:
                    self.full = torch.empty((rows, self.feat_len), dtype=torch.float32, device=self.device)
                    self._own_full = True
                self.full.copy_(x_host_local, non_blocking=True)
                self._copied = s_in.record_event()
                return self
            if self.padded:
                mine = self.full[self.rank * self.slot:(self.rank + 1) * self.slot]
                mine[:rows].copy_(x_host_local, non_blocking=True)
                local = mine[:rows]
            else:
                local = self.full[self.row_lo:self.row_hi]
                local.copy_(x_host_local, non_blocking=True)
            if dist.get_backend(self.group) != "nccl":
                s_in.synchronize()
                self._gather_in_place(local)
                return self
            try:
                # the collective is ordered behind the copy: it is issued with the copy-in stream current
                if self.padded:
                    self._work = dist.all_gather_into_tensor(self.full, mine, group=self.group, async_op=True)
                else:
                    views = [self.full[int(self.bounds[p]):int(self.bounds[p + 1])] for p in range(self.world)]
                    self._work = dist.all_gather(views, local, group=self.group, async_op=True)
            except Exception as exc:
                raise ExchangeError("rank %d of %d: feature all-gather failed: %s" % (self.rank, self.world, exc)) from exc
        return self

    def _gather_in_place(self, local):
        """Backends without stream semantics (gloo): the blocking exchange, this rank's rows already in place."""
        try:
            if self.padded:
                mine = self.full[self.rank * self.slot:(self.rank + 1) * self.slot]
                dist.all_gather([self.full[p * self.slot:(p + 1) * self.slot] for p in range(self.world)],
                                mine.clone(), group=self.group)
            else:
                for p in range(self.world):
                    v = self.full[int(self.bounds[p]):int(self.bounds[p + 1])]
                    if v.numel():
                        dist.broadcast(v, src=dist.get_global_rank(self.group, p) if self.group is not None else p,
                                       group=self.group)
        except Exception as exc:
            raise ExchangeError("rank %d of %d: feature all-gather failed: %s" % (self.rank, self.world, exc)) from exc

    def wait(self):
        """Make the current stream wait for the exchange started by ``gather_async``."""
        copied = getattr(self, "_copied", None)
        if copied is not None:  # world size 1: only the host copy to wait for
            torch.cuda.current_stream(self.device).wait_event(copied)
            self._copied = None
        done = getattr(self, "_peer_done", None)
        if done is not None:
            torch.cuda.current_stream(self.device).wait_event(done)
            self._peer_done = None
        work = getattr(self, "_work", None)
        if work is not None:
            try:
                work.wait()
            except Exception as exc:
                raise ExchangeError("rank %d of %d: feature all-gather failed: %s" % (self.rank, self.world, exc)) from exc
            self._work = None
        return self


# ---- the all-gather as copies by the copy engines ----------------------------------------------------------
# A collective kernel that runs beside the compute kernels takes SMs from them for as long as it lasts.
# The exchange itself needs none: every rank's gather buffer is allocated as symmetric memory (mapped into
# every peer of the node), and a rank delivers its block with plain device-to-device copies (CHUNKS per peer) -
# work for the copy engines, over NVLink, into the peer's own memory.  Two one-element all-reduces on the
# exchange stream order it against the peers: the first says "every rank's kernels have finished reading the
# buffer's previous contents" (each rank enqueues it behind its own compute stream), the second "every rank's
# copies have landed".  Nothing here waits in a kernel of this library; a peer that is gone shows up as the
# process group's timeout on those all-reduces.
def _symmetric_memory():
    """torch's symmetric-memory module, set up for plain peer mappings: the exchanges here only read and write
    peers' buffers through ordinary pointers, so the buffers need not be bound to an NVLink multicast object as
    well (one binding less to undo when a rank goes away)."""
    import os
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm
    return symm


class PeerCopyExchange:
    """The gather buffer of one ``GatheredFeatures`` as symmetric memory, and the streams its copies run on."""

    CHUNKS = 2  # pieces per peer, each on a stream of its own

    @classmethod
    def create(cls, owner, group, device):
        """None where symmetric memory cannot be set up on every rank (the caller then uses the collective).
        The ranks agree on the outcome after each step, so that no rank waits in an exchange its peers do
        not take part in."""
        group = group if group is not None else dist.group.WORLD
        self = cls.__new__(cls)
        self.owner, self.device, self._group = owner, device, group
        self.error = None

        def everyone(ok):
            flag = torch.tensor([1.0 if ok else 0.0], dtype=torch.float32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            return bool(flag.item() > 0.5)

        shape = (owner.n, owner.feat_len)
        try:
            symm = _symmetric_memory()
            with torch.cuda.device(device):
                self.full = symm.empty(shape, dtype=torch.float32, device=device)
                self.full.zero_()
        except Exception as exc:  # no symmetric-memory support in this torch build, or no memory
            self.error = exc
        if not everyone(self.error is None):
            return None
        try:
            with torch.cuda.device(device):
                handle = symm.rendezvous(self.full, group)
                self.peer_full = {p: handle.get_buffer(p, shape, torch.float32)
                                  for p in range(owner.world) if p != owner.rank}
                self._handle = handle
                self._token = torch.zeros(1, dtype=torch.float32, device=device)
                self._stream = torch.cuda.Stream(device)
                self._peer_streams = {p: [torch.cuda.Stream(device) for _ in range(self.CHUNKS)] for p in self.peer_full}
        except Exception as exc:  # the node cannot map peers' memory
            self.error = exc
        return self if everyone(self.error is None) else None

    def _barrier(self):
        """All ranks' exchange streams meet here (enqueued on the current stream)."""
        try:
            dist.all_reduce(self._token, group=self._group, async_op=True).wait()
        except Exception as exc:
            raise ExchangeError("rank %d of %d: feature exchange failed: %s" % (self.owner.rank, self.owner.world, exc)) from exc

    def start(self, x_local):
        """Enqueue the exchange behind the work the current stream holds; returns the event that marks the
        gather buffer complete."""
        o = self.owner
        lo, hi = o._slot(o.rank)
        if tuple(x_local.shape) != (hi - lo, o.feat_len):
            raise ValueError("local block has shape %s, this rank owns %d rows of %d columns"
                             % (tuple(x_local.shape), hi - lo, o.feat_len))
        ex = self._stream
        ex.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(ex):
            self._barrier()  # every rank is past the last reader of its buffer
            mine = self.full[lo:hi]
            if mine.data_ptr() != x_local.data_ptr():
                mine.copy_(x_local, non_blocking=True)
            src = x_local.contiguous()
            ready = ex.record_event()
            # a copy engine moves one copy at a time: several pieces per peer keep more of them busy
            cuts = [lo + (hi - lo) * c // self.CHUNKS for c in range(self.CHUNKS + 1)]
            for c in range(self.CHUNKS):
                a, b = cuts[c], cuts[c + 1]
                if a == b:
                    continue
                for p, streams in self._peer_streams.items():
                    st = streams[c]
                    st.wait_event(ready)
                    with torch.cuda.stream(st):
                        self.peer_full[p][a:b].copy_(src[a - lo:b - lo], non_blocking=True)
                    src.record_stream(st)
                    ex.wait_stream(st)
            self._barrier()  # every rank's copies have landed
            return ex.record_event()


# ---- exchanging only the rows a shard references ---------------------------------------------------------
# An all-gather hands every rank every feature row.  A row shard's column ids reference only some of them:
# nearly all on a graph whose rows each have hundreds of neighbours, a fraction on a skewed graph of millions
# of vertices (R-MAT scale 22 on 8 ranks: about a third).  ``NeededRows`` works out, once per adjacency, which
# rows each rank needs from each peer; per call every rank packs the rows its peers asked for (a small row-gather
# kernel) and one all-to-all delivers them into a compact buffer.  The shard's column ids are remapped into that
# buffer by an increasing map (position in the sorted list of needed ids), so every row's nonzeros keep their
# order and every sum its bits.
NEEDED_ROWS_MAX_FRACTION = 0.7  # the compact exchange is chosen while ranks need at most this share of the rows


def _pack_rows(src, rows, out):
    """out[i] = src[rows[i]] (rows: int64 tensor on src's device)."""
    if rows.numel() == 0:
        return out
    if src.is_cuda:
        import ctypes
        from . import _native
        with torch.cuda.device(src.device):
            _native.check(_native.lib().fg_gather_rows_f32(
                ctypes.c_void_p(src.data_ptr()), src.stride(0), ctypes.c_void_p(rows.data_ptr()), rows.numel(),
                src.shape[1], ctypes.c_void_p(out.data_ptr()), out.stride(0),
                ctypes.c_void_p(torch.cuda.current_stream(src.device).cuda_stream)))
    else:  # CPU ranks (gloo): the host-side bookkeeping tests
        torch.index_select(src, 0, rows, out=out)
    return out


class NeededRows(_ShardedBase):
    """Which feature rows this rank's shard references, and which of its own rows each peer asked for.

    ``adj``: the shard with column ids remapped into the compact buffer (``n_compact`` columns);
    ``recv_counts[q]`` rows arrive from rank q, ``send_counts[p]`` rows go to rank p, ``send_rows`` lists the
    local row ids to send, grouped by receiving rank."""

    def __init__(self, local_adj, bounds, group=None, device=None):
        super().__init__(bounds, group, device)
        assert local_adj.shape[0] == self.row_hi - self.row_lo
        needed = np.unique(local_adj.indices)
        self.needed = needed
        self.n_compact = int(needed.shape[0])
        cut = np.searchsorted(needed, self.bounds)  # needed[cut[q]:cut[q+1]] live on rank q
        self.recv_counts = np.diff(cut).astype(np.int64)
        new_idx = np.searchsorted(needed, local_adj.indices).astype(local_adj.indices.dtype)
        self.adj = scipy.sparse.csr_matrix((local_adj.data, new_idx, local_adj.indptr),
                                           shape=(local_adj.shape[0], max(self.n_compact, 1)))
        self.adj.has_sorted_indices = True
        meta_dev = device if (device is not None and self.world > 1 and dist.get_backend(group) == "nccl") else None
        if self.world == 1:
            self.send_counts = self.recv_counts.copy()
            self.send_rows = torch.from_numpy((needed - self.row_lo).astype(np.int64)).to(device)
            return
        # every rank learns how many rows each peer wants from it, then receives the lists themselves
        mine = torch.from_numpy(self.recv_counts).to(meta_dev)
        counts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(counts, mine, group=group)
        table = torch.stack(counts).cpu().numpy()  # table[p][q]: rows rank p needs from rank q
        self.send_counts = table[:, self.rank].astype(np.int64)
        owner_start = np.repeat(self.bounds[:-1], self.recv_counts)
        requests = torch.from_numpy((needed.astype(np.int64) - owner_start)).to(meta_dev)  # local ids at their owners
        self.request_rows = requests.to(device) if device is not None else requests  # grouped by owner, see recv_counts
        asked = torch.empty((int(self.send_counts.sum()),), dtype=torch.int64, device=meta_dev)
        dist.all_to_all_single(asked, requests, output_split_sizes=[int(v) for v in self.send_counts],
                               input_split_sizes=[int(v) for v in self.recv_counts], group=group)
        self.send_rows = asked.to(device)

    def fraction(self):
        """Share of all feature rows this rank needs."""
        return self.n_compact / float(max(int(self.bounds[-1]), 1))

    def exchange(self, compact, x_local, send_buf=None, async_op=False):
        """``compact[i] = features of needed[i]`` from whichever rank owns that row.  ``send_buf``: a reusable
        [sum(send_counts), d] buffer.  Returns the work handle with ``async_op`` (NCCL), else ``compact``."""
        d = x_local.shape[1]
        if send_buf is None:
            send_buf = torch.empty((int(self.send_counts.sum()), d), dtype=x_local.dtype, device=x_local.device)
        _pack_rows(x_local, self.send_rows, send_buf)
        if self.world == 1:
            compact[:self.n_compact].copy_(send_buf)
            return compact
        try:
            work = dist.all_to_all_single(compact[:self.n_compact], send_buf,
                                          output_split_sizes=[int(v) for v in self.recv_counts],
                                          input_split_sizes=[int(v) for v in self.send_counts], group=self.group,
                                          async_op=async_op)
        except Exception as exc:
            raise ExchangeError("rank %d of %d: needed-rows exchange failed: %s" % (self.rank, self.world, exc)) from exc
        return work if async_op else compact


def needed_rows_pay(needed_rows, group=None):
    """True if, averaged over the ranks, a shard references at most ``NEEDED_ROWS_MAX_FRACTION`` of the feature
    rows (every rank gets the same answer: the choice of exchange must be collective)."""
    frac = torch.tensor([needed_rows.fraction()], dtype=torch.float64)
    if needed_rows.world > 1:
        if dist.get_backend(group) == "nccl":
            frac = frac.to(needed_rows.device)
        dist.all_reduce(frac, group=group)
        frac = frac / needed_rows.world
    return float(frac.item()) <= NEEDED_ROWS_MAX_FRACTION


class PeerPullExchange:
    """The needed-rows exchange without a sender: every rank keeps its own feature rows in symmetric memory
    (mapped into every peer of the node) and a rank fetches the rows it needs itself, one launch of the row-gather
    kernel per owner reading that owner's memory over NVLink (plain loads; the kernel is this library's) and
    writing the compact buffer.  No packing pass, no send buffer, no all-to-all.  Two one-element all-reduces on
    the exchange stream order it: "every rank's rows are in place" before the reads, and, behind the reads and off
    the caller's critical path, "every rank has finished reading" (after which the rows may be rewritten).
    Nothing waits in a kernel."""

    @classmethod
    def create(cls, owner, group, device):
        """None where symmetric memory cannot be set up on every rank (the caller then uses the all-to-all)."""
        group = group if group is not None else dist.group.WORLD
        rows = owner.rows
        self = cls.__new__(cls)
        self.owner, self.device, self._group = owner, device, group
        self.error = None
        self.released = None

        def everyone(ok):
            flag = torch.tensor([1.0 if ok else 0.0], dtype=torch.float32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            return bool(flag.item() > 0.5)

        slot = int(np.diff(rows.bounds).max())  # the same size on every rank, as symmetric memory wants
        shape = (max(slot, 1), owner.feat_len)
        try:
            symm = _symmetric_memory()
            with torch.cuda.device(device):
                self.local = symm.empty(shape, dtype=torch.float32, device=device)
                self.local.zero_()
        except Exception as exc:
            self.error = exc
        if not everyone(self.error is None):
            return None
        try:
            with torch.cuda.device(device):
                handle = symm.rendezvous(self.local, group)
                self._handle = handle
                self._peer_ptrs = [int(v) for v in handle.buffer_ptrs]
                self._token = torch.zeros(1, dtype=torch.float32, device=device)
                # high priority: an exchange that runs beside a compute kernel must not queue behind its blocks
                self._stream = torch.cuda.Stream(device, priority=-1)
            if len(self._peer_ptrs) != rows.world:
                raise RuntimeError("unexpected symmetric-memory pointer table")
            self._peer_ptrs[rows.rank] = self.local.data_ptr()
        except Exception as exc:
            self.error = exc
        if not everyone(self.error is None):
            return None
        # needed[cut[q]:cut[q+1]] live on rank q; request_rows holds their row ids within q's block
        self._cut = np.concatenate([[0], np.cumsum(rows.recv_counts)]).astype(np.int64)
        assert int(self._cut[-1]) == rows.n_compact
        for q in range(rows.world):  # a read past a peer's block would fault: check the lists once, on the host
            seg = rows.request_rows[int(self._cut[q]):int(self._cut[q + 1])]
            if seg.numel() and (int(seg.min()) < 0 or int(seg.max()) >= int(rows.bounds[q + 1] - rows.bounds[q])):
                raise ValueError("needed-row list for rank %d is out of its range" % q)
        return self

    def _barrier(self):
        try:
            dist.all_reduce(self._token, group=self._group, async_op=True).wait()
        except Exception as exc:
            raise ExchangeError("rank %d of %d: needed-rows exchange failed: %s"
                                % (self.owner.rank, self.owner.world, exc)) from exc

    def start(self, x_local):
        """Enqueue the exchange behind the work the current stream holds; returns the event that marks the
        compact buffer complete."""
        import ctypes
        from . import _native
        o, rows = self.owner, self.owner.rows
        n_local = rows.row_hi - rows.row_lo
        if tuple(x_local.shape) != (n_local, o.feat_len):
            raise ValueError("local block has shape %s, this rank owns %d rows of %d columns"
                             % (tuple(x_local.shape), n_local, o.feat_len))
        ex = self._stream
        ex.wait_stream(torch.cuda.current_stream(self.device))
        L = _native.lib()
        with torch.cuda.device(self.device), torch.cuda.stream(ex):
            # (the previous exchange ended with a barrier behind every rank's reads, on this same stream, so
            # this rank's rows may be overwritten here)
            if x_local.data_ptr() != self.local.data_ptr():
                self.local[:n_local].copy_(x_local, non_blocking=True)
                x_local.record_stream(ex)
            self._barrier()  # every rank's rows are in place
            # one launch per owner, own block first, then the peers in ring order from this rank, so that the ranks
            # do not all read from the same owner at once (launches on streams of their own were slower:
            # 6.43 against 6.06 ms per R-MAT step on 4 GPUs)
            s = ctypes.c_void_p(ex.cuda_stream)
            for i in range(rows.world):
                q = (rows.rank + i) % rows.world
                a, b = int(self._cut[q]), int(self._cut[q + 1])
                if a == b:
                    continue
                req = rows.request_rows[a:b]
                dst = o.full[a:b]
                _native.check(L.fg_gather_rows_f32(ctypes.c_void_p(self._peer_ptrs[q]), o.feat_len,
                                                   ctypes.c_void_p(req.data_ptr()), b - a, o.feat_len,
                                                   ctypes.c_void_p(dst.data_ptr()), o.full.stride(0), s))
            done = ex.record_event()
            self._barrier()  # every rank has finished reading: the rows may be rewritten
            self.released = ex.record_event()
            return done

    def local_rows(self):
        """This rank's block of the symmetric buffer ([rows of this rank, d]).  A caller that produces its features
        straight into it and passes it to ``gather_async`` saves the copy; before rewriting it after an exchange,
        make the writing stream wait for ``released`` (``NeededFeatures.wait_writable``)."""
        rows = self.owner.rows
        return self.local[:rows.row_hi - rows.row_lo]


class NeededFeatures:
    """The compact counterpart of ``GatheredFeatures``: the feature rows this rank's shard references, fetched
    by ``NeededRows.exchange``.  Same calls (``gather``, ``gather_async`` / ``wait``, ``.full``), so the sharded
    ops built with ``needed_rows=`` take it in place of the local tensor."""

    def __init__(self, needed_rows, feat_len, device=None, peer_pull=False):
        self.rows = needed_rows
        self.feat_len = int(feat_len)
        self.device = device if device is not None else needed_rows.device
        self.world, self.rank = needed_rows.world, needed_rows.rank
        self.full = torch.zeros((max(needed_rows.n_compact, 1), self.feat_len), dtype=torch.float32, device=self.device)
        self._pull = None
        if peer_pull and self.world > 1 and dist.get_backend(needed_rows.group) == "nccl":
            self._pull = PeerPullExchange.create(self, needed_rows.group, self.device)
        self._send = None if self._pull is not None else \
            torch.empty((int(needed_rows.send_counts.sum()), self.feat_len), dtype=torch.float32, device=self.device)
        self._work = None
        self._pull_done = None

    @property
    def exchange(self):
        """'peer-pull' (this rank's kernel reads the rows it needs from its peers' memory over NVLink) or
        'all-to-all' (peers pack and send them)."""
        return "peer-pull" if self._pull is not None else "all-to-all"

    def gather(self, x_local):
        if self._pull is not None:
            return self.gather_async(x_local).wait()
        self.rows.exchange(self.full, x_local, self._send)
        return self

    def gather_async(self, x_local):
        """Start the exchange behind the work already on the current stream; ``wait()`` before the first use."""
        self._work = None
        if self._pull is not None:
            self._pull_done = self._pull.start(x_local)
            return self
        if self.world == 1 or dist.get_backend(self.rows.group) != "nccl":
            return self.gather(x_local)
        self._work = self.rows.exchange(self.full, x_local, self._send, async_op=True)
        return self

    @property
    def local_input(self):
        """Peer-pull only: this rank's rows of the symmetric buffer, for callers that write their features there
        (``gather_async(self.local_input)`` then copies nothing); None otherwise."""
        return self._pull.local_rows() if self._pull is not None else None

    def wait_writable(self):
        """Peer-pull only: make the current stream wait until every rank has finished reading ``local_input``'s
        previous contents."""
        ev = getattr(self._pull, "released", None) if self._pull is not None else None
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    def wait(self):
        if self._pull_done is not None:
            torch.cuda.current_stream(self.device).wait_event(self._pull_done)
            self._pull_done = None
        if self._work is not None:
            try:
                self._work.wait()
            except Exception as exc:
                raise ExchangeError("rank %d of %d: needed-rows exchange failed: %s" % (self.rank, self.world, exc)) from exc
            self._work = None
        return self


class ShardedSpMM(_ShardedBase):
    """Row-sharded SpMM for a square adjacency.

    ``local_adj``: this rank's rows (``shard_csr_rows``), ``bounds``: the row ranges of all ranks
    (``nnz_balanced_row_ranges`` of the whole graph's indptr)."""

    def __init__(self, local_adj, bounds, group=None, device=None, needed_rows=None):
        from .module import VanillaSpMMcuda
        super().__init__(bounds, group, device)
        assert local_adj.shape[0] == self.row_hi - self.row_lo
        assert local_adj.shape[1] == int(self.bounds[-1]), "square adjacency expected (features are row-sharded)"
        self.needed_rows = needed_rows
        if needed_rows is not None:
            # the kernel gathers from the compact buffer of needed rows (column ids remapped once)
            self.n = max(needed_rows.n_compact, 1)
            self.module = VanillaSpMMcuda(needed_rows.adj, device=device)
            self.device = self.module.ctx
            self.x_full = None
            return
        # the kernel gathers from the all-gather buffer: in the padded layout the column ids are remapped once
        self.module = VanillaSpMMcuda(remap_columns(local_adj, self.bounds), device=device)
        self.device = self.module.ctx
        self.x_full = None

    def build(self, feat_len, feat_tile=0):
        from .placeholder import placeholder
        self.module.build([placeholder((self.n, feat_len))], {}, {"feat_tile": feat_tile})
        self.x_full = torch.zeros((self.n, feat_len), dtype=torch.float32, device=self.device)

    def gather(self, x_local):
        """The exchange step alone: every rank's feature rows into this rank's ``x_full``."""
        if self.needed_rows is not None:
            return self.needed_rows.exchange(self.x_full, x_local)
        if self.world == 1:
            self.x_full = x_local
            return x_local
        return self._gather(self.x_full, x_local)

    def compute(self):
        """The local kernel alone, on the features gathered last."""
        return self.module.run([self.x_full])

    def run(self, x_local):
        """x_local: this rank's rows of the feature matrix, or a ``GatheredFeatures`` that already
        holds every rank's rows.  Returns this rank's rows of A.X."""
        if isinstance(x_local, (GatheredFeatures, NeededFeatures)):
            return self.module.run([x_local.full])
        self.gather(x_local)
        return self.compute()


    def run_host(self, gathered, out_host):
        """Host-result call: the kernel on ``gathered`` (a ``GatheredFeatures`` whose exchange was started by
        ``gather_from_host_async`` or ``gather_async``), then this rank's rows of A.X copied to the pinned
        host tensor ``out_host`` on the copy-out stream.  Only enqueues; ``sharded.host_sync(device)`` waits."""
        gathered.wait()
        wait_for_copy_out(self.module.out, self.device, self)  # the previous result has left the device
        out = self.module.run([gathered.full])
        gathered._read_done = torch.cuda.current_stream(self.device).record_event()
        return copy_out_async(out, out_host, self.device, self)


class ShardedSDDMM(_ShardedBase):
    """Edge-sharded SDDMM by the same row ranges (square adjacency)."""

    def __init__(self, local_adj, bounds, group=None, device=None, needed_rows=None):
        from .module import VanillaSDDMMcuda
        super().__init__(bounds, group, device)
        assert local_adj.shape[0] == self.row_hi - self.row_lo
        self.needed_rows = needed_rows
        if needed_rows is not None:
            self.n = max(needed_rows.n_compact, 1)
            self.module = VanillaSDDMMcuda(needed_rows.adj.tocoo(), device=device)
            self.device = self.module.ctx
            self.src_full = None
            return
        self.module = VanillaSDDMMcuda(remap_columns(local_adj, self.bounds).tocoo(), device=device)
        self.device = self.module.ctx
        self.src_full = None

    def build(self, feat_len):
        from .placeholder import placeholder
        self.module.build([placeholder((self.n, feat_len)), placeholder((self.row_hi - self.row_lo, feat_len))], {}, {})
        self.src_full = torch.zeros((self.n, feat_len), dtype=torch.float32, device=self.device)

    def gather(self, src_local):
        if self.needed_rows is not None:
            return self.needed_rows.exchange(self.src_full, src_local)
        if self.world == 1:
            self.src_full = src_local
            return src_local
        return self._gather(self.src_full, src_local)

    def compute(self, dst_local):
        return self.module.run([self.src_full, dst_local])

    def run(self, src_local, dst_local):
        """src_local: this rank's rows of the column-side matrix (gathered from all ranks), or a
        ``GatheredFeatures`` that already holds them; dst_local: this rank's rows of the row-side
        matrix.  Returns this rank's edges' dots."""
        if isinstance(src_local, (GatheredFeatures, NeededFeatures)):
            return self.module.run([src_local.full, dst_local])
        self.gather(src_local)
        return self.compute(dst_local)

    def run_host(self, gathered, dst_host_local, out_host):
        """Host-buffer call: ``gathered`` as in ``ShardedSpMM.run_host``; this rank's rows of the row-side
        matrix come from the (pinned) host tensor ``dst_host_local`` over the copy-in stream, the per-edge
        result goes to ``out_host`` over the copy-out stream.  Only enqueues; ``sharded.host_sync`` waits."""
        s_in, _ = copy_streams(self.device)
        stream = torch.cuda.current_stream(self.device)
        rows = self.row_hi - self.row_lo
        d = gathered.feat_len
        stages = self.__dict__.setdefault("_dst_stages", {})  # one staging buffer per feature length
        if d not in stages:
            stages[d] = [torch.empty((rows, d), dtype=torch.float32, device=self.device), None]
        stage, last_read = stages[d]
        if last_read is not None:
            s_in.wait_event(last_read)  # the kernel that read the staging buffer last
        with torch.cuda.stream(s_in):
            stage.copy_(dst_host_local, non_blocking=True)
            copied = s_in.record_event()
        gathered.wait()
        stream.wait_event(copied)
        wait_for_copy_out(self.module.out, self.device, self)
        out = self.module.run([gathered.full, stage])
        stages[d][1] = stream.record_event()
        gathered._read_done = stages[d][1]
        return copy_out_async(out, out_host, self.device, self)
