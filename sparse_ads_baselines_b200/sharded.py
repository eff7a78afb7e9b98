"""Table-wise model-parallel TBE: each rank owns ``T/W`` whole tables, looks up the GLOBAL batch
for them and the pooled ``[B, T/W, D]`` rows are exchanged so that every rank ends with its batch
slice of all tables, ``[B/W, T, D]`` -- the wiring of the reference's
``DistributedPartitionShardedSNN`` (models.py:212-227) and ``All2AllFunction``
(sparse_embedding_cuda_ops.py:88-120), with the layout contract of ``forward_all2all_nccl``
(sparse_embedding_cuda.cpp:471-533):  ``out_j[b', r*T/W + t] = in_r[j*B/W + b', t]``.

Two exchanges:
  * ``exchange="fused"`` -- no collective call at all.  The forward kernel stores each pooled row
    straight into the owner rank's ``[B/W, T, D]`` buffer through peer-mapped (symmetric) memory,
    and the backward scatters the local gradient slice to the table owners with one peer-store
    kernel.  Producers and consumers are ordered by step-numbered flags in peer-mapped memory
    (``tbe_peer_signal_wait``: a release store per peer, a bounded acquire poll per peer), and the
    buffers are double-buffered: before a rank overwrites a peer's buffer it has seen that peer's
    "free" flag, which the peer raises when its stream has passed every consumer of the buffer's
    previous contents.  Neither direction needs a transpose copy.

    Contract of the fused mode: ``forward`` returns a view of an exchange buffer.  It stays valid
    until this rank launches its SECOND-next forward; work that reads it must be enqueued on the
    stream ``forward`` ran on (or be ordered after it by events) before that launch.  Keep a
    ``.clone()`` for anything longer-lived.  A wait that runs out (a peer died or never joined) is
    reported by :meth:`TableShardedEmbeddingBags.check_exchange`, never by a hung GPU.
  * ``exchange="nccl"`` -- ``all_to_all_single`` plus the reference's transpose copies; this is the
    baseline the fused path is measured against, and the only mode that runs on CPU tensors (gloo),
    where it serves the host-logic tests.
"""
import ctypes

import torch
import torch.distributed as dist
from torch import nn

from . import _lib
from . import table_batched_embeddings as tbe_ext
from .table_batched_embeddings_ops import Optimizer, TableBatchedEmbeddingBags


def pooled_all_to_all(local, group=None):
    """``[B, T/W, D]`` (own tables, global batch) -> ``[B/W, T, D]`` (own batch slice, all tables)
    with a library all-to-all and the reference's transpose (sparse_embedding_cuda.cpp:524-532)."""
    W = dist.get_world_size(group)
    if W == 1:
        return local
    B, Tl, D = local.shape
    assert B % W == 0, "world size must divide the batch"
    recv = torch.empty_like(local)
    dist.all_to_all_single(recv, local.contiguous(), group=group)
    return recv.view(W, B // W, Tl, D).transpose(0, 1).reshape(B // W, W * Tl, D)


def pooled_all_to_all_backward(grad, group=None):
    """Inverse of :func:`pooled_all_to_all`: ``[B/W, T, D]`` -> ``[B, T/W, D]``
    (sparse_embedding_cuda_ops.py:104-117)."""
    W = dist.get_world_size(group)
    if W == 1:
        return grad
    Bl, T, D = grad.shape
    assert T % W == 0, "world size must divide the number of tables"
    send = grad.view(Bl, W, T // W, D).transpose(0, 1).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.view(W * Bl, T // W, D)


class _NcclExchange(torch.autograd.Function):
    @staticmethod
    def forward(ctx, local, group):
        ctx.group = group
        return pooled_all_to_all(local, group)

    @staticmethod
    def backward(ctx, grad):
        return pooled_all_to_all_backward(grad.contiguous(), ctx.group), None


# rows of the flag matrix every rank owns (one 128-byte line each; slot j of a row is written by rank j)
_OUT_FREE, _OUT_READY, _GRAD_FREE, _GRAD_READY = range(4)
_FLAG_ROW_INTS = 32


class _SymmetricBuffers:
    """Peer-mapped state of one sharded module: two exchanged-output buffers, two incoming-gradient
    buffers (alternating by step) and the flag matrix that orders their use across ranks."""

    def __init__(self, B, T_local, D, dtype, device, group, timeout_s):
        import torch.distributed._symmetric_memory as symm_mem
        W = dist.get_world_size(group)
        assert W <= _lib.TBE_MAX_PEERS
        self.world, self.rank, self.group = W, dist.get_rank(group), group
        ptr_array = ctypes.c_void_p * W

        def shared(shape, dt):
            t = symm_mem.empty(shape, dtype=dt, device=device)
            handle = symm_mem.rendezvous(t, group=group)
            return t, handle, [int(p) for p in handle.buffer_ptrs]

        self.out, self.out_ptrs, self.grad_in, self.grad_ptrs, self._handles = [], [], [], [], []
        for _ in range(2):
            t, h, ptrs = shared((B // W, T_local * W, D), dtype)
            self.out.append(t)
            self.out_ptrs.append(ptr_array(*ptrs))
            self._handles.append(h)
            t, h, ptrs = shared((B, T_local, D), dtype)
            self.grad_in.append(t)
            self.grad_ptrs.append(ptr_array(*ptrs))
            self._handles.append(h)
        self.flags, h, ptrs = shared((4, _FLAG_ROW_INTS), torch.int32)
        self._handles.append(h)
        self.flag_ptrs = [ptr_array(*[p + 4 * _FLAG_ROW_INTS * row for p in ptrs]) for row in range(4)]
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.timeout_ns = int(timeout_s * 1e9)
        self.fwd_step = 0
        self.bwd_step = 0
        self.plan_workspace = None
        # nobody may signal before every rank has zeroed its flags
        self.flags.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def sync(self, row, signal_value, wait_value, stream):
        """Raise this rank's slot of flag ``row`` on every peer to ``signal_value``, then wait (on the
        device, bounded) until every peer's slot here has reached ``wait_value``."""
        _lib.call("tbe_peer_signal_wait", self.flag_ptrs[row], self.flags[row].data_ptr(), self.world, self.rank,
                  signal_value, wait_value, self.timeout_ns, self.status.data_ptr(), stream)

    def check(self, stream):
        host = (ctypes.c_int32 * 4)()
        _lib.call("tbe_peer_status", self.status.data_ptr(), host, stream)


class _FusedShardedLookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weights, module, indices, offsets):
        m = module
        buf = m._buffers_for(indices.device)
        T, B, D = m.local_tables, m.global_batch, m.embedding_dim
        buf.fwd_step += 1
        k, slot = buf.fwd_step, buf.fwd_step & 1
        with torch.cuda.device(weights.device):
            stream = tbe_ext._stream(weights.device)
            # my other output buffer is free from here on (its consumers precede this launch in stream
            # order); the peers' buffers `slot` were declared free one step ago
            buf.sync(_OUT_FREE, k, k - 1, stream)
            _lib.call("tbe_forward_sharded", weights.data_ptr(), m.tbe.table_offsets.data_ptr(), indices.data_ptr(),
                      offsets.data_ptr(), None, buf.out_ptrs[slot], buf.world, T, B, D, T * buf.world, T * buf.rank,
                      tbe_ext._DTYPES[weights.dtype], tbe_ext._POOLING[m.tbe.pooling_mode], stream)
            buf.sync(_OUT_READY, k, k, stream)
        ctx.module = m
        ctx.save_for_backward(weights, indices, offsets)
        return buf.out[slot].view(buf.out[slot].shape)

    @staticmethod
    def backward(ctx, grad):
        m = ctx.module
        weights, indices, offsets = ctx.saved_tensors
        buf = m._buffers_for(indices.device)
        T, B, D = m.local_tables, m.global_batch, m.embedding_dim
        grad = grad.contiguous()
        buf.bwd_step += 1
        k, slot = buf.bwd_step, buf.bwd_step & 1
        # the sort of the lookups needs no gradient: it runs on a side stream under the exchange
        plan = None
        if m.tbe.optimizer in (Optimizer.SGD, Optimizer.EXACT_ROWWISE_ADAGRAD):
            need = tbe_ext._workspace_bytes(indices.numel(), weights.size(0))
            if buf.plan_workspace is None or buf.plan_workspace.numel() < need:
                buf.plan_workspace = torch.empty(int(need * 1.1) + 4096, dtype=torch.uint8, device=weights.device)
            plan = tbe_ext.backward_plan(m.tbe.table_offsets, indices, offsets, weights.size(0),
                                         workspace=buf.plan_workspace)
        with torch.cuda.device(weights.device):
            stream = tbe_ext._stream(weights.device)
            buf.sync(_GRAD_FREE, k, k - 1, stream)
            _lib.call("tbe_all2all_push", grad.data_ptr(), buf.grad_ptrs[slot], buf.world, buf.rank, B // buf.world,
                      T * D * grad.element_size(), stream)
            buf.sync(_GRAD_READY, k, k, stream)
        m.apply_local_backward(buf.grad_in[slot], indices, offsets, plan=plan)
        return None, None, None, None


class TableShardedEmbeddingBags(nn.Module):
    """``tables_per_rank`` tables on every rank of ``group``; ``forward`` takes this rank's tables'
    indices/offsets over the global batch and returns this rank's ``[B/W, T_total, D]`` slice."""

    def __init__(self, tables_per_rank, num_embeddings, embedding_dim, global_batch, optimizer=Optimizer.SGD,
                 learning_rate=0.01, eps=None, fp16=False, pooling_mode="sum", exchange="fused", group=None,
                 sync_timeout_s=30.0):
        super().__init__()
        assert exchange in ("fused", "nccl")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert global_batch % self.world == 0, "world size must divide the global batch"
        self.local_tables = tables_per_rank
        self.embedding_dim = embedding_dim
        self.global_batch = global_batch
        self.exchange = exchange
        self.sync_timeout_s = sync_timeout_s
        self.tbe = TableBatchedEmbeddingBags(tables_per_rank, num_embeddings, embedding_dim, optimizer=optimizer,
                                             learning_rate=learning_rate, eps=eps, fp16=fp16,
                                             pooling_mode=pooling_mode)
        self._symm = None

    def _buffers_for(self, device):
        if self._symm is None:
            w = self.tbe.embedding_weights
            self._symm = _SymmetricBuffers(self.global_batch, self.local_tables, self.embedding_dim, w.dtype, device,
                                           self.group if self.group is not None else dist.group.WORLD,
                                           self.sync_timeout_s)
        return self._symm

    def check_exchange(self):
        """Synchronises the current stream and raises ``TBEError`` (status ``TBE_ERR_TIMEOUT``) if a
        bounded device-side wait of the fused exchange ran out since the module was built -- the
        results of the steps after it are then not to be trusted."""
        if self._symm is not None:
            dev = self.tbe.embedding_weights.device
            with torch.cuda.device(dev):
                self._symm.check(tbe_ext._stream(dev))

    def apply_local_backward(self, grad_local, indices, offsets, plan=None):
        """Fused backward + optimizer of the local tables for ``grad_local = [B, T/W, D]``; ``plan`` is
        an optional :func:`table_batched_embeddings.backward_plan` of the same lookups."""
        t = self.tbe
        if t.optimizer == Optimizer.SGD:
            tbe_ext.backward_sgd(grad_local, t.embedding_weights.data, t.table_offsets, indices, offsets,
                                 t.learning_rate, 200, 1, False, pooling_mode=t.pooling_mode, plan=plan)
        elif t.optimizer == Optimizer.EXACT_ROWWISE_ADAGRAD:
            tbe_ext.backward_exact_adagrad(grad_local, t.embedding_weights.data, t.table_offsets, indices, offsets,
                                           None, t.optimizer_state, t.learning_rate, t.eps, t.stochastic_rounding, 1,
                                           pooling_mode=t.pooling_mode, plan=plan)
        else:
            tbe_ext.backward_approx_adagrad(grad_local, t.embedding_weights.data, t.table_offsets, indices, offsets,
                                            None, t.optimizer_state, t.learning_rate, t.eps, 200,
                                            t.stochastic_rounding, 1)

    def forward(self, indices, offsets):
        if self.world == 1:
            return self.tbe(indices, offsets)
        if self.exchange == "nccl":
            return _NcclExchange.apply(self.tbe(indices, offsets), self.group)
        return _FusedShardedLookup.apply(self.tbe.embedding_weights, self, indices, offsets)


# ---------------------------------------------------------------------------- row-wise sharding
class _FusedRowShardedLookup(torch.autograd.Function):
    """Lookup over this rank's row slice + reduce-scatter, and all-gather + fused backward, with both
    exchanges done by peer stores (no collective call)."""

    @staticmethod
    def forward(ctx, weights, module, indices, offsets):
        m = module
        buf = m._buffers_for(indices.device)
        T, B, D = m.num_tables, m.global_batch, m.embedding_dim
        W, Bl = buf.world, B // buf.world
        es = weights.element_size()
        buf.fwd_step += 1
        k, slot = buf.fwd_step, buf.fwd_step & 1
        out = torch.empty((Bl, T, D), dtype=weights.dtype, device=weights.device)
        with torch.cuda.device(weights.device):
            stream = tbe_ext._stream(weights.device)
            buf.sync(_OUT_FREE, k, k - 1, stream)
            # rank j's staging buffer is [W][B/W][T][D]; this rank fills slot `rank` of every peer's
            slot_bytes = Bl * T * D * es
            dst = (ctypes.c_void_p * W)(*[int(p) + buf.rank * slot_bytes for p in buf.out_ptrs[slot]])
            _lib.call("tbe_forward_sharded", weights.data_ptr(), m.tbe.table_offsets.data_ptr(), indices.data_ptr(),
                      offsets.data_ptr(), None, dst, W, T, B, D, T, 0, tbe_ext._DTYPES[weights.dtype],
                      tbe_ext._POOLING["sum"], stream)
            buf.sync(_OUT_READY, k, k, stream)
            _lib.call("tbe_reduce_slots", buf.out[slot].data_ptr(), out.data_ptr(), W, Bl * T * D,
                      tbe_ext._DTYPES[weights.dtype], stream)
        ctx.module = m
        ctx.save_for_backward(weights, indices, offsets)
        return out

    @staticmethod
    def backward(ctx, grad):
        m = ctx.module
        weights, indices, offsets = ctx.saved_tensors
        buf = m._buffers_for(indices.device)
        grad = grad.contiguous()
        buf.bwd_step += 1
        k, slot = buf.bwd_step, buf.bwd_step & 1
        plan = None
        if m.tbe.optimizer in (Optimizer.SGD, Optimizer.EXACT_ROWWISE_ADAGRAD):
            need = tbe_ext._workspace_bytes(indices.numel(), weights.size(0))
            if buf.plan_workspace is None or buf.plan_workspace.numel() < need:
                buf.plan_workspace = torch.empty(int(need * 1.1) + 4096, dtype=torch.uint8, device=weights.device)
            plan = tbe_ext.backward_plan(m.tbe.table_offsets, indices, offsets, weights.size(0),
                                         workspace=buf.plan_workspace)
        with torch.cuda.device(weights.device):
            stream = tbe_ext._stream(weights.device)
            buf.sync(_GRAD_FREE, k, k - 1, stream)
            _lib.call("tbe_allgather_push", grad.data_ptr(), buf.grad_ptrs[slot], buf.world, buf.rank,
                      grad.numel() * grad.element_size(), stream)
            buf.sync(_GRAD_READY, k, k, stream)
        m.apply_local_backward(buf.grad_in[slot], indices, offsets, plan=plan)
        return None, None, None, None


class _NcclRowExchange(torch.autograd.Function):
    """Reduce-scatter forward, all-gather backward: ReduceScatterFunction of the reference
    (sparse_embedding_cuda_ops.py:78-85) on torch.distributed."""

    @staticmethod
    def forward(ctx, partial, group):
        ctx.group = group
        W = dist.get_world_size(group)
        out = torch.empty((partial.shape[0] // W,) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(out, partial.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        W = dist.get_world_size(ctx.group)
        full = torch.empty((grad.shape[0] * W,) + tuple(grad.shape[1:]), dtype=grad.dtype, device=grad.device)
        dist.all_gather_into_tensor(full, grad.contiguous(), group=ctx.group)
        return full, None


class RowShardedEmbeddingBags(TableShardedEmbeddingBags):
    """Row-wise sharding: every rank holds ``rows_per_rank`` rows of each of ``num_tables`` tables
    (the reference's ``DistributedUniformShardedSNN``, models.py:194-209) and looks up the GLOBAL
    batch with indices local to its slice; ``forward`` returns this rank's batch slice
    ``[B/W, T, D]`` of the sum over ranks (reduce-scatter), ``backward`` all-gathers the gradient
    and applies the fused optimizer to the local rows.  ``exchange="fused"``: the lookup kernel
    stores its partial rows straight into the owner's staging slot and one local kernel sums the
    slots; ``exchange="nccl"``: library reduce-scatter / all-gather.  Sum pooling only (a mean over
    a bag needs the bag's global length, which no single rank sees)."""

    def __init__(self, num_tables, rows_per_rank, embedding_dim, global_batch, optimizer=Optimizer.SGD,
                 learning_rate=0.01, eps=None, fp16=False, exchange="fused", group=None, sync_timeout_s=30.0):
        super().__init__(num_tables, rows_per_rank, embedding_dim, global_batch, optimizer=optimizer,
                         learning_rate=learning_rate, eps=eps, fp16=fp16, pooling_mode="sum", exchange=exchange,
                         group=group, sync_timeout_s=sync_timeout_s)
        self.num_tables = num_tables

    def forward(self, indices, offsets):
        if self.world == 1:
            return self.tbe(indices, offsets)
        if self.exchange == "nccl":
            return _NcclRowExchange.apply(self.tbe(indices, offsets), self.group)
        return _FusedRowShardedLookup.apply(self.tbe.embedding_weights, self, indices, offsets)
