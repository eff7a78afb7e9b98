"""Table-wise model-parallel TBE: each rank owns ``T/W`` whole tables, looks up the GLOBAL batch
for them and the pooled ``[B, T/W, D]`` rows are exchanged so that every rank ends with its batch
slice of all tables, ``[B/W, T, D]`` -- the wiring of the reference's
``DistributedPartitionShardedSNN`` (models.py:212-227) and ``All2AllFunction``
(sparse_embedding_cuda_ops.py:88-120), with the layout contract of ``forward_all2all_nccl``
(sparse_embedding_cuda.cpp:471-533):  ``out_j[b', r*T/W + t] = in_r[j*B/W + b', t]``.

Two exchanges:
  * ``exchange="fused"`` -- no separate collective.  The forward kernel stores each pooled row
    straight into the owner rank's ``[B/W, T, D]`` buffer through peer-mapped (symmetric) memory,
    and the backward scatters the local gradient slice to the table owners with one peer-store
    kernel; a stream-ordered NCCL barrier (a one-element all-reduce) separates producers from
    consumers.  Neither direction needs a transpose copy.
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


class _SymmetricBuffers:
    """Peer-mapped buffers of one sharded module: the exchanged outputs and incoming gradients."""

    def __init__(self, B, T_local, D, dtype, device, group):
        import torch.distributed._symmetric_memory as symm_mem
        W = dist.get_world_size(group)
        self.world, self.rank = W, dist.get_rank(group)
        self.out = symm_mem.empty((B // W, T_local * W, D), dtype=dtype, device=device)
        self.grad_in = symm_mem.empty((B, T_local, D), dtype=dtype, device=device)
        self.out_handle = symm_mem.rendezvous(self.out, group=group)
        self.grad_handle = symm_mem.rendezvous(self.grad_in, group=group)
        ptr_array = ctypes.c_void_p * W
        self.out_ptrs = ptr_array(*[int(p) for p in self.out_handle.buffer_ptrs])
        self.grad_ptrs = ptr_array(*[int(p) for p in self.grad_handle.buffer_ptrs])
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.group = group

    def barrier(self):
        # stream-ordered: completes on the device once every rank's preceding kernels have finished
        dist.all_reduce(self._flag, group=self.group)


class _FusedShardedLookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weights, module, indices, offsets):
        m = module
        buf = m._buffers_for(indices.device)
        T, B, D = m.local_tables, m.global_batch, m.embedding_dim
        with torch.cuda.device(weights.device):
            _lib.call("tbe_forward_sharded", weights.data_ptr(), m.tbe.table_offsets.data_ptr(), indices.data_ptr(),
                      offsets.data_ptr(), None, buf.out_ptrs, buf.world, T, B, D, T * buf.world, T * buf.rank,
                      tbe_ext._DTYPES[weights.dtype], tbe_ext._POOLING[m.tbe.pooling_mode],
                      tbe_ext._stream(weights.device))
            buf.barrier()
        ctx.module = m
        ctx.save_for_backward(weights, indices, offsets)
        return buf.out.view(buf.out.shape)

    @staticmethod
    def backward(ctx, grad):
        m = ctx.module
        weights, indices, offsets = ctx.saved_tensors
        buf = m._buffers_for(indices.device)
        T, B, D = m.local_tables, m.global_batch, m.embedding_dim
        grad = grad.contiguous()
        # the sort of the lookups needs no gradient: it runs on a side stream under the exchange
        plan = None
        if m.tbe.optimizer in (Optimizer.SGD, Optimizer.EXACT_ROWWISE_ADAGRAD):
            plan = tbe_ext.backward_plan(m.tbe.table_offsets, indices, offsets, weights.size(0))
        with torch.cuda.device(weights.device):
            _lib.call("tbe_all2all_push", grad.data_ptr(), buf.grad_ptrs, buf.world, buf.rank, B // buf.world,
                      T * D * grad.element_size(), tbe_ext._stream(weights.device))
            buf.barrier()
        m.apply_local_backward(buf.grad_in, indices, offsets, plan=plan)
        return None, None, None, None


class TableShardedEmbeddingBags(nn.Module):
    """``tables_per_rank`` tables on every rank of ``group``; ``forward`` takes this rank's tables'
    indices/offsets over the global batch and returns this rank's ``[B/W, T_total, D]`` slice."""

    def __init__(self, tables_per_rank, num_embeddings, embedding_dim, global_batch, optimizer=Optimizer.SGD,
                 learning_rate=0.01, eps=None, fp16=False, pooling_mode="sum", exchange="fused", group=None):
        super().__init__()
        assert exchange in ("fused", "nccl")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert global_batch % self.world == 0, "world size must divide the global batch"
        self.local_tables = tables_per_rank
        self.embedding_dim = embedding_dim
        self.global_batch = global_batch
        self.exchange = exchange
        self.tbe = TableBatchedEmbeddingBags(tables_per_rank, num_embeddings, embedding_dim, optimizer=optimizer,
                                             learning_rate=learning_rate, eps=eps, fp16=fp16,
                                             pooling_mode=pooling_mode)
        self._symm = None

    def _buffers_for(self, device):
        if self._symm is None:
            w = self.tbe.embedding_weights
            self._symm = _SymmetricBuffers(self.global_batch, self.local_tables, self.embedding_dim, w.dtype, device,
                                           self.group if self.group is not None else dist.group.WORLD)
        return self._symm

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
