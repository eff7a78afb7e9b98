"""Python op layer of the reference's older embedding op (sparse_embedding_cuda_ops.py:24-120):
``LookupFunction``, ``EmbeddingLocation``, ``UniformShardedEmbeddingBags`` and the collective
autograd functions ``ReduceScatterFunction`` / ``All2AllFunction``.

Left out on purpose: the apex / amp_C / horovod imports and ``FastZeroFusedSGD``
(sparse_embedding_cuda_ops.py:8-17,123-155), which belong to the dense part of the reference's
models; the world size comes from ``torch.distributed`` instead of horovod.
"""
import enum
import logging

import torch
import torch.distributed as dist
from torch import nn

from . import sparse_embedding_cuda
from . import table_batched_embeddings


def _world_size():
    return dist.get_world_size() if dist.is_initialized() else 1


def _empty_sparse_grad(weights):
    return torch.empty(tuple(weights.shape), layout=torch.sparse_coo, dtype=weights.dtype, device=weights.device)


class LookupFunction(torch.autograd.Function):
    LR = 0.05  # the reference hard-codes this step size (sparse_embedding_cuda_ops.py:37)

    @staticmethod
    def forward(ctx, weights, indices, offsets=None):
        ctx.save_for_backward(weights, indices, offsets)
        if offsets is None:
            return sparse_embedding_cuda.forward_fast_single(weights, indices)
        return sparse_embedding_cuda.forward_offsets(weights, indices, offsets)

    @staticmethod
    def backward(ctx, grad_output):
        weights, indices, offsets = ctx.saved_tensors
        if offsets is None:
            sparse_embedding_cuda.backward_update_fast_single(grad_output, weights, indices, LookupFunction.LR)
        else:
            sparse_embedding_cuda.backward_update_offsets(grad_output, weights, indices, offsets, LookupFunction.LR)
        return _empty_sparse_grad(weights), None, None


class EmbeddingLocation(enum.Enum):
    DEVICE = 0
    MANAGED = 1
    HOST_MAPPED = 2


class UniformShardedEmbeddingBags(nn.Module):
    """``num_tables`` equally sized tables stored interleaved as ``[E, T, D]``; ``forward`` takes
    dense ``[B, T, L]`` indices, or flat indices with ``offsets [B, T+1]``, and returns ``[B, T, D]``."""

    def __init__(self, num_tables, num_embeddings, embedding_dim, managed=EmbeddingLocation.DEVICE, fp16=False):
        super().__init__()
        dtype = torch.float16 if fp16 else torch.float32
        device = torch.device("cuda", torch.cuda.current_device())
        shape = (num_embeddings, num_tables, embedding_dim)
        if managed == EmbeddingLocation.DEVICE:
            logging.info("Allocating device embedding bag")
            data = torch.randn(*shape, device=device, dtype=dtype)
        else:
            # the reference allocates managed memory for both MANAGED and HOST_MAPPED
            # (sparse_embedding_cuda_ops.py:61-68)
            logging.info("Allocating managed embedding bag")
            data = table_batched_embeddings.new_managed_tensor(torch.empty(1, device=device, dtype=dtype), shape)
            data.normal_()
        self.embedding_weights = nn.Parameter(data)

    def forward(self, sharded_sparse_features, sharded_offsets=None):
        return LookupFunction.apply(self.embedding_weights, sharded_sparse_features, sharded_offsets)


class ReduceScatterFunction(torch.autograd.Function):
    """Row-wise sharding: every rank holds partial sums ``[B, T, D]``; forward reduce-scatters them
    over the batch, backward all-gathers the gradient (sparse_embedding_cuda_ops.py:78-85)."""

    @staticmethod
    def forward(ctx, sharded_embeddings):
        return sparse_embedding_cuda.forward_reducescatter(sharded_embeddings)

    @staticmethod
    def backward(ctx, grad_output):
        return sparse_embedding_cuda.forward_allgather(grad_output)


class All2AllFunction(torch.autograd.Function):
    """Table-wise sharding: ``[B, T/W, D]`` -> ``[B/W, T, D]`` and back
    (sparse_embedding_cuda_ops.py:88-120)."""

    @staticmethod
    def forward(ctx, partitioned_embeddings):
        B = partitioned_embeddings.size(0)
        assert B % _world_size() == 0
        return sparse_embedding_cuda.forward_all2all_nccl(partitioned_embeddings)

    @staticmethod
    def backward(ctx, grad_output):
        from .sharded import pooled_all_to_all_backward
        if _world_size() == 1:
            return grad_output
        return pooled_all_to_all_backward(grad_output.contiguous())
