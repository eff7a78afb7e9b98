"""Python op layer with the surface of the reference's ``table_batched_embeddings_ops``
(table_batched_embeddings_ops.py:9-201): ``LookupFunction``, ``Optimizer``, ``EmbeddingLocation`` and
``TableBatchedEmbeddingBags``; the optimizer step is fused into the backward, which updates
``embedding_weights`` (and ``optimizer_state``) in place.

Differences, all opt-in or fixes:
  * ``pooling_mode="sum"|"mean"`` keyword (the reference only sums);
  * ``plan_ahead`` keyword: sort the lookups for the backward on a side stream while the forward runs;
  * SGD sums the gradients of repeated rows before the update (the reference's kernel races on
    them, and its Python branch raises a TypeError at table_batched_embeddings_ops.py:66);
  * tensors must be on a CUDA device: there is no CPU path.
"""
import enum
import logging

import numpy as np
import torch
from torch import nn

from . import table_batched_embeddings


class Optimizer(enum.Enum):
    SGD = 1
    APPROX_ROWWISE_ADAGRAD = 2
    EXACT_ROWWISE_ADAGRAD = 3


class EmbeddingLocation(enum.Enum):
    DEVICE = 0
    HOST_MAPPED = 1


_L_MAX_HINT = 200  # launch hint of the reference's kernels; ignored by this library


def _bt_block_hint(embedding_dim):
    return max(256 // int(embedding_dim), 1)


def _empty_sparse_grad(weights):
    # The reference hands autograd an empty sparse tensor for the weights slot
    # (table_batched_embeddings_ops.py:111): the real update already happened in place.
    return torch.empty(tuple(weights.shape), layout=torch.sparse_coo, dtype=weights.dtype, device=weights.device)


class LookupFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weights, table_offsets, indices, offsets, per_sample_weights, optimizer, optimizer_state,
                learning_rate, eps, stochastic_rounding, pooling_mode="sum", plan_ahead=False):
        ctx.optimizer = optimizer
        ctx.learning_rate = learning_rate
        ctx.eps = eps
        ctx.stochastic_rounding = stochastic_rounding
        ctx.pooling_mode = pooling_mode
        ctx.plan = None
        ctx.save_for_backward(weights, table_offsets, indices, offsets, per_sample_weights, optimizer_state)
        if (plan_ahead and weights.requires_grad and optimizer != Optimizer.APPROX_ROWWISE_ADAGRAD):
            # launched before the forward so its kernels are queued first
            ctx.plan = table_batched_embeddings.backward_plan(table_offsets, indices, offsets, weights.size(0))
        return table_batched_embeddings.forward(
            weights, table_offsets, indices, offsets, per_sample_weights, _L_MAX_HINT,
            _bt_block_hint(weights.shape[1]), False, pooling_mode=pooling_mode)

    @staticmethod
    def backward(ctx, grad_output):
        weights, table_offsets, indices, offsets, per_sample_weights, optimizer_state = ctx.saved_tensors
        assert ctx.optimizer in (Optimizer.SGD, Optimizer.APPROX_ROWWISE_ADAGRAD, Optimizer.EXACT_ROWWISE_ADAGRAD)
        grad_per_sample_weight = None
        if ctx.optimizer == Optimizer.SGD:
            assert per_sample_weights is None
            table_batched_embeddings.backward_sgd(
                grad_output, weights, table_offsets, indices, offsets, ctx.learning_rate, _L_MAX_HINT,
                _bt_block_hint(weights.shape[1]), False, pooling_mode=ctx.pooling_mode, plan=ctx.plan)
        elif ctx.optimizer == Optimizer.APPROX_ROWWISE_ADAGRAD:
            assert ctx.pooling_mode == "sum", "approximate rowwise Adagrad supports sum pooling only"
            grad_per_sample_weight = table_batched_embeddings.backward_approx_adagrad(
                grad_output, weights, table_offsets, indices, offsets, per_sample_weights, optimizer_state,
                ctx.learning_rate, ctx.eps, _L_MAX_HINT, ctx.stochastic_rounding, 1)
        else:
            table_batched_embeddings.backward_exact_adagrad(
                grad_output, weights, table_offsets, indices, offsets, per_sample_weights, optimizer_state,
                ctx.learning_rate, ctx.eps, ctx.stochastic_rounding, 1, pooling_mode=ctx.pooling_mode, plan=ctx.plan)
        ctx.plan = None
        return (_empty_sparse_grad(weights), None, None, None, grad_per_sample_weight, None, None, None, None,
                None, None, None)


class TableBatchedEmbeddingBags(nn.Module):
    """T tables of ``num_embeddings`` rows and ``embedding_dim`` columns behind one lookup.

    ``forward(indices, offsets[, per_sample_weights])`` takes int32 ``indices`` flattened as
    ``[T][B][L]`` and int32 ``offsets`` of length ``T*B+1`` and returns ``[B, T, D]``.
    """

    def __init__(self, num_tables, num_embeddings, embedding_dim, optimizer=Optimizer.SGD, learning_rate=0.01,
                 eps=None, stochastic_rounding=False, fp16=False, managed=EmbeddingLocation.DEVICE, *,
                 pooling_mode="sum", plan_ahead=False):
        super().__init__()
        assert managed in (EmbeddingLocation.DEVICE, EmbeddingLocation.HOST_MAPPED)
        assert pooling_mode in ("sum", "mean")
        dtype = torch.float16 if fp16 else torch.float32
        device = torch.device("cuda", torch.cuda.current_device())
        total_rows = num_tables * num_embeddings
        if managed == EmbeddingLocation.DEVICE:
            logging.info("Allocating device embedding bag")
            embedding_data = torch.randn(total_rows, embedding_dim, device=device, dtype=dtype)
        else:
            logging.info("Allocating host-mapped embedding bag")
            proto = torch.empty(1, device=device, dtype=dtype)
            embedding_data = table_batched_embeddings.new_managed_tensor(proto, (total_rows, embedding_dim))
            embedding_data.normal_()
        self.embedding_weights = nn.Parameter(embedding_data)
        self.register_buffer(
            "table_offsets",
            torch.tensor([0] + np.cumsum([num_embeddings] * (num_tables - 1)).tolist(), dtype=torch.int32))
        self.register_buffer("optimizer_state", torch.zeros(total_rows, dtype=torch.float32))
        self.optimizer = optimizer
        self.learning_rate = learning_rate
        self.eps = eps
        self.stochastic_rounding = stochastic_rounding
        self.pooling_mode = pooling_mode
        self.plan_ahead = plan_ahead

    def forward(self, sharded_sparse_features, sharded_offsets, per_sample_weights=None):
        return LookupFunction.apply(
            self.embedding_weights, self.table_offsets, sharded_sparse_features, sharded_offsets,
            per_sample_weights, self.optimizer, self.optimizer_state, self.learning_rate, self.eps,
            self.stochastic_rounding, self.pooling_mode, self.plan_ahead)


class MixedDimLookupFunction(torch.autograd.Function):
    """Lookup over tables of different width and height (table_batched_embeddings_ops.py:204-321)."""

    @staticmethod
    def forward(ctx, weights, table_offsets, table_dim_offsets, dim_offsets, total_D, indices, offsets,
                per_sample_weights, optimizer, optimizer_state, learning_rate, eps, stochastic_rounding):
        ctx.optimizer = optimizer
        ctx.learning_rate = learning_rate
        ctx.eps = eps
        ctx.stochastic_rounding = stochastic_rounding
        ctx.total_D = total_D
        ctx.save_for_backward(weights, table_offsets, table_dim_offsets, dim_offsets, indices, offsets,
                              per_sample_weights, optimizer_state)
        return table_batched_embeddings.forward_mixed_D(weights, table_offsets, dim_offsets, total_D, indices, offsets,
                                                        per_sample_weights, _L_MAX_HINT, 1, False)

    @staticmethod
    def backward(ctx, grad_output):
        (weights, table_offsets, table_dim_offsets, dim_offsets, indices, offsets, per_sample_weights,
         optimizer_state) = ctx.saved_tensors
        assert ctx.optimizer in (Optimizer.APPROX_ROWWISE_ADAGRAD, Optimizer.EXACT_ROWWISE_ADAGRAD)
        if ctx.optimizer == Optimizer.APPROX_ROWWISE_ADAGRAD:
            grad_psw = table_batched_embeddings.backward_approx_adagrad_mixed_D(
                grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, ctx.total_D, indices, offsets,
                per_sample_weights, optimizer_state, ctx.learning_rate, ctx.eps, _L_MAX_HINT, ctx.stochastic_rounding, 1)
        else:
            grad_psw = table_batched_embeddings.backward_exact_adagrad_mixed_D(
                grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, ctx.total_D, indices, offsets,
                per_sample_weights, optimizer_state, ctx.learning_rate, ctx.eps, ctx.stochastic_rounding, 1)
        return (_empty_sparse_grad(weights), None, None, None, None, None, None, grad_psw, None, None, None, None,
                None)


class MixedDimTableBatchedEmbeddingBags(nn.Module):
    """``embeddings = [(rows, dim), ...]``: one flat weights vector, ``table_offsets`` (int64, element
    offset of every table, T+1 entries), ``table_dim_offsets`` (int32, row offset, T+1), ``dim_offsets``
    (int32, output column offset, T+1); ``forward`` returns ``[B, sum(dim)]``."""

    def __init__(self, embeddings, optimizer=Optimizer.SGD, learning_rate=0.01, eps=None, stochastic_rounding=False,
                 fp16=False, managed=EmbeddingLocation.DEVICE):
        super().__init__()
        assert managed in (EmbeddingLocation.DEVICE, EmbeddingLocation.HOST_MAPPED)
        rows, dims = zip(*embeddings)
        dtype = torch.float16 if fp16 else torch.float32
        device = torch.device("cuda", torch.cuda.current_device())
        numel = sum(r * d for r, d in embeddings)
        if managed == EmbeddingLocation.DEVICE:
            data = torch.randn(numel, device=device, dtype=dtype)
        else:
            data = table_batched_embeddings.new_managed_tensor(torch.empty(1, device=device, dtype=dtype), (numel,))
            data.normal_()
        self.embedding_weights = nn.Parameter(data)
        self.register_buffer("table_dim_offsets", torch.tensor([0] + np.cumsum(rows).tolist(), dtype=torch.int32))
        self.register_buffer("table_offsets",
                             torch.tensor([0] + np.cumsum([r * d for r, d in embeddings]).tolist(), dtype=torch.int64))
        self.register_buffer("dim_offsets", torch.tensor([0] + np.cumsum(dims).tolist(), dtype=torch.int32))
        self.register_buffer("optimizer_state", torch.zeros(sum(rows), dtype=torch.float32))
        self.total_D = sum(dims)
        self.optimizer = optimizer
        self.learning_rate = learning_rate
        self.eps = eps
        self.stochastic_rounding = stochastic_rounding

    def forward(self, sharded_sparse_features, sharded_offsets, per_sample_weights=None):
        return MixedDimLookupFunction.apply(
            self.embedding_weights, self.table_offsets, self.table_dim_offsets, self.dim_offsets, self.total_D,
            sharded_sparse_features, sharded_offsets, per_sample_weights, self.optimizer, self.optimizer_state,
            self.learning_rate, self.eps, self.stochastic_rounding)

    def _T(self):
        return self.table_offsets.numel() - 1

    def split_embedding_weights(self):
        """The weights of every table as ``[rows, dim]`` views."""
        eo, ro, do = self.table_offsets.tolist(), self.table_dim_offsets.tolist(), self.dim_offsets.tolist()
        return [self.embedding_weights.detach()[eo[i]:eo[i + 1]].view(ro[i + 1] - ro[i], do[i + 1] - do[i])
                for i in range(self._T())]

    def split_optimizer_state(self):
        ro = self.table_dim_offsets.tolist()
        return [self.optimizer_state.detach()[ro[i]:ro[i + 1]] for i in range(self._T())]

    def split_output(self, output):
        do = self.dim_offsets.tolist()
        return [output[:, do[i]:do[i + 1]] for i in range(self._T())]
