"""The functions of the reference's older ``sparse_embedding_cuda`` extension
(sparse_embedding_cuda.cpp:568-601) on top of libtbe_b200.so and torch.distributed.

That extension keeps the tables interleaved, ``weights[E][T][D]`` (row ``i`` of table ``t`` at
``weights[i][t]``), and orders bags batch-major.  Seen as a matrix ``[E*T, D]`` this is ONE table
whose row ``i*T + t`` is looked up by bag ``b*T + t``, so every call here rewrites the indices to
``i*T + t`` and runs the table-batched kernels with a single table and ``B*T`` bags; the pooled
``[B*T, 1, D]`` result is the reference's ``[B, T, D]``.  SGD sums repeated rows instead of racing
on them (sparse_embedding_cuda_kernel.cu:464-583 does unsynchronised read-modify-writes).

Collectives use the default ``torch.distributed`` process group instead of the reference's private
MPI-bootstrapped NCCL communicator (sparse_embedding_cuda.cpp:386-415).
"""
import torch
import torch.distributed as dist

from . import table_batched_embeddings as tbe


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _single_table(weights):
    _require(weights.dim() == 3 and weights.is_contiguous(), "weights must be a contiguous [E, T, D] tensor")
    E, T, D = weights.shape
    return weights.view(E * T, D), torch.zeros(1, dtype=torch.int32, device=weights.device), E, T, D


def _dense_lookups(indices, T):
    """[B, T, L] indices -> (int32 row ids i*T + t flattened bag-major, int32 offsets [B*T + 1])."""
    _require(indices.dim() == 3 and indices.size(1) == T, "indices must be [B, T, L]")
    B, _, L = indices.shape
    t = torch.arange(T, device=indices.device, dtype=torch.int64).view(1, T, 1)
    rows = (indices.to(torch.int64) * T + t).to(torch.int32).reshape(-1)
    offsets = torch.arange(B * T + 1, device=indices.device, dtype=torch.int32) * L
    return rows, offsets, B


def _csr_lookups(indices, offsets, T):
    """Flat indices + offsets [B, T+1] (bag (b,t) = offsets[b][t] .. offsets[b][t+1], rows of the
    offsets matrix back to back) -> the same pair as :func:`_dense_lookups`."""
    _require(offsets.dim() == 2 and offsets.size(1) == T + 1, "offsets must be [B, T + 1]")
    B = offsets.size(0)
    offs = offsets.to(torch.int64)
    lengths = (offs[:, 1:] - offs[:, :-1]).reshape(-1)
    flat = torch.cat([offs[:, :-1].reshape(-1), offs[-1, -1:]]).to(torch.int32)
    table_of_bag = torch.arange(B * T, device=indices.device, dtype=torch.int64) % T
    table_of_pos = torch.repeat_interleave(table_of_bag, lengths, output_size=indices.numel())
    rows = (indices.to(torch.int64) * T + table_of_pos).to(torch.int32)
    return rows, flat, B


def forward_fast_single(weights, indices):
    """``[E,T,D]`` weights, ``[B,T,L]`` indices -> pooled sums ``[B,T,D]``
    (sparse_embedding_cuda.cpp:265-274)."""
    w2, to, E, T, D = _single_table(weights)
    rows, offsets, B = _dense_lookups(indices, T)
    return tbe.forward(w2, to, rows, offsets, None, 200, 1, False).view(B, T, D)


forward_single = forward_fast_single  # same contract, slower kernel in the reference (:254-263)


def forward_offsets(weights, indices, offsets):
    """CSR variant: flat ``indices`` and ``offsets [B, T+1]`` (sparse_embedding_cuda.cpp:276-289)."""
    w2, to, E, T, D = _single_table(weights)
    rows, flat, B = _csr_lookups(indices, offsets, T)
    return tbe.forward(w2, to, rows, flat, None, 200, 1, False).view(B, T, D)


def backward_update_fast_single(grad_output, weights, indices, lr):
    """In-place SGD ``weights[i][t] -= lr * grad[b][t]`` for every lookup
    (sparse_embedding_cuda.cpp:309-316)."""
    w2, to, E, T, D = _single_table(weights)
    rows, offsets, B = _dense_lookups(indices, T)
    tbe.backward_sgd(grad_output.reshape(B * T, 1, D), w2, to, rows, offsets, lr, 200, 1, False)


backward_update_single = backward_update_fast_single


def backward_update_offsets(grad_output, weights, indices, offsets, lr):
    """CSR variant of the fused SGD update (sparse_embedding_cuda.cpp:318-322)."""
    w2, to, E, T, D = _single_table(weights)
    rows, flat, B = _csr_lookups(indices, offsets, T)
    tbe.backward_sgd(grad_output.reshape(B * T, 1, D), w2, to, rows, flat, lr, 200, 1, False)


def forward(sharded_weights, scattered_indices):
    raise RuntimeError("the single-process multi-device forward (sparse_embedding_cuda.cpp:207-252) is not provided: "
                       "run one process per GPU")


def forward_all2all(embeddings, result):
    raise RuntimeError("the MPI all-to-all (sparse_embedding_cuda.cpp:358-384) is not provided: use "
                       "forward_all2all_nccl")


def forward_all2all_nccl(embeddings):
    """``[B, T/W, D]`` -> ``[B/W, T, D]`` (sparse_embedding_cuda.cpp:471-533)."""
    from .sharded import pooled_all_to_all
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return embeddings
    _require(embeddings.is_contiguous(), "embeddings must be contiguous")
    return pooled_all_to_all(embeddings)


def forward_reducescatter(embeddings):
    """``[B, T, D]`` partial sums on every rank -> this rank's ``[B/W, T, D]`` slice of their sum
    (sparse_embedding_cuda.cpp:417-448)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return embeddings
    W = dist.get_world_size()
    B, T, D = embeddings.shape
    _require(B % W == 0, "world size must divide the batch")
    out = torch.empty((B // W, T, D), dtype=embeddings.dtype, device=embeddings.device)
    dist.reduce_scatter_tensor(out, embeddings.contiguous())
    return out


def forward_allgather(embeddings):
    """``[B/W, T, D]`` -> ``[B, T, D]`` (sparse_embedding_cuda.cpp:535-566)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return embeddings
    W = dist.get_world_size()
    Bl, T, D = embeddings.shape
    out = torch.empty((Bl * W, T, D), dtype=embeddings.dtype, device=embeddings.device)
    dist.all_gather_into_tensor(out, embeddings.contiguous())
    return out
