"""The step on the input side of a table-sharded lookup: the index all-to-all.

A data-parallel trainer reads, on every rank, the sparse features of ITS batch slice for ALL tables
(``indices`` flattened ``[T][B/W][L]``, ``offsets`` of length ``T*B/W + 1``).  The table-sharded
lookup (``sharded.TableShardedEmbeddingBags``) wants, on rank r, the features of ITS ``T/W`` tables
for the GLOBAL batch, flattened ``[T/W][B][L]`` with sample ``b = j*B/W + b'`` coming from rank j.
The reference's benchmark skips this step and draws table-sharded indices locally on every rank
(pytorch_distributed_benchmark.py:227-231); a real trainer cannot.

Three phases: bag lengths are exchanged with a fixed-size all-to-all; the index counts that follow
from them size a variable-size all-to-all of the indices (one host synchronisation, for the split
sizes); the received ``[W][T/W][B/W]`` bags are then put in ``[T/W][B]`` order on the device by
``tbe_permute_bags``.  The collectives are torch.distributed's (NCCL on GPUs, gloo in the host-logic
tests); the rearrangement is this library's kernel and needs CUDA tensors.
"""
import torch
import torch.distributed as dist

from . import _lib
from . import table_batched_embeddings as tbe_ext


def exchange_indices(indices, offsets, num_tables, group=None):
    """Phases 1 and 2.  Returns ``(recv_indices, recv_lengths)``: the indices received from rank
    0, 1, ... concatenated (each block ordered ``[T/W][B/W][L]``) and the bag lengths
    ``int32 [W, T/W, B/W]``.  Works on CPU tensors with a gloo group (host-logic tests)."""
    W = dist.get_world_size(group)
    T = int(num_tables)
    assert T % W == 0, "world size must divide the number of tables"
    assert (offsets.numel() - 1) % T == 0, "offsets must have T*B_local+1 entries"
    Bl = (offsets.numel() - 1) // T
    Tl = T // W
    lengths = (offsets[1:] - offsets[:-1]).to(torch.int32).contiguous()  # [T][Bl], table-major
    recv_lengths = torch.empty_like(lengths)
    dist.all_to_all_single(recv_lengths, lengths, group=group)  # block j: rank j's [Tl][Bl] for my tables
    recv_lengths = recv_lengths.view(W, Tl, Bl)
    # index counts per peer: what I send is a contiguous range per destination (tables are contiguous)
    bounds = offsets[::Tl * Bl].to(torch.int64)
    send_counts = bounds[1:] - bounds[:-1]
    recv_counts = recv_lengths.view(W, -1).sum(dim=1, dtype=torch.int64)
    counts = torch.stack([send_counts, recv_counts]).cpu().tolist()  # the one host synchronisation
    recv_indices = torch.empty(int(sum(counts[1])), dtype=indices.dtype, device=indices.device)
    dist.all_to_all_single(recv_indices, indices.contiguous(), output_split_sizes=[int(c) for c in counts[1]],
                           input_split_sizes=[int(c) for c in counts[0]], group=group)
    return recv_indices, recv_lengths


def regroup_bags(recv_indices, recv_lengths):
    """Phase 3 (CUDA tensors): ``[W][T/W][B/W]`` bags -> ``(indices, offsets)`` in ``[T/W][B]``
    order, where global sample ``j*B/W + b'`` of table t is source bag ``(j, t, b')``."""
    tbe_ext._check_cuda("recv_indices", recv_indices, torch.int32)
    tbe_ext._check_cuda("recv_lengths", recv_lengths, torch.int32)
    W, Tl, Bl = recv_lengths.shape
    dev = recv_indices.device
    nbags = W * Tl * Bl
    src_offsets = torch.zeros(nbags + 1, dtype=torch.int32, device=dev)
    torch.cumsum(recv_lengths.reshape(-1), 0, out=src_offsets[1:])
    dst_lengths = recv_lengths.permute(1, 0, 2).reshape(-1)  # [Tl][W][Bl] = [Tl][B]
    dst_offsets = torch.zeros(nbags + 1, dtype=torch.int32, device=dev)
    torch.cumsum(dst_lengths, 0, out=dst_offsets[1:])
    src_bag = torch.arange(nbags, dtype=torch.int32, device=dev).view(W, Tl, Bl).permute(1, 0, 2).reshape(-1).contiguous()
    out = torch.empty_like(recv_indices)
    with torch.cuda.device(dev):
        _lib.call("tbe_permute_bags", recv_indices.data_ptr(), src_offsets.data_ptr(), src_bag.data_ptr(),
                  dst_offsets.data_ptr(), out.data_ptr(), nbags, tbe_ext._stream(dev))
    return out, dst_offsets


def indices_all_to_all(indices, offsets, num_tables, group=None):
    """Data-parallel sparse features of this rank -> table-sharded ``(indices, offsets)`` of this
    rank's ``T/W`` tables over the global batch, ready for ``TableShardedEmbeddingBags.forward``."""
    recv_indices, recv_lengths = exchange_indices(indices, offsets, num_tables, group)
    return regroup_bags(recv_indices, recv_lengths)
