"""CPU oracle for the table-batched embedding-bag (TBE) hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, what the reference computes on its TBE path.  It is imported by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` -- never by the product package, which has no CPU path.

The arithmetic of the pooled lookup lives in a third-party dependency of the reference, PyTorch
(this container pins torch 2.11.0+cu128): the reference's own tests use per-table
``torch.nn.EmbeddingBag(E, D, mode="sum", sparse=True)`` as their oracle
(test_table_batched_embeddings.py:127,138-141,174,186,238,255-260), and so does this file, following
the formulas of those tests:
  forward          test_table_batched_embeddings.py:115-160
  SGD              test_table_batched_embeddings.py:163-216   (w - lr * grad)
  rowwise Adagrad  test_table_batched_embeddings.py:296-318   (state = sum_d grad^2,
                                                               w - lr * grad / (sqrt(state) + eps))

Parity is PINNED by the reference itself: ``oracle/build_ref.py`` builds the reference's
``table_batched_embeddings`` extension from its own sources (kernels unmodified),
``tests/golden/make_reference_golden.py`` ran it on a B200 and stored its outputs as
``tests/golden/reference_*.npz``, and ``tests/test_oracle_reference_pin.py`` checks every function
below that has a counterpart there (forward, weighted forward, SGD, exact and approximate rowwise
Adagrad with state and per-sample-weight gradient, mixed widths, construct_offsets) against them.
The reference ships no golden vectors of its own (every test draws fresh random inputs).
Parts with no counterpart in the reference -- mean pooling, SGD on repeated rows (the reference
races), the all-to-all layout (its test asserts nothing), the row cache -- remain unpinned by it
and are pinned here by EmbeddingBag(mode="mean"), by ``w - lr * grad.to_dense()``, by the layout
formula of sparse_embedding_cuda.cpp:475-532 and by this file's own cache model.
"""
import numpy as np
import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ layout helpers
def table_row_ranges(table_offsets, total_rows):
    """[(first_row, end_row)] per table from the reference's ``table_offsets`` buffer
    (table_batched_embeddings_ops.py:170-176: first row of each table, length T)."""
    offs = [int(x) for x in table_offsets]
    ends = offs[1:] + [int(total_rows)]
    return list(zip(offs, ends))


def get_table_batched_offsets_from_dense(merged_indices):
    """[T][B][L] dense indices -> (flat int32 indices, int32 offsets of length T*B+1); follows
    table_batched_embeddings_benchmark.py:17-24 / test_table_batched_embeddings.py:24-31."""
    merged_indices = np.asarray(merged_indices)
    T, B, L = merged_indices.shape
    offsets = np.arange(T * B + 1, dtype=np.int64) * L
    return merged_indices.reshape(-1).astype(np.int32), offsets.astype(np.int32)


def offsets_from_lengths(lengths):
    """[T][B] bag lengths -> int32 offsets [T*B+1] (cumsum with a leading zero)."""
    flat = np.asarray(lengths, dtype=np.int64).reshape(-1)
    return np.concatenate([[0], np.cumsum(flat)]).astype(np.int32)


def construct_offsets(batch_offsets_per_table, total_indices_per_table):
    """Restates construct_offsets_kernel (table_batched_embeddings_cuda.cu:1165-1188): output[0]=0 and
    output[1+t*B+b] = length of bag (t,b); the caller applies cumsum
    (test_table_batched_embeddings.py:49-58)."""
    begin = np.asarray(batch_offsets_per_table, dtype=np.int64)
    totals = np.asarray(total_indices_per_table, dtype=np.int64)
    T, B = begin.shape
    out = np.zeros(1 + T * B, dtype=np.int32)
    for t in range(T):
        upper = np.concatenate([begin[t, 1:], totals[t:t + 1]])
        out[1 + t * B:1 + (t + 1) * B] = (upper - begin[t]).astype(np.int32)
    return out


def _per_table_inputs(indices, offsets, T, B, t):
    """Indices of table t and bag offsets local to it (int64, as EmbeddingBag wants)."""
    offsets = np.asarray(offsets, dtype=np.int64)
    lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
    idx = torch.from_numpy(np.asarray(indices[lo:hi], dtype=np.int64))
    off = torch.from_numpy(offsets[t * B:(t + 1) * B] - lo)
    return idx, off, lo, hi


# ------------------------------------------------------------------ forward / gradients
def forward(weights, table_offsets, indices, offsets, per_sample_weights=None, pooling_mode="sum",
            compute_dtype=None):
    """Pooled lookup ``[B, T, D]`` as the concatenation of per-table EmbeddingBag outputs
    (test_table_batched_embeddings.py:138-146).  ``compute_dtype`` upcasts the table first (the
    CUDA kernels accumulate fp16 tables in fp32); the result is cast back to the table dtype."""
    weights = torch.as_tensor(weights)
    T = len(table_offsets)
    B = (len(offsets) - 1) // T
    D = weights.shape[1]
    out_dtype = weights.dtype
    cd = compute_dtype or weights.dtype
    outs = []
    for t, (r0, r1) in enumerate(table_row_ranges(table_offsets, weights.shape[0])):
        idx, off, lo, hi = _per_table_inputs(indices, offsets, T, B, t)
        psw = None
        if per_sample_weights is not None:
            psw = torch.as_tensor(per_sample_weights)[lo:hi].to(cd)
        o = F.embedding_bag(idx, weights[r0:r1].to(cd), off, mode=pooling_mode, per_sample_weights=psw)
        outs.append(o.view(B, 1, D))
    return torch.cat(outs, dim=1).to(out_dtype)


def dense_gradients(weights, table_offsets, indices, offsets, grad_output, per_sample_weights=None,
                    pooling_mode="sum", compute_dtype=None):
    """Per-table dense gradient ``[E_t, D]`` of sum(out * grad_output), obtained the way the
    reference's tests do: a sparse EmbeddingBag backward, then ``weight.grad.to_dense()``
    (test_table_batched_embeddings.py:186-193,255-262).  Also returns the gradient of the per-sample
    weights (or None)."""
    weights = torch.as_tensor(weights)
    grad_output = torch.as_tensor(grad_output)
    T = len(table_offsets)
    B = (len(offsets) - 1) // T
    cd = compute_dtype or weights.dtype
    grads, psw_grads = [], []
    for t, (r0, r1) in enumerate(table_row_ranges(table_offsets, weights.shape[0])):
        idx, off, lo, hi = _per_table_inputs(indices, offsets, T, B, t)
        bag = torch.nn.EmbeddingBag(r1 - r0, weights.shape[1], mode=pooling_mode, sparse=True)
        bag.weight = torch.nn.Parameter(weights[r0:r1].detach().clone().to(cd))
        psw = None
        if per_sample_weights is not None:
            psw = torch.as_tensor(per_sample_weights)[lo:hi].detach().clone().to(cd).requires_grad_(True)
        out = bag(idx, off, per_sample_weights=psw)
        out.backward(grad_output[:, t, :].to(cd))
        g = bag.weight.grad
        grads.append(g.to_dense() if g is not None else torch.zeros(r1 - r0, weights.shape[1], dtype=cd))
        if psw is not None:
            psw_grads.append(psw.grad)
    psw_grad = torch.cat(psw_grads) if psw_grads else None
    return grads, psw_grad


def sgd_step(weights, table_offsets, indices, offsets, grad_output, lr, pooling_mode="sum", compute_dtype=None):
    """weights after one fused SGD step: ``w - lr * dense_grad`` per table
    (test_table_batched_embeddings.py:191-193)."""
    weights = torch.as_tensor(weights)
    grads, _ = dense_gradients(weights, table_offsets, indices, offsets, grad_output, None, pooling_mode,
                               compute_dtype)
    cd = compute_dtype or weights.dtype
    new = weights.detach().clone()
    for (r0, r1), g in zip(table_row_ranges(table_offsets, weights.shape[0]), grads):
        new[r0:r1] = (weights[r0:r1].to(cd) - g * lr).to(weights.dtype)
    return new


def exact_rowwise_adagrad_step(weights, state, table_offsets, indices, offsets, grad_output, lr, eps,
                               pooling_mode="sum", compute_dtype=torch.float32):
    """(weights, state) after one exact rowwise-Adagrad step.  Follows the reference's test formula
    (test_table_batched_embeddings.py:296-318) and kernel (table_batched_embeddings_cuda.cu:442-455,
    1547-1585): state += sum over D of the squared summed gradient (a SUM, not a mean), then
    w -= lr * G / (sqrt(state_new) + eps)."""
    weights = torch.as_tensor(weights)
    grads, _ = dense_gradients(weights, table_offsets, indices, offsets, grad_output, None, pooling_mode,
                               compute_dtype)
    new_w = weights.detach().clone()
    new_s = torch.as_tensor(state).detach().clone().float()
    for (r0, r1), g in zip(table_row_ranges(table_offsets, weights.shape[0]), grads):
        g = g.float()
        new_s[r0:r1] += g.pow(2).sum(dim=1)
        denom = new_s[r0:r1].sqrt().add(eps).view(-1, 1)
        new_w[r0:r1] = torch.addcdiv(weights[r0:r1].float(), g, denom, value=-lr).to(weights.dtype)
    return new_w, new_s


def approx_rowwise_adagrad_step(weights, state, table_offsets, indices, offsets, grad_output, lr, eps,
                                per_sample_weights=None):
    """(weights, state, grad_per_sample_weights) after one approximate rowwise-Adagrad step.

    Restates batched_embedding_backward_adagrad_approx_kernel_1 and its functors
    (table_batched_embeddings_cuda.cu:437-555,648-704) with the lookups applied one at a time in
    ascending index position: per lookup l of bag (b,t) with row r,
        g2 = |grad[b][t]|^2 * w_l^2;  state[r] += g2;
        mult = w_l * lr / (sqrt(state[r]) + eps);  weights[r] -= mult * grad[b][t]
    and grad_psw[l] = <weights_before_step[r], grad[b][t]>.  A row is kept in fp32 across its
    lookups and rounded to the table dtype once.  The reference applies lookups concurrently
    without atomics, so only inputs without repeated rows are comparable with it.
    Pure-Python loop: small cases only."""
    w0 = torch.as_tensor(weights).detach().clone()
    w = w0.float().clone()
    s = torch.as_tensor(state).detach().clone().float()
    go = torch.as_tensor(grad_output).float()
    T = len(table_offsets)
    B = (len(offsets) - 1) // T
    psw = None if per_sample_weights is None else torch.as_tensor(per_sample_weights).float()
    grad_psw = None if psw is None else torch.zeros(len(indices), dtype=torch.float32)
    g2_bag = go.pow(2).sum(dim=2)  # [B, T]
    for t in range(T):
        r0 = int(table_offsets[t])
        for b in range(B):
            for p in range(int(offsets[t * B + b]), int(offsets[t * B + b + 1])):
                r = r0 + int(indices[p])
                wl = 1.0 if psw is None else float(psw[p])
                if grad_psw is not None:
                    grad_psw[p] = torch.dot(w0[r].float(), go[b, t])
                s[r] += g2_bag[b, t] * wl * wl
                mult = wl * lr / (float(torch.sqrt(s[r])) + eps)
                w[r] -= mult * go[b, t]
    return w.to(w0.dtype), s, (None if grad_psw is None else grad_psw.to(w0.dtype))


# ------------------------------------------------------------------ integer bookkeeping
def sort_segments(table_offsets, indices, offsets):
    """The backward's bookkeeping, restating linear_index_weight_offsets_kernel + the radix sort +
    the segment scan (table_batched_embeddings_cuda.cu:1471-1497,1523-1539,1638-1655) with a
    stable sort: returns (sorted_rows, sorted_bags, segment_starts) as int32 arrays."""
    indices = np.asarray(indices, dtype=np.int64)
    offsets = np.asarray(offsets, dtype=np.int64)
    T = len(table_offsets)
    B = (len(offsets) - 1) // T
    lengths = np.diff(offsets)
    bag_of_pos = np.repeat(np.arange(T * B, dtype=np.int64), lengths)
    row0 = np.asarray([int(x) for x in table_offsets], dtype=np.int64)
    linear = row0[bag_of_pos // B] + indices
    order = np.argsort(linear, kind="stable")
    rows = linear[order]
    bags = bag_of_pos[order]
    if len(rows):
        starts = np.flatnonzero(np.concatenate([[True], rows[1:] != rows[:-1]]))
    else:
        starts = np.zeros(0, dtype=np.int64)
    return rows.astype(np.int32), bags.astype(np.int32), starts.astype(np.int32)


def unique_rows(table_offsets, indices, offsets):
    """Number of distinct (table,row) pairs in a batch (U in the roofline byte count)."""
    rows, _, starts = sort_segments(table_offsets, indices, offsets)
    return int(len(starts))


# ------------------------------------------------------------------ table-sharded exchange
def all_to_all_pooled(per_rank_outputs):
    """Layout contract of forward_all2all_nccl (sparse_embedding_cuda.cpp:471-533): rank r holds
    in_r = [B][T/W][D] for its own tables over the global batch; rank j receives
    out_j[b', r*(T/W) + t, :] = in_r[j*(B/W) + b', t, :]."""
    W = len(per_rank_outputs)
    B, Tl, D = per_rank_outputs[0].shape
    assert B % W == 0
    Bl = B // W
    outs = []
    for j in range(W):
        outs.append(torch.cat([torch.as_tensor(per_rank_outputs[r])[j * Bl:(j + 1) * Bl] for r in range(W)], dim=1))
    return outs


def all_to_all_pooled_backward(per_rank_grads):
    """Inverse exchange (All2AllFunction.backward, sparse_embedding_cuda_ops.py:104-117): rank j
    holds grad_j = [B/W][T][D]; rank r receives grad_in_r[j*(B/W)+b', t, :] = grad_j[b', r*(T/W)+t, :]."""
    W = len(per_rank_grads)
    Bl, T, D = per_rank_grads[0].shape
    assert T % W == 0
    Tl = T // W
    outs = []
    for r in range(W):
        outs.append(torch.cat([torch.as_tensor(per_rank_grads[j])[:, r * Tl:(r + 1) * Tl] for j in range(W)], dim=0))
    return outs


def index_all_to_all(per_rank_indices, per_rank_offsets, num_tables):
    """What the index all-to-all must deliver (no counterpart in the reference, which fabricates
    table-sharded indices, pytorch_distributed_benchmark.py:227-231): rank j holds the features of its
    batch slice for all T tables ([T][B/W] bags); rank r receives, for its tables
    [r*T/W, (r+1)*T/W), bag (t, j*B/W + b') = rank j's bag (r*T/W + t, b').  Returns per rank
    (indices, offsets) in [T/W][B] order.  Pure-Python loops: small cases only."""
    W = len(per_rank_indices)
    T = int(num_tables)
    Tl = T // W
    Bl = (len(per_rank_offsets[0]) - 1) // T
    out = []
    for r in range(W):
        idx, lens = [], []
        for t in range(Tl):
            for j in range(W):
                off = np.asarray(per_rank_offsets[j], dtype=np.int64)
                for b in range(Bl):
                    bag = (r * Tl + t) * Bl + b
                    seg = np.asarray(per_rank_indices[j][off[bag]:off[bag + 1]])
                    idx.append(seg)
                    lens.append(len(seg))
        indices = np.concatenate(idx).astype(np.int32) if idx else np.zeros(0, dtype=np.int32)
        out.append((indices, np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)))
    return out


def reduce_scatter_pooled(per_rank_partials):
    """Row-wise sharding, forward (forward_reducescatter, sparse_embedding_cuda.cpp:417-448, tested by
    test_sparse_embedding_cuda.py:138-171): every rank holds partial pooled rows [B][T][D] for the
    global batch; rank j receives the sum over ranks of rows [j*B/W, (j+1)*B/W)."""
    W = len(per_rank_partials)
    B = per_rank_partials[0].shape[0]
    assert B % W == 0
    Bl = B // W
    total = torch.stack([torch.as_tensor(p).double() for p in per_rank_partials]).sum(0)
    return [total[j * Bl:(j + 1) * Bl].to(torch.as_tensor(per_rank_partials[0]).dtype) for j in range(W)]


def all_gather_pooled_backward(per_rank_grads):
    """Backward of the reduce-scatter (forward_allgather, sparse_embedding_cuda.cpp:535-566): every rank
    receives the concatenation over ranks of the gradient slices [B/W][T][D] -> [B][T][D]."""
    full = torch.cat([torch.as_tensor(g) for g in per_rank_grads], dim=0)
    return [full.clone() for _ in per_rank_grads]


# ------------------------------------------------------------------ timed CPU baseline
class PerTableEmbeddingBags:
    """The reference's CPU path for this workload: one ``nn.EmbeddingBag(sparse=True)`` per table,
    forward, backward, sparse SGD (sparse_embedding_cuda_benchmark.py:39-42,56-57,91-96;
    models.py:11-34).  Used as the timed CPU baseline."""

    def __init__(self, num_tables, num_embeddings, embedding_dim, dtype=torch.float32, pooling_mode="sum", seed=0):
        gen = torch.Generator().manual_seed(seed)
        self.bags = []
        for _ in range(num_tables):
            bag = torch.nn.EmbeddingBag(num_embeddings, embedding_dim, mode=pooling_mode, sparse=True)
            w = (torch.rand(num_embeddings, embedding_dim, generator=gen) * 0.02 - 0.01).to(dtype)
            bag.weight = torch.nn.Parameter(w)
            self.bags.append(bag)

    def step(self, per_table_indices, per_table_offsets, per_table_grads, lr, backward=True):
        outs = []
        for bag, idx, off in zip(self.bags, per_table_indices, per_table_offsets):
            outs.append(bag(idx, off))
        if backward:
            for bag, out, g in zip(self.bags, outs, per_table_grads):
                bag.weight.grad = None
                out.backward(g)
                bag.weight.data.add_(bag.weight.grad, alpha=-lr)
        return outs


# ------------------------------------------------------------------ LXU cache model
class LXUCacheModel:
    """CPU model of the set-associative row cache (no counterpart in the reference: parity unpinned
    by it; this model IS the specification the CUDA cache is compared with, slot by slot).

    Row r lives in set ``mix(r) % num_sets`` where ``mix`` is a fixed bijection of 31-bit ids (so that
    rows a table-size apart do not collide); "ascending order" below is ascending ``mix(r)``.  Per step, with ``now`` = 1, 2, ...: every distinct row of
    the batch is looked up first -- a hit sets ``last_use = now`` and adds one to ``use_count`` --
    then the misses of each set, in ascending mixed-id order, claim a way with ``last_use < now`` (or an
    empty one): empty ways first, then the smallest ``last_use`` (LRU) or the smallest
    ``use_count`` (LFU), ties to the lowest way.  A claimed way gets ``last_use = now``,
    ``use_count = 1``.  A miss with no claimable way stays uncached for the step (location -1)."""

    def __init__(self, num_sets, ways, policy="lru"):
        self.num_sets, self.ways, self.policy = num_sets, ways, policy
        self.tags = np.full(num_sets * ways, -1, dtype=np.int32)
        self.last_use = np.zeros(num_sets * ways, dtype=np.int32)
        self.use_count = np.zeros(num_sets * ways, dtype=np.int32)
        self.now = 0

    @staticmethod
    def mix(r):
        x = int(r) & 0x7FFFFFFF
        x ^= x >> 16
        x = (x * 0x45D9F3B) & 0x7FFFFFFF
        x ^= x >> 16
        x = (x * 0x45D9F3B) & 0x7FFFFFFF
        x ^= x >> 16
        return x

    def set_of(self, r):
        return self.mix(r) % self.num_sets

    def step(self, table_offsets, indices, offsets):
        """Returns (locations int32 [N], stats dict) for one batch and updates the model."""
        self.now += 1
        indices = np.asarray(indices, dtype=np.int64)
        offsets = np.asarray(offsets, dtype=np.int64)
        T = len(table_offsets)
        B = (len(offsets) - 1) // T
        bag_of_pos = np.repeat(np.arange(T * B, dtype=np.int64), np.diff(offsets))
        rows = np.asarray([int(x) for x in table_offsets], dtype=np.int64)[bag_of_pos // B] + indices
        uniq, counts = np.unique(rows, return_counts=True)
        where = {}
        hit_lookups = hit_rows = 0
        by_set = {}
        for r, c in zip(uniq.tolist(), counts.tolist()):
            by_set.setdefault(self.set_of(r), []).append((r, c))
        fetched = uncached = 0
        for s, members in by_set.items():
            base = s * self.ways
            misses = []
            for r, c in members:  # hits first
                hit = [w for w in range(self.ways) if self.tags[base + w] == r]
                if hit:
                    w = hit[0]
                    self.last_use[base + w] = self.now
                    self.use_count[base + w] += 1
                    where[r] = base + w
                    hit_lookups += c
                    hit_rows += 1
                else:
                    misses.append(r)
            for r in sorted(misses, key=self.mix):
                best = None
                for w in range(self.ways):
                    slot = base + w
                    if self.tags[slot] >= 0 and self.last_use[slot] >= self.now:
                        continue
                    prio = 0 if self.tags[slot] < 0 else int(self.last_use[slot] if self.policy == "lru"
                                                             else self.use_count[slot]) + 1
                    if best is None or (prio, w) < best:
                        best = (prio, w)
                if best is None:
                    where[r] = -1
                    uncached += 1
                    continue
                slot = base + best[1]
                self.tags[slot] = r
                self.last_use[slot] = self.now
                self.use_count[slot] = 1
                where[r] = slot
                fetched += 1
        loc = np.asarray([where[r] for r in rows.tolist()], dtype=np.int32)
        stats = {"lookups": len(rows), "rows": len(uniq), "fetched": fetched, "hit_lookups": hit_lookups,
                 "hit_rows": hit_rows, "uncached": uncached}
        return loc, stats
