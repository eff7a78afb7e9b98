"""Seeded synthetic TBE workloads: the five benchmark configurations and the headline target.

No public dataset stands behind the reference's benchmarks (its own micro-benchmark draws random
indices, table_batched_embeddings_benchmark.py:133-145), so these generators are the stand-in:
``numpy.random.default_rng(seed)``, weights ~ U(-0.01, 0.01), int32 indices flattened ``[T][B][L]``
and ``offsets = [0] + cumsum(lengths)`` (table_batched_embeddings_benchmark.py:17-24).
"""
import dataclasses

import numpy as np


@dataclasses.dataclass
class Workload:
    name: str
    T: int                    # tables (per rank when sharded)
    E: int                    # rows per table
    D: int
    B: int                    # batch (global batch when sharded)
    dtype: str                # "fp16" | "fp32"
    pooling: str = "sum"
    optimizer: str = "sgd"    # "none" | "sgd" | "exact_rowwise_adagrad"
    lr: float = 0.1
    eps: float = 1e-8
    L: int = 0                # fixed bag length, 0 = variable
    L_dist: str = "fixed"     # "fixed" | "poisson"
    L_mean: float = 0.0
    L_min: int = 1
    L_max: int = 0
    index_dist: str = "uniform"  # "uniform" | "zipf"
    zipf_alpha: float = 0.0
    seed: int = 0

    @property
    def elem_bytes(self):
        return 2 if self.dtype == "fp16" else 4


WORKLOADS = {
    # CPU-runnable correctness case
    "cfg1": Workload("cfg1", T=4, E=10_000, D=64, B=128, dtype="fp32", L=10, optimizer="sgd", lr=0.1),
    # single-GPU forward only
    "cfg2": Workload("cfg2", T=64, E=1_000_000, D=128, B=2048, dtype="fp16", L=38, optimizer="none"),
    # single-GPU fwd+bwd, fused exact rowwise Adagrad, Zipf rows, Poisson lengths, mean pooling
    "cfg3": Workload("cfg3", T=64, E=1_000_000, D=128, B=2048, dtype="fp32", pooling="mean",
                     optimizer="exact_rowwise_adagrad", lr=0.01, eps=1e-8, L_dist="poisson", L_mean=20.0,
                     L_min=1, L_max=100, index_dist="zipf", zipf_alpha=1.05),
    # cached TBE over host-resident tables
    "cfg4": Workload("cfg4", T=32, E=10_000_000, D=128, B=4096, dtype="fp16", L=20, optimizer="sgd", lr=0.05,
                     index_dist="zipf", zipf_alpha=1.2),
    # table-sharded TBE, 64 tables per GPU over the global batch
    "cfg5": Workload("cfg5", T=64, E=1_000_000, D=128, B=65_536, dtype="fp16", L=32, optimizer="sgd", lr=0.05),
    # Stand-ins of the same kernels for profiler captures: a quarter / an eighth of the tables of the
    # target / cfg3 with everything per table unchanged (rows, bags, bag lengths, index distribution),
    # so every kernel sees the same row reuse, sort geometry and 4 GB of tables (far above L2) while
    # one launch lasts a quarter / an eighth as long.  Per-launch traffic scales by the table count.
    "prof": Workload("prof", T=16, E=1_000_000, D=128, B=2048, dtype="fp16", L=38, optimizer="sgd", lr=0.05),
    "prof_cfg3": Workload("prof_cfg3", T=8, E=1_000_000, D=128, B=2048, dtype="fp32", pooling="mean",
                          optimizer="exact_rowwise_adagrad", lr=0.01, eps=1e-8, L_dist="poisson", L_mean=20.0,
                          L_min=1, L_max=100, index_dist="zipf", zipf_alpha=1.05),
    "prof_cfg5": Workload("prof_cfg5", T=8, E=1_000_000, D=128, B=65_536, dtype="fp16", L=32, optimizer="sgd", lr=0.05),
    # the headline target: cfg2's shapes with forward + backward + fused exact SGD
    "target": Workload("target", T=64, E=1_000_000, D=128, B=2048, dtype="fp16", L=38, optimizer="sgd", lr=0.05),
}


def bag_lengths(w, rng, T=None, B=None):
    T = w.T if T is None else T
    B = w.B if B is None else B
    if w.L_dist == "fixed":
        return np.full((T, B), w.L, dtype=np.int64)
    if w.L_dist == "poisson":
        return np.clip(rng.poisson(w.L_mean, size=(T, B)), w.L_min, w.L_max).astype(np.int64)
    raise ValueError("unknown length distribution %r" % w.L_dist)


def draw_indices(w, rng, n, E=None):
    E = w.E if E is None else E
    if w.index_dist == "uniform":
        return rng.integers(0, E, size=n, dtype=np.int64).astype(np.int32)
    if w.index_dist == "zipf":
        # folded into [0, E) in int64, as table_batched_embeddings_benchmark.py:133-136 folds with % E
        return (rng.zipf(w.zipf_alpha, size=n).astype(np.int64) % E).astype(np.int32)
    raise ValueError("unknown index distribution %r" % w.index_dist)


def make_inputs(w, seed=None, T=None, B=None, E=None):
    """(indices int32 [N], offsets int32 [T*B+1]) for workload ``w``; T/B/E override its sizes."""
    rng = np.random.default_rng(w.seed if seed is None else seed)
    lengths = bag_lengths(w, rng, T, B)
    offsets = np.concatenate([[0], np.cumsum(lengths.reshape(-1))])
    assert offsets[-1] < 2 ** 31 - 1, "N exceeds int32 offsets"
    indices = draw_indices(w, rng, int(offsets[-1]), E)
    return indices, offsets.astype(np.int32)


def make_weights(w, seed=None, T=None, E=None):
    """float32 numpy weights [T*E, D] ~ U(-0.01, 0.01); cast to the table dtype by the caller."""
    rng = np.random.default_rng((w.seed if seed is None else seed) + 1)
    T = w.T if T is None else T
    E = w.E if E is None else E
    return rng.uniform(-0.01, 0.01, size=(T * E, w.D)).astype(np.float32)


def make_grad(w, seed=None, T=None, B=None):
    rng = np.random.default_rng((w.seed if seed is None else seed) + 2)
    T = w.T if T is None else T
    B = w.B if B is None else B
    return rng.standard_normal(size=(B, T, w.D), dtype=np.float32)


def count_unique_rows(indices, offsets, T, B, E):
    """U = distinct (table,row) pairs of a batch."""
    lengths = np.diff(offsets.astype(np.int64))
    table_of_pos = np.repeat(np.arange(T * B, dtype=np.int64) // B, lengths)
    return int(np.unique(table_of_pos * E + indices.astype(np.int64)).size)


def algorithmic_bytes(w, N, U, nbags, backward=None):
    """Bytes one step must move between HBM and the SMs at minimum: every distinct row read once
    (and written once by the optimizer), pooled outputs written, gradients read, indices and
    offsets read once per pass, rowwise state read+written.  Sort scratch is overhead, not counted."""
    s = w.elem_bytes
    row = w.D * s
    idx = 4 * N + 4 * (nbags + 1)
    fwd = U * row + nbags * row + idx
    if backward is None:
        backward = w.optimizer != "none"
    if not backward:
        return {"fwd": fwd, "bwd": 0, "step": fwd}
    bwd = 2 * U * row + nbags * row + idx + (8 * U if w.optimizer == "exact_rowwise_adagrad" else 0)
    return {"fwd": fwd, "bwd": bwd, "step": fwd + bwd}


def lookup_bytes(w, N, backward=None):
    """The reference's own bandwidth convention: elem*N*D forward, 2*elem*N*D backward
    (table_batched_embeddings_benchmark.py:240,356)."""
    if backward is None:
        backward = w.optimizer != "none"
    f = w.elem_bytes * N * w.D
    return f + (2 * f if backward else 0)
