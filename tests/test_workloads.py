"""Workload generators: determinism, shapes and the roofline byte count."""
import numpy as np

from sparse_ads_baselines_b200 import workloads as W


def test_inputs_are_seeded_and_well_formed():
    w = W.WORKLOADS["cfg1"]
    i1, o1 = W.make_inputs(w)
    i2, o2 = W.make_inputs(w)
    assert np.array_equal(i1, i2) and np.array_equal(o1, o2)
    assert i1.dtype == np.int32 and o1.dtype == np.int32
    assert len(o1) == w.T * w.B + 1 and o1[0] == 0 and o1[-1] == len(i1) == w.T * w.B * w.L
    assert i1.min() >= 0 and i1.max() < w.E


def test_cfg3_lengths_and_zipf_skew():
    w = W.WORKLOADS["cfg3"]
    idx, off = W.make_inputs(w, T=2, B=512)
    L = np.diff(off)
    assert L.min() >= 1 and L.max() <= 100 and 18 < L.mean() < 22
    assert idx.min() >= 0 and idx.max() < w.E
    U = W.count_unique_rows(idx, off, 2, 512, w.E)
    assert U < 0.9 * len(idx)  # rows repeat heavily


def test_algorithmic_bytes_matches_hand_count():
    w = W.WORKLOADS["target"]
    N, U, bags = 4_980_736, 4_789_000, 64 * 2048
    b = W.algorithmic_bytes(w, N, U, bags)
    row = 128 * 2
    idx = 4 * N + 4 * (bags + 1)
    assert b["fwd"] == U * row + bags * row + idx
    assert b["bwd"] == 2 * U * row + bags * row + idx
    assert b["step"] == b["fwd"] + b["bwd"]
    assert W.lookup_bytes(w, N) == 3 * 2 * N * 128
    a = W.algorithmic_bytes(W.WORKLOADS["cfg3"], 100, 60, 10)
    assert a["bwd"] == 2 * 60 * 512 + 10 * 512 + 4 * 100 + 4 * 11 + 8 * 60
