"""Pins the CPU oracle to outputs of the reference's own CUDA kernels.

``tests/golden/reference_*.npz`` were written by ``tests/golden/make_reference_golden.py``, which
calls the reference's ``table_batched_embeddings`` extension (built from its unmodified kernels by
``oracle/build_ref.py``) on a B200.  Every stored output is compared here with the oracle's answer on
the stored inputs: forward (sum, per-sample weights), SGD, exact and approximate rowwise Adagrad
(weights, optimizer state, per-sample-weight gradient), the mixed-width variants and
``construct_offsets``.  Tolerances are the north-star ones: integers exact, fp32 1e-5, fp16 1e-2.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TOL = {"fp32": dict(rtol=1e-5, atol=1e-5), "fp16": dict(rtol=1e-2, atol=1e-2)}
CASES = sorted(os.path.basename(p)[len("reference_"):-4] for p in glob.glob(os.path.join(GOLDEN, "reference_*.npz")))
LOOKUP_CASES = [c for c in CASES if c not in ("mixed_exact_fp32", "construct_offsets")]


def load_reference_case(name):
    """The stored case with tensors rebuilt in the table dtype; config-1 sized cases regenerate their
    weights from the stored seed and their constant optimizer state."""
    z = dict(np.load(os.path.join(GOLDEN, "reference_%s.npz" % name)))
    dtype = str(z["dtype"])
    tdt = torch.float16 if dtype == "fp16" else torch.float32
    T, E, D = int(z["T"]), int(z["E"]), int(z["D"])
    if "weights" not in z:
        z["weights"] = np.random.default_rng(int(z["weights_seed"])).uniform(-0.01, 0.01, size=(T * E, D)).astype(np.float32)
        z["state"] = np.full(T * E, float(z["state_constant"]), dtype=np.float32)
    c = dict(z)
    c.update(T=T, E=E, D=D, B=int(z["B"]), dtype=dtype, tdt=tdt, optimizer=str(z["optimizer"]), weighted=bool(z["weighted"]),
             lr=float(z["lr"]), eps=float(z["eps"]),
             weights_t=torch.from_numpy(z["weights"]).to(tdt), grad_t=torch.from_numpy(z["grad"]).to(tdt),
             psw_t=torch.from_numpy(z["psw"]).to(tdt) if "psw" in z else None,
             state_t=torch.from_numpy(z["state"]), table_offsets_l=[int(x) for x in z["table_offsets"]])
    return c


def expected_after(c):
    """(weights_after, state_after) of the reference for every row, or for the stored sample."""
    if "weights_after" in c:
        return torch.from_numpy(c["weights_after"]), torch.from_numpy(c["state_after"]), None
    rows = torch.from_numpy(c["sample_rows"])
    return torch.from_numpy(c["weights_after_sample"]), torch.from_numpy(c["state_after_sample"]), rows


def test_reference_vectors_are_present():
    assert len(LOOKUP_CASES) >= 11 and "mixed_exact_fp32" in CASES and "construct_offsets" in CASES


@pytest.mark.parametrize("name", LOOKUP_CASES)
def test_oracle_forward_matches_reference_kernel(name):
    c = load_reference_case(name)
    out = oracle.forward(c["weights_t"], c["table_offsets_l"], c["indices"], c["offsets"],
                         c["psw_t"] if c["weighted"] else None, "sum", compute_dtype=torch.float32)
    torch.testing.assert_close(out.float(), torch.from_numpy(c["out"]), **TOL[c["dtype"]])


@pytest.mark.parametrize("name", [c for c in LOOKUP_CASES if "sgd" in c or "exact" in c or "approx" in c])
def test_oracle_optimizer_step_matches_reference_kernel(name):
    c = load_reference_case(name)
    args = (c["table_offsets_l"], c["indices"], c["offsets"], c["grad_t"])
    gpsw = None
    if c["optimizer"] == "sgd":
        w = oracle.sgd_step(c["weights_t"], *args, c["lr"], compute_dtype=torch.float32)
        s = c["state_t"]
    elif c["optimizer"] == "exact_rowwise_adagrad":
        w, s = oracle.exact_rowwise_adagrad_step(c["weights_t"], c["state_t"], *args, c["lr"], c["eps"])
    else:
        w, s, gpsw = oracle.approx_rowwise_adagrad_step(c["weights_t"], c["state_t"], *args, c["lr"], c["eps"],
                                                         c["psw_t"] if c["weighted"] else None)
    ref_w, ref_s, rows = expected_after(c)
    if rows is not None:
        # whole-table float64 sums cover the rows outside the sample
        np.testing.assert_allclose(w.double().view(c["T"], -1).sum(1).numpy(), c["weights_after_table_sums"], rtol=1e-6)
        np.testing.assert_allclose(s.double().view(c["T"], -1).sum(1).numpy(), c["state_after_table_sums"], rtol=1e-6)
        w, s = w[rows], s[rows]
    torch.testing.assert_close(w.float(), ref_w, **TOL[c["dtype"]])
    torch.testing.assert_close(s.float(), ref_s, rtol=1e-5, atol=1e-5)
    if c["optimizer"] == "sgd":
        assert torch.equal(s, ref_s)  # SGD leaves the state alone
    if "grad_psw" in c:
        torch.testing.assert_close(gpsw.float(), torch.from_numpy(c["grad_psw"]), **TOL[c["dtype"]])


def test_reference_touches_only_looked_up_rows():
    c = load_reference_case("exact_fp32_repeats")
    rows, _, starts = oracle.sort_segments(c["table_offsets_l"], c["indices"], c["offsets"])
    touched = np.zeros(c["T"] * c["E"], dtype=bool)
    touched[rows[starts]] = True
    changed = (c["weights_after"] != c["weights"]).any(axis=1)
    assert not (changed & ~touched).any() and changed[touched].all()
    assert np.array_equal(c["state_after"][~touched], c["state"][~touched])


def test_oracle_construct_offsets_matches_reference_kernel():
    z = np.load(os.path.join(GOLDEN, "reference_construct_offsets.npz"))
    assert np.array_equal(oracle.construct_offsets(z["begin"], z["totals"]), z["lengths_out"])


def mixed_tables(z):
    """Per-table (weights [E, D], state [E], indices, offsets, grad [B, 1, D], column range) views of
    a stored mixed-width case (layout of MixedDimTableBatchedEmbeddingBags,
    table_batched_embeddings_ops.py:324-434)."""
    B = int(z["B"])
    elems, rows, cols = z["table_offsets"], z["table_dim_offsets"], z["dim_offsets"]
    out = []
    for t, (E, D) in enumerate(z["shapes"]):
        lo, hi = int(z["offsets"][t * B]), int(z["offsets"][(t + 1) * B])
        out.append(dict(E=int(E), D=int(D), lo=lo, hi=hi, c0=int(cols[t]), c1=int(cols[t + 1]),
                        e0=int(elems[t]), e1=int(elems[t + 1]), r0=int(rows[t]), r1=int(rows[t + 1]),
                        indices=z["indices"][lo:hi], offsets=(z["offsets"][t * B:(t + 1) * B + 1] - lo).astype(np.int32)))
    return out, B


def test_oracle_mixed_width_matches_reference_kernel():
    z = np.load(os.path.join(GOLDEN, "reference_mixed_exact_fp32.npz"))
    tables, B = mixed_tables(z)
    lr, eps = float(z["lr"]), float(z["eps"])
    for tb in tables:
        w = torch.from_numpy(z["weights"][tb["e0"]:tb["e1"]]).view(tb["E"], tb["D"])
        s = torch.from_numpy(z["state"][tb["r0"]:tb["r1"]])
        g = torch.from_numpy(z["grad"][:, tb["c0"]:tb["c1"]]).reshape(B, 1, tb["D"])
        out = oracle.forward(w, [0], tb["indices"], tb["offsets"])
        torch.testing.assert_close(out.view(B, tb["D"]), torch.from_numpy(z["out"][:, tb["c0"]:tb["c1"]]), **TOL["fp32"])
        w2, s2 = oracle.exact_rowwise_adagrad_step(w, s, [0], tb["indices"], tb["offsets"], g, lr, eps)
        torch.testing.assert_close(w2.reshape(-1), torch.from_numpy(z["weights_after"][tb["e0"]:tb["e1"]]), **TOL["fp32"])
        torch.testing.assert_close(s2, torch.from_numpy(z["state_after"][tb["r0"]:tb["r1"]]), rtol=1e-5, atol=1e-5)
