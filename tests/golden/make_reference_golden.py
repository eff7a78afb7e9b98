"""Generates ``reference_*.npz``: outputs of the REFERENCE's own CUDA kernels on seeded inputs.

    python oracle/build_ref.py                       # where the reference sources are present
    python tests/golden/make_reference_golden.py OUT_DIR   # on a machine with a CUDA device

``oracle/build_ref.py`` compiles the reference's ``table_batched_embeddings`` extension (its
unmodified kernels) into ``oracle/_ref/``; this script calls that extension's functions
(table_batched_embeddings.cpp:56-70) on small seeded cases and stores inputs and outputs in full.
The files pin the CPU oracle (tests/test_oracle.py) and are compared with this library's kernels
(tests/test_gpu_reference_golden.py); they are the only vectors here that the reference itself
produced.  Cases whose result the reference leaves to a race (SGD and approximate Adagrad on
repeated rows, table_batched_embeddings_cuda.cu:323,648-704) use duplicate-free indices, as the
reference's own tests do (test_table_batched_embeddings.py:177-182).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402


def seeded_table(seed, rows, D, lo=-0.01, hi=0.01):
    """Weights of the config-1 sized cases: regenerated from the seed instead of stored."""
    return np.random.default_rng(seed).uniform(lo, hi, size=(rows, D)).astype(np.float32)


def ragged_case(rng, T, E, D, B, Lmax, dtype, unique=False, fixed_L=None, empty=True, weights_seed=None):
    if fixed_L is not None:
        lengths = np.full((T, B), fixed_L, dtype=np.int64)
    else:
        lengths = rng.integers(0 if empty else 1, Lmax + 1, size=(T, B))
    offsets = np.concatenate([[0], np.cumsum(lengths.reshape(-1))]).astype(np.int32)
    N = int(offsets[-1])
    if unique:
        per_table = lengths.sum(axis=1)
        assert per_table.max() <= E
        indices = np.concatenate([rng.permutation(E)[:n] for n in per_table]).astype(np.int32)
    else:
        indices = rng.integers(0, E, size=N).astype(np.int32)
    tdt = torch.float16 if dtype == "fp16" else torch.float32
    if weights_seed is None:
        weights = torch.from_numpy(rng.uniform(-1, 1, size=(T * E, D)).astype(np.float32)).to(tdt)
    else:
        weights = torch.from_numpy(seeded_table(weights_seed, T * E, D)).to(tdt)
    grad = torch.from_numpy(rng.standard_normal(size=(B, T, D)).astype(np.float32)).to(tdt)
    psw = torch.from_numpy(rng.uniform(0.5, 1.5, size=N).astype(np.float32)).to(tdt)
    if weights_seed is None:
        state = rng.uniform(0.0, 0.5, size=T * E).astype(np.float32)
    else:
        state = np.full(T * E, 0.25, dtype=np.float32)
    return dict(state=state, T=T, E=E, D=D, B=B, Lmax=int(lengths.max()) if lengths.size else 0, dtype=dtype,
                indices=indices, offsets=offsets, weights=weights, grad=grad, psw=psw,
                table_offsets=np.arange(T, dtype=np.int32) * E)


def run_case(ref, c, optimizer, weighted, lr=0.05, eps=0.1, dev="cuda"):
    w = c["weights"].to(dev).clone()
    to = torch.from_numpy(c["table_offsets"]).to(dev)
    idx = torch.from_numpy(c["indices"]).to(dev)
    off = torch.from_numpy(c["offsets"]).to(dev)
    go = c["grad"].to(dev)
    psw = c["psw"].to(dev) if weighted else None
    L_max = max(c["Lmax"], 1)
    rec = dict(T=c["T"], E=c["E"], D=c["D"], B=c["B"], dtype=c["dtype"], optimizer=optimizer, weighted=int(weighted),
               lr=lr, eps=eps, indices=c["indices"], offsets=c["offsets"], table_offsets=c["table_offsets"],
               weights=c["weights"].float().numpy(), grad=c["grad"].float().numpy())
    if weighted:
        rec["psw"] = c["psw"].float().numpy()
    out = ref.forward(w, to, idx, off, psw, L_max, 1, False)
    out_shmem = ref.forward(w, to, idx, off, psw, L_max, 1, True)
    torch.cuda.synchronize()
    assert torch.equal(out, out_shmem), "the reference's two forward variants disagree"
    rec["out"] = out.float().cpu().numpy()
    state = torch.from_numpy(c["state"]).to(dev)
    rec["state"] = c["state"]
    gpsw = None
    if optimizer == "sgd":
        ref.backward_sgd(go, w, to, idx, off, lr, L_max, 1, False)
    elif optimizer == "exact_rowwise_adagrad":
        gpsw = ref.backward_exact_adagrad(go, w, to, idx, off, None, state, lr, eps, False, 1)
    elif optimizer == "approx_rowwise_adagrad":
        gpsw = ref.backward_approx_adagrad(go, w, to, idx, off, psw, state, lr, eps, L_max, False, 1)
    torch.cuda.synchronize()
    if optimizer != "none":
        rec["weights_after"] = w.float().cpu().numpy()
        rec["state_after"] = state.cpu().numpy()
    if gpsw is not None:
        rec["grad_psw"] = gpsw.float().cpu().numpy()
    return rec


def mixed_case(ref, rng, dev="cuda"):
    """forward_mixed_D + backward_exact_adagrad_mixed_D on three tables of different shape
    (table_batched_embeddings_ops.py:324-434 lays the flat vectors out like this)."""
    shapes = [(50, 8), (30, 16), (70, 4)]
    B, Lmax, lr, eps = 6, 5, 0.05, 0.1
    T = len(shapes)
    lengths = rng.integers(0, Lmax + 1, size=(T, B))
    offsets = np.concatenate([[0], np.cumsum(lengths.reshape(-1))]).astype(np.int32)
    indices = np.concatenate([rng.integers(0, shapes[t][0], size=int(lengths[t].sum())) for t in range(T)]).astype(np.int32)
    elems = np.concatenate([[0], np.cumsum([e * d for e, d in shapes])]).astype(np.int64)      # weights offsets
    rows = np.concatenate([[0], np.cumsum([e for e, _ in shapes])]).astype(np.int32)           # state offsets
    cols = np.concatenate([[0], np.cumsum([d for _, d in shapes])]).astype(np.int32)           # output columns
    total_D = int(cols[-1])
    weights = rng.uniform(-1, 1, size=int(elems[-1])).astype(np.float32)
    grad = rng.standard_normal(size=(B, total_D)).astype(np.float32)
    state0 = rng.uniform(0, 0.5, size=int(rows[-1])).astype(np.float32)
    w = torch.from_numpy(weights).to(dev)
    st = torch.from_numpy(state0).to(dev)
    to, tdo, do = (torch.from_numpy(x).to(dev) for x in (elems, rows, cols))
    idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
    out = ref.forward_mixed_D(w, to, do, total_D, idx, off, None, Lmax, 1, False)
    ref.backward_exact_adagrad_mixed_D(torch.from_numpy(grad).to(dev), w, to, tdo, do, total_D, idx, off, None, st, lr, eps,
                                       False, 1)
    torch.cuda.synchronize()
    return dict(shapes=np.array(shapes), B=B, lr=lr, eps=eps, indices=indices, offsets=offsets, table_offsets=elems,
                table_dim_offsets=rows, dim_offsets=cols, weights=weights, grad=grad, state=state0,
                out=out.cpu().numpy(), weights_after=w.cpu().numpy(), state_after=st.cpu().numpy())


def offsets_case(ref, rng, dev="cuda"):
    """construct_offsets (table_batched_embeddings_cuda.cu:1190-1213) on ragged per-table CSR begins."""
    T, B = 5, 9
    lengths = rng.integers(0, 7, size=(T, B))
    begin = np.concatenate([np.zeros((T, 1), dtype=np.int64), np.cumsum(lengths, axis=1)[:, :-1]], axis=1).astype(np.int32)
    totals = lengths.sum(axis=1).astype(np.int32)
    out = ref.construct_offsets(torch.from_numpy(begin).to(dev), torch.from_numpy(totals).to(dev))
    torch.cuda.synchronize()
    return dict(begin=begin, totals=totals, lengths_out=out.cpu().numpy())


def main(out_dir):
    ref = build_ref.load()
    os.makedirs(out_dir, exist_ok=True)
    rng = np.random.default_rng(20240607)
    cases = {
        # name: (case kwargs, optimizer, weighted)
        "fwd_fp32_ragged": (dict(T=3, E=40, D=36, B=7, Lmax=9, dtype="fp32"), "none", False),
        "fwd_fp16_ragged": (dict(T=3, E=40, D=64, B=7, Lmax=9, dtype="fp16"), "none", False),
        "fwd_fp32_weighted": (dict(T=2, E=30, D=20, B=5, Lmax=6, dtype="fp32"), "none", True),
        "sgd_fp32_unique": (dict(T=3, E=200, D=32, B=8, Lmax=6, dtype="fp32", unique=True), "sgd", False),
        "sgd_fp16_unique": (dict(T=2, E=200, D=128, B=8, Lmax=6, dtype="fp16", unique=True), "sgd", False),
        "exact_fp32_repeats": (dict(T=3, E=25, D=32, B=10, Lmax=8, dtype="fp32"), "exact_rowwise_adagrad", False),
        "exact_fp16_repeats": (dict(T=2, E=25, D=128, B=10, Lmax=8, dtype="fp16"), "exact_rowwise_adagrad", False),
        "approx_fp32_unique": (dict(T=3, E=200, D=32, B=8, Lmax=6, dtype="fp32", unique=True),
                               "approx_rowwise_adagrad", False),
        "approx_fp32_unique_weighted": (dict(T=2, E=200, D=16, B=8, Lmax=6, dtype="fp32", unique=True),
                                        "approx_rowwise_adagrad", True),
        # config 1's shapes (T=4, E=10,000, D=64 fp32, B=128, L=10, uniform indices with natural repeats)
        "cfg1_exact_fp32": (dict(T=4, E=10000, D=64, B=128, Lmax=10, dtype="fp32", fixed_L=10, weights_seed=11),
                            "exact_rowwise_adagrad", False),
        "cfg1_sgd_fp32_unique": (dict(T=4, E=10000, D=64, B=128, Lmax=10, dtype="fp32", fixed_L=10, unique=True,
                                      weights_seed=12), "sgd", False),
    }
    for name, (kw, optimizer, weighted) in cases.items():
        c = ragged_case(rng, **kw)
        rec = run_case(ref, c, optimizer, weighted)
        if name.startswith("cfg1"):
            # keep the file small: weights come back from their seed, the state was all rows' start
            # value; of the results keep a sample of the touched rows and float64 sums per table
            per_table = np.diff(c["offsets"]).reshape(c["T"], -1).sum(1)
            rows = np.unique(np.repeat(c["table_offsets"], per_table).astype(np.int64) + c["indices"])
            w_after, s_after = rec.pop("weights_after"), rec.pop("state_after")
            mask = np.ones(len(w_after), dtype=bool)
            mask[rows] = False
            assert np.array_equal(w_after[mask], rec["weights"][mask]), "the reference changed a row not looked up"
            assert np.array_equal(s_after[mask], rec["state"][mask])
            sample = rows[:: max(len(rows) // 400, 1)]
            rec.update(weights_seed=kw["weights_seed"], touched_rows=rows, sample_rows=sample,
                       weights_after_sample=w_after[sample], state_after_sample=s_after[sample],
                       weights_after_table_sums=w_after.astype(np.float64).reshape(c["T"], -1).sum(1),
                       state_after_table_sums=s_after.astype(np.float64).reshape(c["T"], -1).sum(1),
                       state_constant=np.float32(0.25))
            del rec["weights"], rec["state"]
        np.savez_compressed(os.path.join(out_dir, "reference_%s.npz" % name), **rec)
        print("wrote", name, {k: getattr(v, "shape", v) for k, v in rec.items() if k in ("out", "weights_after")})
    np.savez_compressed(os.path.join(out_dir, "reference_mixed_exact_fp32.npz"), **mixed_case(ref, rng))
    np.savez_compressed(os.path.join(out_dir, "reference_construct_offsets.npz"), **offsets_case(ref, rng))
    print("done")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
