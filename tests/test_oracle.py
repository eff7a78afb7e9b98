"""The CPU oracle against hand computation, its own golden fixtures and algebraic properties."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import workloads

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _naive_forward(weights, table_offsets, indices, offsets, psw, pooling):
    T = len(table_offsets)
    B = (len(offsets) - 1) // T
    out = np.zeros((B, T, weights.shape[1]), dtype=np.float64)
    for t in range(T):
        for b in range(B):
            s, e = offsets[t * B + b], offsets[t * B + b + 1]
            for p in range(s, e):
                w = 1.0 if psw is None else psw[p]
                out[b, t] += w * weights[table_offsets[t] + indices[p]].astype(np.float64)
            if pooling == "mean" and e > s:
                out[b, t] /= (e - s)
    return out


def _naive_dense_grad(shape, table_offsets, indices, offsets, grad, pooling):
    T = len(table_offsets)
    B = (len(offsets) - 1) // T
    g = np.zeros(shape, dtype=np.float64)
    for t in range(T):
        for b in range(B):
            s, e = offsets[t * B + b], offsets[t * B + b + 1]
            for p in range(s, e):
                scale = 1.0 / (e - s) if pooling == "mean" else 1.0
                g[table_offsets[t] + indices[p]] += scale * grad[b, t].astype(np.float64)
    return g


@pytest.mark.parametrize("name", sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "tiny_*.npz"))))
def test_tiny_golden_matches_naive_loops(name):
    """Every stored tiny vector equals a triple-loop float64 restatement of the formulas the
    reference's tests check (forward sum; w - lr*grad; state = sum_d grad^2, addcdiv)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    T, E = int(z["T"]), int(z["E"])
    table_offsets = [t * E for t in range(T)]
    fp16 = str(z["dtype"]) == "fp16"
    tol = dict(rtol=1e-2, atol=1e-2) if fp16 else dict(rtol=1e-5, atol=1e-6)
    psw = z["psw"] if "psw" in z.files else None
    pooling, opt = str(z["pooling"]), str(z["optimizer"])
    out = _naive_forward(z["weights"], table_offsets, z["indices"], z["offsets"], psw, pooling)
    np.testing.assert_allclose(z["out"], out, **tol)
    lr, eps = float(z["lr"]), float(z["eps"])
    if opt == "sgd":
        g = _naive_dense_grad(z["weights"].shape, table_offsets, z["indices"], z["offsets"], z["grad"], pooling)
        np.testing.assert_allclose(z["weights_after"], z["weights"] - lr * g, **tol)
    elif opt == "exact_rowwise_adagrad":
        g = _naive_dense_grad(z["weights"].shape, table_offsets, z["indices"], z["offsets"], z["grad"], pooling)
        state = z["state0"] + (g ** 2).sum(axis=1)
        np.testing.assert_allclose(z["state_after"], state, rtol=1e-3 if fp16 else 1e-5)
        np.testing.assert_allclose(z["weights_after"], z["weights"] - lr * g / (np.sqrt(state) + eps)[:, None], **tol)
    # the bookkeeping
    rows, bags, starts = z["sorted_rows"], z["sorted_bags"], z["segment_starts"]
    assert np.all(np.diff(rows) >= 0)
    assert len(starts) == len(np.unique(rows))
    B = int(z["B"])
    for i in range(len(rows)):
        t = bags[i] // B
        s, e = z["offsets"][bags[i]], z["offsets"][bags[i] + 1]
        assert (rows[i] - table_offsets[t]) in z["indices"][s:e]


def test_oracle_reproduces_golden_files():
    """Regenerating from the stored inputs gives the stored outputs bit for bit."""
    z = np.load(os.path.join(GOLDEN, "tiny_fp32_sum_sgd.npz"))
    T, E = int(z["T"]), int(z["E"])
    table_offsets = [t * E for t in range(T)]
    w = torch.from_numpy(z["weights"])
    out = oracle.forward(w, table_offsets, z["indices"], z["offsets"], compute_dtype=torch.float32)
    assert np.array_equal(out.numpy(), z["out"])
    w1 = oracle.sgd_step(w, table_offsets, z["indices"], z["offsets"], torch.from_numpy(z["grad"]), float(z["lr"]),
                         compute_dtype=torch.float32)
    assert np.array_equal(w1.numpy(), z["weights_after"])


def test_cfg1_golden():
    """Config 1 (T=4, E=10000, D=64 fp32, B=128, L=10, SGD lr=0.1, seed 0) regenerated from its seed."""
    z = np.load(os.path.join(GOLDEN, "cfg1.npz"))
    w = workloads.WORKLOADS["cfg1"]
    indices, offsets = workloads.make_inputs(w)
    assert np.array_equal(indices[:64], z["indices_head"])
    assert len(indices) == int(z["N"]) == w.T * w.B * w.L
    weights = torch.from_numpy(workloads.make_weights(w))
    grad = torch.from_numpy(workloads.make_grad(w))
    table_offsets = [t * w.E for t in range(w.T)]
    out = oracle.forward(weights, table_offsets, indices, offsets)
    np.testing.assert_allclose(out.numpy(), z["out"], rtol=1e-6, atol=1e-7)
    w1 = oracle.sgd_step(weights, table_offsets, indices, offsets, grad, w.lr)
    np.testing.assert_allclose(w1.double().view(w.T, -1).sum(dim=1).numpy(), z["weights_sum"], rtol=1e-9)
    np.testing.assert_allclose(w1[torch.from_numpy(z["sample_rows"])].numpy(), z["sample_values"], rtol=1e-6)
    rows, _, starts = oracle.sort_segments(table_offsets, indices, offsets)
    assert len(starts) == int(z["num_unique"]) == workloads.count_unique_rows(indices, offsets, w.T, w.B, w.E)
    assert np.array_equal(rows[:256], z["sorted_rows_head"])
    # repeated rows exist, so the duplicate-summing path is exercised
    assert len(starts) < len(indices)


def test_forward_is_linear_in_weights():
    rng = np.random.default_rng(0)
    T, E, D, B = 3, 20, 8, 6
    lengths = rng.integers(0, 5, size=(T, B))
    offsets = oracle.offsets_from_lengths(lengths)
    indices = rng.integers(0, E, size=int(offsets[-1])).astype(np.int32)
    to = [t * E for t in range(T)]
    a = torch.from_numpy(rng.standard_normal((T * E, D)))
    b = torch.from_numpy(rng.standard_normal((T * E, D)))
    for mode in ("sum", "mean"):
        fa = oracle.forward(a, to, indices, offsets, pooling_mode=mode)
        fb = oracle.forward(b, to, indices, offsets, pooling_mode=mode)
        fab = oracle.forward(2 * a - 3 * b, to, indices, offsets, pooling_mode=mode)
        torch.testing.assert_close(fab, 2 * fa - 3 * fb, rtol=1e-10, atol=1e-10)


def test_empty_bags_pool_to_zero():
    to = [0, 4]
    weights = torch.ones(8, 4)
    offsets = np.array([0, 0, 2, 2, 2], dtype=np.int32)  # T=2, B=2: bags (0,0) and (1,*) are empty
    indices = np.array([1, 3], dtype=np.int32)
    for mode in ("sum", "mean"):
        out = oracle.forward(weights, to, indices, offsets, pooling_mode=mode)
        assert out.shape == (2, 2, 4)
        assert torch.all(out[0, 0] == 0) and torch.all(out[:, 1] == 0)
        assert torch.all(out[1, 0] == (2.0 if mode == "sum" else 1.0))


def test_construct_offsets_matches_reference_test_contract():
    """Bag extents after cumsum equal the per-table extents (test_table_batched_embeddings.py:94-105)."""
    rng = np.random.default_rng(3)
    T, B = 5, 7
    Ls = rng.integers(1, 9, size=(T, B))
    begin = np.concatenate([np.zeros((T, 1), dtype=np.int64), np.cumsum(Ls, axis=1)[:, :-1]], axis=1)
    totals = Ls.sum(axis=1)
    fused = np.cumsum(oracle.construct_offsets(begin, totals))
    assert fused[0] == 0 and len(fused) == T * B + 1
    for t in range(T):
        for b in range(B):
            assert fused[t * B + b + 1] - fused[t * B + b] == Ls[t, b]


def test_all_to_all_layout_and_inverse():
    """out_j[b', r*T/W + t] = in_r[j*B/W + b', t] (sparse_embedding_cuda.cpp:475-487,531-532), and the
    backward exchange is its inverse."""
    W, B, Tl, D = 4, 8, 3, 2
    ins = [torch.arange(B * Tl * D, dtype=torch.float32).view(B, Tl, D) + 1000 * r for r in range(W)]
    outs = oracle.all_to_all_pooled(ins)
    Bl = B // W
    for j in range(W):
        assert outs[j].shape == (Bl, Tl * W, D)
        for r in range(W):
            for bp in range(Bl):
                for t in range(Tl):
                    assert torch.equal(outs[j][bp, r * Tl + t], ins[r][j * Bl + bp, t])
    # the reference's own formulation: view [W][B/W][T/W][D], exchange chunk r, transpose(1,0), view
    for j in range(W):
        recv = torch.stack([ins[r].view(W, Bl, Tl, D)[j] for r in range(W)])  # [W][Bl][Tl][D]
        assert torch.equal(recv.transpose(1, 0).contiguous().view(Bl, Tl * W, D), outs[j])
    back = oracle.all_to_all_pooled_backward(outs)
    for r in range(W):
        assert torch.equal(back[r], ins[r])


def test_approx_equals_exact_formula_without_repeats():
    """With no repeated row and zero initial state the approximate optimizer's state is |grad_bag|^2
    per looked-up row (table_batched_embeddings_cuda.cu:669-689)."""
    rng = np.random.default_rng(5)
    T, E, D, B, L = 2, 64, 8, 4, 3
    idx = np.stack([rng.permutation(E)[:B * L].reshape(B, L) for _ in range(T)])
    indices, offsets = oracle.get_table_batched_offsets_from_dense(idx)
    to = [0, E]
    w = torch.from_numpy(rng.standard_normal((T * E, D)).astype(np.float32))
    go = torch.from_numpy(rng.standard_normal((B, T, D)).astype(np.float32))
    w1, s1, _ = oracle.approx_rowwise_adagrad_step(w, torch.zeros(T * E), to, indices, offsets, go, 0.5, 0.2)
    grads, _ = oracle.dense_gradients(w, to, indices, offsets, go)
    for t in range(T):
        g = grads[t]
        s = s1[t * E:(t + 1) * E]
        torch.testing.assert_close(s, g.pow(2).sum(dim=1), rtol=1e-5, atol=1e-6)
        expect = torch.addcdiv(w[t * E:(t + 1) * E], g, s.sqrt().add(0.2).view(-1, 1), value=-0.5)
        torch.testing.assert_close(w1[t * E:(t + 1) * E], expect, rtol=1e-5, atol=1e-6)


def test_lxu_cache_model_by_hand():
    """2 sets x 2 ways, LRU: hits refresh, misses take empty ways first, then the least recently
    used way; a set whose ways were all used in the step leaves further rows uncached."""
    m = oracle.LXUCacheModel(num_sets=2, ways=2, policy="lru")
    to = [0]
    # rows by set, each list in ascending mixed-id order (the model's claim order)
    in_set = {0: [], 1: []}
    for r in sorted(range(64), key=m.mix):
        in_set[m.set_of(r)].append(r)
    a, b, c, d, e = in_set[0][:5]
    z = in_set[1][0]

    def step(model, rows):
        idx = np.asarray(rows, dtype=np.int32)
        off = np.asarray([0, len(rows)], dtype=np.int32)
        return model.step(to, idx, off)

    loc, st = step(m, [a, b, z])               # set 0: a, b -> ways 0, 1; set 1: z -> way 0
    assert loc.tolist() == [0, 1, 2] and st["fetched"] == 3 and st["hit_lookups"] == 0
    loc, st = step(m, [b, b, c])               # b hits (twice); c evicts a (older)
    assert loc.tolist() == [1, 1, 0] and st["hit_lookups"] == 2 and st["hit_rows"] == 1 and st["fetched"] == 1
    assert m.tags.tolist() == [c, b, z, -1]
    loc, st = step(m, [a, d, e])               # three misses, two ways (both last used at step 2: tie -> way 0
    assert st["uncached"] == 1                 # first); the last one in claim order finds no free way
    assert m.tags[:2].tolist() == [a, d] and loc.tolist() == [0, 1, -1]
    lfu = oracle.LXUCacheModel(num_sets=1, ways=2, policy="lfu")
    for rows in ([1, 2], [1], [1], [2]):
        step(lfu, rows)
    step(lfu, [3])
    assert sorted(lfu.tags.tolist()) == [1, 3]  # row 2 (2 uses) goes, row 1 (3 uses) stays although 2 was used later
