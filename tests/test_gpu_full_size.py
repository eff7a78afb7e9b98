"""The benchmark configurations at their own sizes, through size-independent properties.

The CPU oracle cannot replay 10^6..10^8 lookups over tens of gigabytes of tables in a test, so
these cases check what does not need it: the table-segmented plan equals the device radix sort's
(exact integers), the device's run count equals an independent unique count, only looked-up rows
change, sampled bags and sampled runs (the longest ones included) equal an independent fp64
recomputation from the inputs, and an lr / -lr round trip restores the table.
  config 3: T=64, E=1M, D=128 fp32, B=2048, Poisson(20) lengths in [1,100], Zipf(1.05) rows, mean
            pooling, exact rowwise Adagrad -- hot rows with thousands of lookups, oversize buckets.
  config 5 (one rank's share at 8 ranks): T=64, E=1M, D=128 fp16, B=65,536, L=32 -- 134 M lookups,
            two per row: the wide sort variants and 32-bit position arithmetic near its range.
  config 4 (rows per table and cache rows scaled by 0.05): LXU cache transparency at B=4096, L=20,
            Zipf(1.2).
"""
import numpy as np
import pytest
import torch

from sparse_ads_baselines_b200 import table_batched_embeddings as tbe
from sparse_ads_baselines_b200 import table_batched_embeddings_ops as ops
from sparse_ads_baselines_b200 import workloads
from sparse_ads_baselines_b200.lxu_cache import LXUCachedEmbeddingBags

pytestmark = pytest.mark.gpu


def _fill_uniform(weights, T, E, gen, lo=-0.01, hi=0.01):
    for t in range(T):  # table by table: no full-size fp32 temporary
        block = weights[t * E:(t + 1) * E]
        block.copy_(torch.rand(block.shape, device=weights.device, generator=gen) * (hi - lo) + lo)


def _unique_rows_per_table(idx, off, T, B):
    """Distinct (table, row) pairs, counted table by table with torch.unique (an independent count)."""
    bounds = off[::B].cpu().tolist()
    return sum(int(torch.unique(idx[bounds[t]:bounds[t + 1]]).numel()) for t in range(T))


def _sample_runs(starts_c, n_total, rng, n_random, n_longest):
    lens = np.diff(np.concatenate([starts_c, [n_total]]))
    picks = list(rng.integers(0, len(starts_c), size=n_random)) + list(np.argsort(lens)[-n_longest:])
    return [(int(u), int(starts_c[u]), int(starts_c[u] + lens[u])) for u in picks], lens


def test_config3_full_size_properties(cuda_device):
    w = workloads.WORKLOADS["cfg3"]
    dev = cuda_device
    indices, offsets = workloads.make_inputs(w)
    N = indices.size
    gen = torch.Generator(device=dev).manual_seed(3)
    weights = torch.empty(w.T * w.E, w.D, dtype=torch.float32, device=dev)
    _fill_uniform(weights, w.T, w.E, gen)
    state = torch.rand(w.T * w.E, device=dev, generator=gen) * 1e-4
    grad = torch.randn(w.B, w.T, w.D, device=dev, generator=gen) * 0.01
    to = torch.arange(w.T, dtype=torch.int32, device=dev) * w.E
    idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)

    # plan: two-level sort (hot rows -> oversize buckets) == device radix sort, exactly
    rows, bags, starts = tbe.sort_segments(to, idx, off, w.T * w.E, max_rows_per_table=w.E)
    rows_r, bags_r, starts_r = tbe.sort_segments(to, idx, off, w.T * w.E)
    assert torch.equal(rows, rows_r) and torch.equal(bags, bags_r) and torch.equal(starts, starts_r)
    del rows_r, bags_r, starts_r
    assert starts.numel() == _unique_rows_per_table(idx, off, w.T, w.B)
    assert bool((rows[1:] >= rows[:-1]).all())

    # forward, mean pooling: sampled bags in fp64
    out = tbe.forward(weights, to, idx, off, None, 100, 2, False, pooling_mode="mean")
    rng = np.random.default_rng(1)
    for bag in rng.integers(0, w.T * w.B, size=48):
        t, b = divmod(int(bag), w.B)
        s, e = int(offsets[bag]), int(offsets[bag + 1])
        r = torch.from_numpy(indices[s:e].astype(np.int64)).to(dev) + t * w.E
        expect = weights[r].double().sum(0) / (e - s)
        torch.testing.assert_close(out[b, t].double(), expect, rtol=1e-5, atol=1e-7)

    before_w, before_s = weights.clone(), state.clone()
    tbe.backward_exact_adagrad(grad, weights, to, idx, off, None, state, w.lr, w.eps, False, 1, pooling_mode="mean")
    torch.cuda.synchronize()

    # only looked-up rows change, weights and state
    touched = torch.zeros(w.T * w.E, dtype=torch.bool, device=dev)
    touched[rows[starts.long()].long()] = True
    for t in range(w.T):
        sl = slice(t * w.E, (t + 1) * w.E)
        changed = (weights[sl] != before_w[sl]).any(dim=1) | (state[sl] != before_s[sl])
        assert not bool((changed & ~touched[sl]).any())

    # sampled runs (random ones + the longest, which take the queued CTA-per-run path) in fp64
    starts_c, rows_c, bags_c = starts.cpu().numpy(), rows.cpu().numpy(), bags.cpu().numpy()
    runs, lens = _sample_runs(starts_c, N, rng, 48, 24)
    assert lens.max() > 1000, "config 3's hottest row should see thousands of lookups"
    inv_len = 1.0 / np.diff(offsets.astype(np.int64))
    for (u, s, e) in runs:
        r = int(rows_c[s])
        bg = torch.from_numpy(bags_c[s:e].astype(np.int64)).to(dev)
        scale = torch.from_numpy(inv_len[bags_c[s:e]]).to(dev)
        G = (grad[bg % w.B, bg // w.B].double() * scale[:, None]).sum(0)
        st = before_s[r].double() + (G * G).sum()
        expect_w = before_w[r].double() - w.lr * G / (st.sqrt() + w.eps)
        # a run of thousands of cancelling fp32 terms summed in another order: 1e-4 on its squared norm
        torch.testing.assert_close(state[r].double(), st, rtol=1e-5 if e - s <= 64 else 1e-4, atol=1e-12)
        torch.testing.assert_close(weights[r].double(), expect_w, rtol=1e-5, atol=2e-7)


def test_config5_per_gpu_shapes_properties(cuda_device):
    w = workloads.WORKLOADS["cfg5"]
    dev = cuda_device
    rng = np.random.default_rng(5)
    N = w.T * w.B * w.L
    assert N == 134_217_728
    idx = torch.from_numpy(rng.integers(0, w.E, size=N, dtype=np.int64).astype(np.int32)).to(dev)
    off = (torch.arange(w.T * w.B + 1, dtype=torch.int64, device=dev) * w.L).to(torch.int32)
    gen = torch.Generator(device=dev).manual_seed(5)
    weights = torch.empty(w.T * w.E, w.D, dtype=torch.float16, device=dev)
    _fill_uniform(weights, w.T, w.E, gen)
    grad = (torch.randn(w.B, w.T, w.D, device=dev, generator=gen) * 0.01).half()
    to = torch.arange(w.T, dtype=torch.int32, device=dev) * w.E

    # the wide variants of the table-segmented sort (2.1 M lookups per 1 M-row table) == radix sort
    rows, bags, starts = tbe.sort_segments(to, idx, off, w.T * w.E, max_rows_per_table=w.E)
    rows_r, bags_r, starts_r = tbe.sort_segments(to, idx, off, w.T * w.E)
    assert torch.equal(rows, rows_r) and torch.equal(bags, bags_r) and torch.equal(starts, starts_r)
    del rows_r, bags_r, starts_r
    U = starts.numel()
    assert U == _unique_rows_per_table(idx, off, w.T, w.B)
    assert 0.40 < U / N < 0.44  # two lookups per row: U/N ~ 0.418 for uniform rows

    out = tbe.forward(weights, to, idx, off, None, 32, 2, False)
    for bag in rng.integers(0, w.T * w.B, size=48):
        t, b = divmod(int(bag), w.B)
        r = idx[bag * w.L:(bag + 1) * w.L].long() + t * w.E
        torch.testing.assert_close(out[b, t].float(), weights[r].float().sum(0), rtol=2e-3, atol=1e-4)
    del out

    before = weights.clone()
    tbe.backward_sgd(grad, weights, to, idx, off, w.lr, 32, 2, False)
    touched = torch.zeros(w.T * w.E, dtype=torch.bool, device=dev)
    touched[rows[starts.long()].long()] = True
    for t in range(w.T):
        sl = slice(t * w.E, (t + 1) * w.E)
        changed = (weights[sl] != before[sl]).any(dim=1)
        assert not bool((changed & ~touched[sl]).any())
    starts_c = starts.cpu().numpy()
    runs, _ = _sample_runs(starts_c, N, rng, 64, 8)
    for (u, s, e) in runs:
        r = int(rows[s])
        bg = bags[s:e].long()
        G = grad[bg % w.B, bg // w.B].float().sum(0)
        expect = (before[r].float() - w.lr * G).half()
        torch.testing.assert_close(weights[r].float(), expect.float(), rtol=2e-3, atol=1e-5)
    del rows, bags, starts, touched
    tbe.backward_sgd(grad, weights, to, idx, off, -w.lr, 32, 2, False)
    worst = 0.0
    for t in range(w.T):
        sl = slice(t * w.E, (t + 1) * w.E)
        worst = max(worst, (weights[sl].float() - before[sl].float()).abs().max().item())
    assert worst <= 2.0 ** -15


def test_config4_scaled_cache_is_transparent(cuda_device):
    """Config 4 with rows per table and cache rows scaled by 0.05 (4.1 GB of host-resident tables,
    100,000 cache rows, 4-way LRU): several fwd + SGD steps give the uncached device-resident module's
    outputs and table, lookups start to hit, and sampled bags equal a direct recomputation."""
    w = workloads.WORKLOADS["cfg4"]
    dev = cuda_device
    E, cache_rows = w.E // 20, 100_000
    cached = LXUCachedEmbeddingBags(w.T, E, w.D, cache_rows=cache_rows, ways=4, policy="lru", learning_rate=w.lr, fp16=True)
    plain = ops.TableBatchedEmbeddingBags(w.T, E, w.D, optimizer=ops.Optimizer.SGD, learning_rate=w.lr, fp16=True).to(dev)
    gen = torch.Generator(device=dev).manual_seed(4)
    _fill_uniform(plain.embedding_weights.data, w.T, E, gen)
    cached.embedding_weights.data.copy_(plain.embedding_weights.data)
    grad = (torch.randn(w.B, w.T, w.D, device=dev, generator=gen) * 0.01).half()
    rates = []
    rng = np.random.default_rng(0)
    for step in range(4):
        indices, offsets = workloads.make_inputs(w, seed=100 + step, E=E)
        idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
        out_c = cached(idx, off)
        out_p = plain(idx, off)
        torch.testing.assert_close(out_c.float(), out_p.detach().float(), rtol=1e-2, atol=1e-3)
        if step == 0:
            for bag in rng.integers(0, w.T * w.B, size=32):
                t, b = divmod(int(bag), w.B)
                r = idx[bag * w.L:(bag + 1) * w.L].long() + t * E
                torch.testing.assert_close(out_c[b, t].float(), plain.embedding_weights.data[r].float().sum(0),
                                           rtol=2e-3, atol=1e-4)
        out_c.backward(grad)
        out_p.backward(grad)
        rates.append(cached.last_stats())
    # 523 k distinct rows per batch against 100 k cache rows: the hot rows stay, a fifth of the lookups hit
    assert rates[0]["hit_rate"] == 0.0 and rates[-1]["hit_rate"] > 0.15 and rates[-1]["hit_rate"] >= rates[1]["hit_rate"], rates
    assert rates[-1]["fetched"] > 0 and rates[-1]["uncached"] > 0, rates  # evictions and overflowing sets both happen
    assert all(r["lookups"] == w.T * w.B * w.L for r in rates)
    table = cached.state_dict()["embedding_weights"]
    for t in range(w.T):
        sl = slice(t * E, (t + 1) * E)
        torch.testing.assert_close(table[sl].float(), plain.embedding_weights.data[sl].float(), rtol=1e-2, atol=1e-4)
