"""The LXU cache on the GPU: slot bookkeeping exactly equal to the CPU model, and transparency (the
cached module computes what the uncached module and the per-table EmbeddingBag oracle compute)."""
import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import table_batched_embeddings_ops as ops
from sparse_ads_baselines_b200.lxu_cache import LXUCachedEmbeddingBags

pytestmark = pytest.mark.gpu


def _batch(rng, T, E, B, Lmax, zipf=None):
    lengths = rng.integers(0, Lmax + 1, size=(T, B))
    offsets = oracle.offsets_from_lengths(lengths)
    n = int(offsets[-1])
    if zipf:
        idx = (rng.zipf(zipf, size=n).astype(np.int64) % E).astype(np.int32)
    else:
        idx = rng.integers(0, E, size=n).astype(np.int32)
    return idx, offsets


@pytest.mark.parametrize("policy", ["lru", "lfu"])
@pytest.mark.parametrize("ways", [1, 2, 4, 8])
def test_slot_bookkeeping_matches_cpu_model(cuda_device, policy, ways):
    """Tags, last-use steps, use counts, per-lookup locations and hit counters equal the CPU model
    exactly, step after step, with a cache small enough that sets overflow and rows stay uncached."""
    T, E, D, B, Lmax = 3, 40, 8, 6, 5
    cache_rows = 8 * ways
    m = LXUCachedEmbeddingBags(T, E, D, cache_rows=cache_rows, ways=ways, policy=policy, learning_rate=0.0)
    model = oracle.LXUCacheModel(cache_rows // ways, ways, policy)
    to = [t * E for t in range(T)]
    rng = np.random.default_rng(ways * 10 + (policy == "lfu"))
    saw_uncached = saw_eviction = False
    for step in range(8):
        idx, off = _batch(rng, T, E, B, Lmax, zipf=1.3 if step % 2 else None)
        m._prefetch(torch.from_numpy(idx).cuda(), torch.from_numpy(off).cuda())
        loc, stats = model.step(to, idx, off)
        assert np.array_equal(m._locations[:len(idx)].cpu().numpy(), loc), "locations, step %d" % step
        assert np.array_equal(m.tags.cpu().numpy(), model.tags), "tags, step %d" % step
        assert np.array_equal(m.last_use.cpu().numpy(), model.last_use), "last_use, step %d" % step
        assert np.array_equal(m.use_count.cpu().numpy(), model.use_count), "use_count, step %d" % step
        got = m.last_stats()
        for k in ("lookups", "rows", "fetched", "hit_lookups", "hit_rows", "uncached"):
            assert got[k] == stats[k], (k, got, stats)
        saw_uncached |= stats["uncached"] > 0
        saw_eviction |= step > 0 and stats["fetched"] > 0
    assert saw_eviction
    if ways <= 2:
        assert saw_uncached  # tiny associativity: some set overflowed


@pytest.mark.parametrize("fp16", [False, True])
@pytest.mark.parametrize("pooling", ["sum", "mean"])
@pytest.mark.parametrize("fill", ["direct", "deferred", "staged", "staged_rounds"])
def test_cached_module_is_transparent(cuda_device, fp16, pooling, fill):
    """Several fwd + SGD steps through a small cache (evictions, write-backs, uncached rows) give the
    outputs and the final table of the uncached device-resident module and of the oracle, whichever way
    the rows cross the host link: SM-issued loads and stores (direct, deferred write-backs) or staged
    copies with the host gathering and scattering rows (one round, or several rounds of 3 claims)."""
    T, E, D, B, Lmax, lr = 3, 60, 32, 8, 6, 0.05
    dtype = torch.float16 if fp16 else torch.float32
    torch.manual_seed(0)
    plain = ops.TableBatchedEmbeddingBags(T, E, D, optimizer=ops.Optimizer.SGD, learning_rate=lr, fp16=fp16,
                                          pooling_mode=pooling).cuda()
    plain.embedding_weights.data.uniform_(-1, 1)
    cached = LXUCachedEmbeddingBags(T, E, D, cache_rows=16, ways=4, policy="lru", learning_rate=lr, fp16=fp16,
                                    pooling_mode=pooling, deferred_writeback=fill == "deferred",
                                    staged_fill=fill.startswith("staged"), stage_rows=3 if fill == "staged_rounds" else 4096)
    cached.embedding_weights.data.copy_(plain.embedding_weights.data)
    w_ref = plain.embedding_weights.detach().cpu().clone()
    to = [t * E for t in range(T)]
    rng = np.random.default_rng(3)
    tol = dict(rtol=1e-2, atol=1e-2) if fp16 else dict(rtol=1e-5, atol=1e-5)
    for step in range(6):
        idx, off = _batch(rng, T, E, B, Lmax, zipf=1.2 if step % 2 else None)
        idx_d, off_d = torch.from_numpy(idx).cuda(), torch.from_numpy(off).cuda()
        go = torch.randn(B, T, D, device="cuda").to(dtype)
        out_p = plain(idx_d, off_d)
        out_c = cached(idx_d, off_d)
        ref = oracle.forward(w_ref, to, idx, off, None, pooling, compute_dtype=torch.float32)
        torch.testing.assert_close(out_c.float().cpu(), ref.float(), **tol)
        torch.testing.assert_close(out_c.float(), out_p.detach().float(), **tol)
        out_p.backward(go)
        out_c.backward(go)
        w_ref = oracle.sgd_step(w_ref, to, idx, off, go.cpu(), lr, pooling, compute_dtype=torch.float32)
    assert cached.dirty.any()
    sd = cached.state_dict()  # flushes the dirty rows
    assert not cached.dirty.any()
    torch.testing.assert_close(sd["embedding_weights"].float().cpu(), w_ref.float(), **tol)
    torch.testing.assert_close(sd["embedding_weights"].float().cpu(), plain.embedding_weights.detach().float().cpu(),
                               **tol)


@pytest.mark.parametrize("stage_rows", [131072, 5000])
def test_large_rounds_of_the_staged_fill(cuda_device, stage_rows):
    """Tens of thousands of misses per step: one large round of the staged fill (its gather handed to
    the copy engine in pieces), or several rounds with 5000 staging rows.  Three steps of lookups + SGD through a cache that keeps evicting must leave the
    table the plain device-resident module computes, bit for bit (fp32, same kernels' arithmetic)."""
    T, E, D, B, L, lr = 2, 100_000, 32, 2048, 8, 0.05
    torch.manual_seed(2)
    plain = ops.TableBatchedEmbeddingBags(T, E, D, optimizer=ops.Optimizer.SGD, learning_rate=lr).cuda()
    plain.embedding_weights.data.uniform_(-1, 1)
    cached = LXUCachedEmbeddingBags(T, E, D, cache_rows=32768, ways=4, policy="lru", learning_rate=lr,
                                    staged_fill=True, stage_rows=stage_rows)
    cached.embedding_weights.data.copy_(plain.embedding_weights.data)
    rng = np.random.default_rng(7)
    off = torch.from_numpy((np.arange(T * B + 1) * L).astype(np.int32)).cuda()
    for step in range(3):
        idx = torch.from_numpy(rng.integers(0, E, size=T * B * L).astype(np.int32)).cuda()
        go = torch.randn(B, T, D, device="cuda")
        out_p, out_c = plain(idx, off), cached(idx, off)
        torch.testing.assert_close(out_c, out_p.detach(), rtol=1e-5, atol=1e-5)
        assert cached.last_stats()["fetched"] > 8192
        out_p.backward(go)
        out_c.backward(go)
    sd = cached.state_dict()
    torch.testing.assert_close(sd["embedding_weights"].cpu(), plain.embedding_weights.detach().cpu(), rtol=1e-5, atol=1e-5)


def test_empty_batch_clears_every_counter(cuda_device):
    """A step without lookups after a step with uncached rows reports zeros in all five counters."""
    T, E, D, B = 2, 40, 8, 4
    m = LXUCachedEmbeddingBags(T, E, D, cache_rows=4, ways=1, policy="lru", learning_rate=0.0)
    rng = np.random.default_rng(1)
    idx, off = _batch(rng, T, E, B, 6)
    m(torch.from_numpy(idx).cuda(), torch.from_numpy(off).cuda())
    assert m.last_stats()["uncached"] > 0
    m(torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(T * B + 1, dtype=torch.int32, device="cuda"))
    got = m.last_stats()
    assert all(got[k] == 0 for k in ("lookups", "rows", "fetched", "hit_lookups", "hit_rows", "uncached")), got


def test_hit_rate_grows_with_reuse(cuda_device):
    """Zipf lookups through a cache larger than the hot set: after a few steps most lookups hit."""
    T, E, D, B, L = 4, 5000, 16, 64, 20
    m = LXUCachedEmbeddingBags(T, E, D, cache_rows=4096, ways=4, policy="lru", learning_rate=0.0)
    rng = np.random.default_rng(0)
    rates = []
    for step in range(6):
        idx = (rng.zipf(1.2, size=T * B * L).astype(np.int64) % E).astype(np.int32)
        off = (np.arange(T * B + 1) * L).astype(np.int32)
        m(torch.from_numpy(idx).cuda(), torch.from_numpy(off).cuda())
        rates.append(m.last_stats()["hit_rate"])
    assert rates[0] == 0.0 and rates[-1] > 0.5, rates


@pytest.mark.parametrize("B", [300, 4000])
@pytest.mark.parametrize("fp16,D", [(False, 32), (True, 128), (False, 260)])
def test_hot_rows_take_the_long_run_path(cuda_device, fp16, D, B):
    """A few rows receive hundreds of lookups each (more than the 64 a single warp handles): the
    CTA-per-run kernel must give the oracle's SGD update, deterministically.  With B = 4000 a row
    sees ~2,000 lookups and its run is cut into parts summed by several CTAs."""
    T, E, L, lr = 2, 6, 3, 0.01
    dtype = torch.float16 if fp16 else torch.float32
    cached = LXUCachedEmbeddingBags(T, E, D, cache_rows=8, ways=4, policy="lru", learning_rate=lr, fp16=fp16)
    torch.manual_seed(1)
    w0 = (torch.rand(T * E, D) * 2 - 1).to(dtype)
    rng = np.random.default_rng(5)
    idx = rng.integers(0, E, size=T * B * L).astype(np.int32)
    off = (np.arange(T * B + 1) * L).astype(np.int32)
    go = (torch.randn(B, T, D) * 0.05).to(dtype)
    results = []
    for _ in range(2):
        cached.embedding_weights.data.copy_(w0.cuda())
        cached.tags.fill_(-1)
        cached.dirty.zero_()
        out = cached(torch.from_numpy(idx).cuda(), torch.from_numpy(off).cuda())
        out.backward(go.cuda())
        results.append(cached.state_dict()["embedding_weights"].float().cpu().clone())
    ref = oracle.sgd_step(w0, [0, E], idx, off, go, lr, compute_dtype=torch.float32)
    tol = dict(rtol=1e-2, atol=1e-2) if fp16 else dict(rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(results[0], ref.float(), **tol)
    assert torch.equal(results[0], results[1])
