"""Mixed-D tables (per-table rows and width), after the reference's test_forward_mixed and
test_backward_adagrad_mixed (test_table_batched_embeddings.py:343-521): one EmbeddingBag per table."""
import numpy as np
import pytest
import torch

from sparse_ads_baselines_b200 import table_batched_embeddings_ops as ops

pytestmark = pytest.mark.gpu


def _setup(T, B, L, fp16, seed, optimizer, replace, dims=None):
    rs = np.random.RandomState(seed)
    dims = dims or [int(rs.randint(1, 40)) * 4 for _ in range(T)]
    rows = [int(rs.randint(60, 300)) for _ in range(T)]
    torch.manual_seed(seed)
    bs = [torch.nn.EmbeddingBag(E, D, mode="sum", sparse=True) for E, D in zip(rows, dims)]
    if fp16:
        bs = [b.half() for b in bs]
    xs = [torch.from_numpy(rs.choice(E, size=(B, L), replace=replace).astype(np.int64)) for E in rows]
    cc = ops.MixedDimTableBatchedEmbeddingBags(list(zip(rows, dims)), optimizer=optimizer, learning_rate=0.5, eps=0.2,
                                               fp16=fp16).cuda()
    for t, w in enumerate(cc.split_embedding_weights()):
        w.copy_(bs[t].weight.data.cuda())
    indices = torch.cat([x.reshape(-1) for x in xs]).int().cuda()          # flattened [T][B][L]
    offsets = (torch.arange(T * B + 1) * L).int().cuda()
    return dims, rows, bs, xs, cc, indices, offsets


@pytest.mark.parametrize("T,B,L", [(1, 1, 1), (3, 8, 5), (6, 33, 12)])
@pytest.mark.parametrize("fp16", [False, True])
@pytest.mark.parametrize("weighted", [False, True])
def test_forward_mixed(cuda_device, T, B, L, fp16, weighted):
    dims, rows, bs, xs, cc, indices, offsets = _setup(T, B, L, fp16, T * 7 + B, ops.Optimizer.APPROX_ROWWISE_ADAGRAD, True)
    xws = [torch.randn(B, L) for _ in range(T)]
    if fp16:
        xws = [w.half() for w in xws]
    fs = [b(x, per_sample_weights=xw) if weighted else b(x) for b, x, xw in zip(bs, xs, xws)]
    f = torch.cat(fs, dim=1)
    psw = torch.cat([w.reshape(-1) for w in xws]).cuda() if weighted else None
    out = cc(indices, offsets, psw)
    assert out.shape == (B, sum(dims))
    tol = dict(rtol=1e-2, atol=2e-2) if fp16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.detach().float().cpu(), f.detach().float(), **tol)
    for o, ref in zip(cc.split_output(out), fs):
        assert o.shape == ref.shape


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("fp16", [False, True])
@pytest.mark.parametrize("dims", [None, [32, 32, 32, 64, 16, 16, 128]])
def test_backward_adagrad_mixed(cuda_device, exact, fp16, dims):
    """``dims`` with runs of equal widths: consecutive tables of one width take one sort and one update
    launch together (different row counts per table inside the run)."""
    T, B, L = (len(dims), 9, 5) if dims else (4, 6, 4)
    opt = ops.Optimizer.EXACT_ROWWISE_ADAGRAD if exact else ops.Optimizer.APPROX_ROWWISE_ADAGRAD
    # exact: rows repeat; approximate: unique rows per table (the reference's racy kernel is only
    # defined there)
    dims, rows, bs, xs, cc, indices, offsets = _setup(T, B, L, fp16, 11, opt, replace=exact, dims=dims)
    fs = [b(x) for b, x in zip(bs, xs)]
    gos = [torch.randn_like(f) for f in fs]
    [f.backward(go) for f, go in zip(fs, gos)]
    out = cc(indices, offsets)
    out.backward(torch.cat(gos, dim=1).cuda())
    lr, eps = 0.5, 0.2
    tol = dict(rtol=1e-2, atol=1e-2) if fp16 else dict(rtol=1e-4, atol=1e-4)
    for t, (w, s) in enumerate(zip(cc.split_embedding_weights(), cc.split_optimizer_state())):
        dense = bs[t].weight.grad.float().to_dense()
        torch.testing.assert_close(s.cpu(), dense.pow(2).sum(dim=1), **tol)
        expect = torch.addcdiv(bs[t].weight.detach().float(), dense, s.cpu().sqrt().add(eps).view(-1, 1), value=-lr)
        torch.testing.assert_close(w.float().cpu(), expect, **tol)
