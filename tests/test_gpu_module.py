"""The nn.Module / autograd surface, written after the reference's own tests
(test_table_batched_embeddings.py:115-340): a fused module against one EmbeddingBag per table."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings
import hypothesis.strategies as st

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import table_batched_embeddings_ops as ops

pytestmark = pytest.mark.gpu


def _bags(T, E, D, fp16, mode="sum"):
    torch.manual_seed(0)
    bs = [torch.nn.EmbeddingBag(E, D, mode=mode, sparse=True) for _ in range(T)]
    return [b.half() for b in bs] if fp16 else bs


def _fill(cc, bs, T, E, D):
    for t in range(T):
        cc.embedding_weights.data.view(T, E, D)[t, :, :] = bs[t].weight.data.to(cc.embedding_weights.device)


@given(st.integers(1, 4), st.integers(1, 64), st.integers(1, 32), st.integers(1, 32), st.booleans(), st.booleans())
@settings(deadline=None, max_examples=12, derandomize=True)
def test_forward(T, D, B, L, fp16, weighted):
    D = D * 4
    E = int(1e4)
    bs = _bags(T, E, D, fp16)
    xs = [torch.randint(low=0, high=E, size=(B, L)) for _ in range(T)]
    xws = [torch.randn(size=(B, L)) for _ in range(T)]
    if fp16:
        xws = [xw.half() for xw in xws]
    fs = ([b(x) for (b, x) in zip(bs, xs)] if not weighted
          else [b(x, per_sample_weights=xw) for (b, x, xw) in zip(bs, xs, xws)])
    f = torch.cat([f.view(B, 1, D) for f in fs], dim=1)
    cc = ops.TableBatchedEmbeddingBags(T, E, D, fp16=fp16).cuda()
    _fill(cc, bs, T, E, D)
    x = torch.cat([x.view(1, B, L) for x in xs], dim=0)
    xw = torch.cat([xw.view(1, B, L) for xw in xws], dim=0)
    indices, offsets = oracle.get_table_batched_offsets_from_dense(x.numpy())
    indices, offsets = torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda()
    fc2 = cc(indices, offsets) if not weighted else cc(indices, offsets, xw.contiguous().view(-1).cuda())
    tol = dict(rtol=1e-2, atol=1e-2) if fp16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(fc2.detach().cpu().float(), f.detach().float(), **tol)


@given(st.integers(1, 4), st.integers(1, 64), st.integers(1, 32), st.integers(1, 32), st.booleans(), st.booleans())
@settings(deadline=None, max_examples=12, derandomize=True)
def test_backward_sgd(T, D, B, L, fp16, repeats):
    D = D * 4
    E = int(1e4) if not repeats else 50
    bs = _bags(T, E, D, fp16)
    xs = [torch.from_numpy(np.random.RandomState(t).choice(E, size=(B, L), replace=repeats).astype(np.int64))
          for t in range(T)]
    fs = [b(x) for (b, x) in zip(bs, xs)]
    gos = [torch.randn_like(f) for f in fs]
    [f.backward(go) for (f, go) in zip(fs, gos)]
    lr = 0.05
    new_weights = [(b.weight.float() - b.weight.grad.float().to_dense() * lr) for b in bs]
    cc = ops.TableBatchedEmbeddingBags(T, E, D, optimizer=ops.Optimizer.SGD, learning_rate=lr, fp16=fp16).cuda()
    _fill(cc, bs, T, E, D)
    x = torch.cat([x.view(1, B, L) for x in xs], dim=0)
    indices, offsets = oracle.get_table_batched_offsets_from_dense(x.numpy())
    fc2 = cc(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda())
    fc2.backward(torch.cat([go.view(B, 1, D) for go in gos], dim=1).cuda())
    tol = dict(rtol=1e-2, atol=1e-2) if fp16 else dict(rtol=1e-5, atol=1e-5)
    for t in range(T):
        torch.testing.assert_close(cc.embedding_weights.detach().view(T, E, D)[t].cpu().float(),
                                   new_weights[t].detach(), **tol)
    g = cc.embedding_weights.grad
    assert g is not None and g.is_sparse and g._nnz() == 0  # the reference's empty sparse grad


@given(st.integers(1, 6), st.integers(1, 64), st.integers(1, 64), st.integers(1, 10), st.booleans(),
       st.sampled_from(["sum", "mean"]))
@settings(deadline=None, max_examples=12, derandomize=True)
def test_backward_exact_adagrad(T, D, B, L, fp16, mode):
    D = D * 4
    E = 100
    bs = _bags(T, E, D, fp16, mode)
    xs = [torch.from_numpy(np.random.RandomState(t).choice(E, size=(B, L), replace=True).astype(np.int64))
          for t in range(T)]
    fs = [b(x) for (b, x) in zip(bs, xs)]
    gos = [torch.randn_like(f) for f in fs]
    [f.backward(go) for (f, go) in zip(fs, gos)]
    lr, eps = 0.5, 0.2
    cc = ops.TableBatchedEmbeddingBags(T, E, D, optimizer=ops.Optimizer.EXACT_ROWWISE_ADAGRAD, learning_rate=lr,
                                       eps=eps, fp16=fp16, pooling_mode=mode).cuda()
    _fill(cc, bs, T, E, D)
    x = torch.cat([x.view(1, B, L) for x in xs], dim=0)
    indices, offsets = oracle.get_table_batched_offsets_from_dense(x.numpy())
    fc2 = cc(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda())
    fc2.backward(torch.cat([go.view(B, 1, D) for go in gos], dim=1).cuda())
    tol = dict(atol=1e-2, rtol=1e-2) if fp16 else dict(atol=1e-4, rtol=1e-4)
    for t in range(T):
        dense = bs[t].weight.grad.float().to_dense()
        torch.testing.assert_close(cc.optimizer_state.view(T, E)[t].cpu(), dense.pow(2).sum(dim=1), **tol)
        expect = torch.addcdiv(bs[t].weight.detach().float(), dense,
                               cc.optimizer_state.view(T, E)[t].cpu().sqrt().add(eps).view(E, 1), value=-lr)
        torch.testing.assert_close(cc.embedding_weights.detach().view(T, E, D)[t].cpu().float(), expect, **tol)


def test_module_state_dict_round_trip():
    cc = ops.TableBatchedEmbeddingBags(2, 10, 8, optimizer=ops.Optimizer.EXACT_ROWWISE_ADAGRAD, learning_rate=0.1,
                                       eps=0.1).cuda()
    sd = cc.state_dict()
    assert set(sd) == {"embedding_weights", "table_offsets", "optimizer_state"}
    assert sd["table_offsets"].tolist() == [0, 10] and sd["table_offsets"].dtype == torch.int32
    dd = ops.TableBatchedEmbeddingBags(2, 10, 8).cuda()
    dd.load_state_dict(sd)
    assert torch.equal(dd.embedding_weights, cc.embedding_weights)


def test_host_mapped_table_forward_backward():
    """EmbeddingLocation.HOST_MAPPED keeps the table in host-preferred managed memory
    (table_batched_embeddings_ops.py:159-167); results equal the device-resident module."""
    T, E, D, B, L = 2, 500, 16, 8, 5
    dev_m = ops.TableBatchedEmbeddingBags(T, E, D, learning_rate=0.1).cuda()
    host_m = ops.TableBatchedEmbeddingBags(T, E, D, learning_rate=0.1, managed=ops.EmbeddingLocation.HOST_MAPPED).cuda()
    assert host_m.embedding_weights.is_cuda
    host_m.embedding_weights.data.copy_(dev_m.embedding_weights.data)
    x = np.random.RandomState(0).randint(0, E, size=(T, B, L))
    indices, offsets = oracle.get_table_batched_offsets_from_dense(x)
    indices, offsets = torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda()
    go = torch.randn(B, T, D, device="cuda")
    a = dev_m(indices, offsets)
    b = host_m(indices, offsets)
    torch.testing.assert_close(a, b, rtol=0, atol=0)
    a.backward(go)
    b.backward(go)
    torch.testing.assert_close(dev_m.embedding_weights.data, host_m.embedding_weights.data, rtol=0, atol=0)
