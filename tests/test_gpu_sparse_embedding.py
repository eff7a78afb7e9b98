"""The older ``sparse_embedding_cuda`` op surface ([E][T][D] weights, batch-major bags), written after
the reference's test_sparse_embedding_cuda.py:12-135: fused module against one EmbeddingBag per table,
dense and CSR inputs, forward and fused SGD (lr fixed at 0.05)."""
import numpy as np
import pytest
import torch

from sparse_ads_baselines_b200 import sparse_embedding_cuda_ops as se_ops

pytestmark = pytest.mark.gpu


def _merged_offsets(B, T, L, device):
    # offsets[b][t] = (b*T + t) * L, shape [B, T+1] (test_sparse_embedding_cuda.py:60-72)
    o = np.fromfunction(lambda b, t: (b * T + t) * L, (B, T + 1), dtype=np.int64).astype(np.int32)
    return torch.from_numpy(o).to(device)


@pytest.mark.parametrize("T,D,B,L", [(1, 4, 1, 1), (4, 64, 32, 32), (3, 256, 7, 5), (2, 128, 16, 40)])
@pytest.mark.parametrize("fp16", [False, True])
def test_forward(cuda_device, T, D, B, L, fp16):
    E = 1000
    torch.manual_seed(T * 100 + D)
    bs = [torch.nn.EmbeddingBag(E, D, mode="sum", sparse=True) for _ in range(T)]
    xs = [torch.randint(low=0, high=E, size=(B, L)) for _ in range(T)]
    f = torch.cat([b(x).view(B, 1, D) for b, x in zip(bs, xs)], dim=1)
    cc = se_ops.UniformShardedEmbeddingBags(T, E, D, fp16=fp16).cuda()
    for t in range(T):
        cc.embedding_weights.data[:, t, :] = bs[t].weight.data.to(cc.embedding_weights.dtype).cuda()
    x = torch.cat([x.view(B, 1, L) for x in xs], dim=1).cuda()
    fc = cc(x.int())
    fc2 = cc(x.int().contiguous().view(-1), _merged_offsets(B, T, L, cuda_device))
    tol = dict(rtol=1e-2, atol=2e-2) if fp16 else dict(rtol=1e-5, atol=1e-5)
    assert fc.shape == (B, T, D)
    torch.testing.assert_close(fc.detach().float().cpu(), f.detach(), **tol)
    torch.testing.assert_close(fc2.detach().float().cpu(), f.detach(), **tol)


@pytest.mark.parametrize("T,D,B,L,repeats", [(2, 8, 4, 3, False), (4, 64, 16, 10, False), (3, 32, 8, 6, True)])
@pytest.mark.parametrize("fp16", [False, True])
def test_backward(cuda_device, T, D, B, L, repeats, fp16):
    E = 10_000 if not repeats else 20
    rs = np.random.RandomState(T + D)
    torch.manual_seed(1)
    bs = [torch.nn.EmbeddingBag(E, D, mode="sum", sparse=True) for _ in range(T)]
    xs = [torch.from_numpy(rs.choice(E, size=(B, L), replace=repeats).astype(np.int64)) for _ in range(T)]
    fs = [b(x) for b, x in zip(bs, xs)]
    gos = [torch.randn_like(f) for f in fs]
    [f.backward(go) for f, go in zip(fs, gos)]
    lr = 0.05
    new_weights = [b.weight.detach() - b.weight.grad.to_dense() * lr for b in bs]
    go = torch.cat([g.view(B, 1, D) for g in gos], dim=1).cuda()
    x = torch.cat([x.view(B, 1, L) for x in xs], dim=1).cuda()
    tol = dict(rtol=1e-2, atol=2e-2) if fp16 else dict(rtol=1e-5, atol=1e-5)
    for csr in (False, True):
        cc = se_ops.UniformShardedEmbeddingBags(T, E, D, fp16=fp16).cuda()
        for t in range(T):
            cc.embedding_weights.data[:, t, :] = bs[t].weight.data.to(cc.embedding_weights.dtype).cuda()
        if csr:
            out = cc(x.int().contiguous().view(-1), _merged_offsets(B, T, L, cuda_device))
        else:
            out = cc(x.int())
        out.backward(go.to(out.dtype))
        for t in range(T):
            torch.testing.assert_close(cc.embedding_weights.detach()[:, t, :].float().cpu(), new_weights[t], **tol)


def test_collectives_are_identities_without_a_process_group(cuda_device):
    """At world size 1 every collective returns its input (sparse_embedding_cuda.cpp:423-425,492-494,
    541-543), which is what lets the reference's single-process model test pass."""
    x = torch.randn(4, 3, 8, device=cuda_device, requires_grad=True)
    assert se_ops.All2AllFunction.apply(x).shape == x.shape
    assert se_ops.ReduceScatterFunction.apply(x).shape == x.shape
    se_ops.All2AllFunction.apply(x).sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
