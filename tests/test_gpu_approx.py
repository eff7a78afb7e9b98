"""GPU parity of the approximate rowwise-Adagrad backward and of the per-sample-weight gradient
against the CPU oracle, through libtbe_b200.so (reference: test_table_batched_embeddings.py:219-340)."""
import os

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import table_batched_embeddings as tbe
from sparse_ads_baselines_b200 import table_batched_embeddings_ops as ops

from tbe_testlib import assert_close, make_case, to_device

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _approx(c, state, lr, eps, weighted, sr=False):
    w = c["weights_d"].clone()
    s = state.clone()
    gp = tbe.backward_approx_adagrad(c["grad_d"], w, c["table_offsets_d"], c["indices_d"], c["offsets_d"],
                                     c["psw_d"] if weighted else None, s, lr, eps, 200, sr, 1)
    return w, s, gp


@pytest.mark.parametrize("D", [4, 12, 64, 128, 260, 1024])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("weighted", [False, True])
def test_approx_adagrad_unique_rows_matches_reference_formula(cuda_device, D, dtype, weighted):
    """No repeated rows (the only inputs on which the reference's racy kernel is well defined):
    state = |grad_bag|^2 * w_l^2 and w - w_l*lr*grad/(sqrt(state)+eps), lr = 0.5, eps = 0.2
    (test_table_batched_embeddings.py:296-318)."""
    c = to_device(make_case(T=3, E=400, D=D, B=8, Lmax=10, dtype=dtype, seed=D, fixed_L=10, unique=True,
                            weighted=weighted), cuda_device)
    s0 = torch.zeros(c["T"] * c["E"], device=cuda_device)
    w1, s1, gp = _approx(c, s0, 0.5, 0.2, weighted)
    rw, rs, rgp = oracle.approx_rowwise_adagrad_step(c["weights"], s0.cpu(), c["table_offsets"], c["indices"],
                                                     c["offsets"], c["grad"], 0.5, 0.2, c["psw"] if weighted else None)
    st = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(s1.cpu(), rs, **st)
    assert_close(w1, rw, dtype)
    if weighted:
        scale = (c["weights"].float().abs().max() * c["grad"].float().abs().max() * D).item()
        tol = (1e-2 if dtype == torch.float16 else 1e-5) * scale
        assert (gp.float().cpu() - rgp.float()).abs().max().item() <= tol
    else:
        assert gp is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("weighted", [False, True])
def test_approx_adagrad_repeated_rows_are_applied_in_index_order(cuda_device, dtype, weighted):
    c = to_device(make_case(T=2, E=9, D=32, B=12, Lmax=6, dtype=dtype, seed=3, weighted=weighted), cuda_device)
    s0 = torch.rand(c["T"] * c["E"], device=cuda_device)
    w1, s1, _ = _approx(c, s0, 0.1, 0.2, weighted)
    rw, rs, _ = oracle.approx_rowwise_adagrad_step(c["weights"], s0.cpu(), c["table_offsets"], c["indices"],
                                                   c["offsets"], c["grad"], 0.1, 0.2, c["psw"] if weighted else None)
    st = dict(rtol=2e-3, atol=2e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(s1.cpu(), rs, **st)
    assert_close(w1, rw, dtype)
    # deterministic
    w2, s2, _ = _approx(c, s0, 0.1, 0.2, weighted)
    assert torch.equal(w1, w2) and torch.equal(s1, s2)


@pytest.mark.parametrize("dtype,D", [(torch.float32, 32), (torch.float16, 128), (torch.float32, 68)])
@pytest.mark.parametrize("T,E,B,L", [(2, 6, 300, 3), (3, 40, 64, 9), (1, 2, 700, 1)])
def test_approx_adagrad_hot_rows(cuda_device, dtype, D, T, E, B, L):
    """Rows with hundreds of lookups: runs that cross the 32-entry tiles and runs long enough for the
    CTA-per-run kernel.  The per-lookup state sequence (a prefix sum on the device) and the weighted
    sum of gradient rows must give the oracle's one-lookup-at-a-time result, deterministically."""
    c = to_device(make_case(T=T, E=E, D=D, B=B, Lmax=L, dtype=dtype, seed=D + B, fixed_L=L), cuda_device)
    c["grad_d"] = c["grad_d"] * 0.1
    c["grad"] = c["grad_d"].cpu()
    s0 = torch.rand(T * E, device=cuda_device) * 0.5
    w1, s1, _ = _approx(c, s0, 0.05, 0.1, False)
    rw, rs, _ = oracle.approx_rowwise_adagrad_step(c["weights"], s0.cpu(), c["table_offsets"], c["indices"],
                                                   c["offsets"], c["grad"], 0.05, 0.1)
    torch.testing.assert_close(s1.cpu(), rs, rtol=1e-3 if dtype == torch.float16 else 1e-5, atol=1e-5)
    # hundreds of terms per row, summed in another order than the oracle's: absolute 1e-5 in fp32
    tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(w1.float().cpu(), rw.float(), **tol)
    w2, s2, _ = _approx(c, s0, 0.05, 0.1, False)
    assert torch.equal(w1, w2) and torch.equal(s1, s2)


def test_approx_golden(cuda_device):
    z = np.load(os.path.join(GOLDEN, "tiny_fp32_weighted_approx.npz"))
    T, E = int(z["T"]), int(z["E"])
    dev = cuda_device
    w = torch.from_numpy(z["weights"]).to(dev)
    s = torch.from_numpy(z["state0"]).to(dev)
    to = torch.tensor([t * E for t in range(T)], dtype=torch.int32, device=dev)
    gp = tbe.backward_approx_adagrad(torch.from_numpy(z["grad"]).to(dev), w, to, torch.from_numpy(z["indices"]).to(dev),
                                     torch.from_numpy(z["offsets"]).to(dev), torch.from_numpy(z["psw"]).to(dev), s,
                                     float(z["lr"]), float(z["eps"]), 200, False, 1)
    torch.testing.assert_close(s.cpu(), torch.from_numpy(z["state_after"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(w.cpu(), torch.from_numpy(z["weights_after"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(gp.cpu(), torch.from_numpy(z["grad_psw"]), rtol=1e-4, atol=1e-5)


def test_per_sample_weight_gradient_matches_autograd(cuda_device):
    """With lr = 0 the module is a pure function of the per-sample weights; its gradient must equal
    EmbeddingBag's (the reference runs torch.autograd.gradcheck in fp64 here,
    test_table_batched_embeddings.py:320-340)."""
    T, E, D, B, L = 3, 50, 8, 6, 5
    c = to_device(make_case(T=T, E=E, D=D, B=B, Lmax=L, dtype=torch.float64, seed=1, fixed_L=L, weighted=True),
                  cuda_device)
    m = ops.TableBatchedEmbeddingBags(T, E, D, optimizer=ops.Optimizer.APPROX_ROWWISE_ADAGRAD, learning_rate=0.0,
                                      eps=0.2).cuda().double()
    m.embedding_weights.data.copy_(c["weights_d"])
    psw = c["psw_d"].clone().requires_grad_(True)
    out = m(c["indices_d"], c["offsets_d"], psw)
    out.backward(c["grad_d"])
    _, ref = oracle.dense_gradients(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], c["psw"])
    torch.testing.assert_close(psw.grad.cpu(), ref, rtol=1e-10, atol=1e-10)
    assert torch.equal(m.embedding_weights.data, c["weights_d"])  # lr = 0 leaves the table alone


def test_module_approx_adagrad(cuda_device):
    T, E, D, B, L = 4, 10_000, 64, 16, 10
    c = make_case(T=T, E=E, D=D, B=B, Lmax=L, dtype=torch.float32, seed=5, fixed_L=L, unique=True)
    m = ops.TableBatchedEmbeddingBags(T, E, D, optimizer=ops.Optimizer.APPROX_ROWWISE_ADAGRAD, learning_rate=0.5,
                                      eps=0.2).cuda()
    m.embedding_weights.data.copy_(c["weights"].cuda())
    out = m(torch.from_numpy(c["indices"]).cuda(), torch.from_numpy(c["offsets"]).cuda())
    out.backward(c["grad"].cuda())
    rw, rs, _ = oracle.approx_rowwise_adagrad_step(c["weights"], torch.zeros(T * E), c["table_offsets"], c["indices"],
                                                   c["offsets"], c["grad"], 0.5, 0.2)
    torch.testing.assert_close(m.optimizer_state.cpu(), rs, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(m.embedding_weights.detach().cpu(), rw, rtol=1e-4, atol=1e-4)
