"""This library's CUDA path against the REFERENCE's own kernels.

Two layers.  (1) Stored vectors: ``tests/golden/reference_*.npz`` hold outputs of the reference's
``table_batched_embeddings`` extension (tests/golden/make_reference_golden.py); the same inputs go
through this library's functions of the same names and arguments.  (2) Live: when the reference
extension built by ``oracle/build_ref.py`` is present (``oracle/_ref/``), both modules are called
side by side on larger seeded inputs -- skewed indices, ragged bags, fp16 rows -- with the same
argument lists.  Cases where the reference races on repeated rows (SGD, approximate Adagrad) use
duplicate-free indices, as the reference's tests do (test_table_batched_embeddings.py:177-182).
Tolerances: fp32 1e-5, fp16 1e-2; the optimizer state within 1e-5.
"""
import os

import numpy as np
import pytest
import torch

from oracle import build_ref
from sparse_ads_baselines_b200 import table_batched_embeddings as tbe
from test_oracle_reference_pin import LOOKUP_CASES, TOL, expected_after, load_reference_case, mixed_tables, GOLDEN

pytestmark = pytest.mark.gpu


def _dev(c, dev):
    return dict(w=c["weights_t"].to(dev).clone(), to=torch.tensor(c["table_offsets_l"], dtype=torch.int32, device=dev),
                idx=torch.from_numpy(c["indices"]).to(dev), off=torch.from_numpy(c["offsets"]).to(dev),
                go=c["grad_t"].to(dev), psw=c["psw_t"].to(dev) if c["weighted"] else None,
                state=c["state_t"].to(dev).clone())


@pytest.mark.parametrize("name", LOOKUP_CASES)
def test_stored_reference_vectors(cuda_device, name):
    c = load_reference_case(name)
    d = _dev(c, cuda_device)
    out = tbe.forward(d["w"], d["to"], d["idx"], d["off"], d["psw"], 10, 1, False)
    torch.testing.assert_close(out.float().cpu(), torch.from_numpy(c["out"]), **TOL[c["dtype"]])
    if c["optimizer"] == "none":
        return
    gpsw = None
    if c["optimizer"] == "sgd":
        tbe.backward_sgd(d["go"], d["w"], d["to"], d["idx"], d["off"], c["lr"], 10, 1, False)
    elif c["optimizer"] == "exact_rowwise_adagrad":
        tbe.backward_exact_adagrad(d["go"], d["w"], d["to"], d["idx"], d["off"], None, d["state"], c["lr"], c["eps"], False, 1)
    else:
        gpsw = tbe.backward_approx_adagrad(d["go"], d["w"], d["to"], d["idx"], d["off"], d["psw"], d["state"], c["lr"],
                                           c["eps"], 10, False, 1)
    w, s = d["w"].float().cpu(), d["state"].cpu()
    ref_w, ref_s, rows = expected_after(c)
    if rows is not None:
        np.testing.assert_allclose(w.double().view(c["T"], -1).sum(1).numpy(), c["weights_after_table_sums"], rtol=1e-6)
        np.testing.assert_allclose(s.double().view(c["T"], -1).sum(1).numpy(), c["state_after_table_sums"], rtol=1e-6)
        w, s = w[rows], s[rows]
    torch.testing.assert_close(w, ref_w, **TOL[c["dtype"]])
    torch.testing.assert_close(s, ref_s, rtol=1e-5, atol=1e-5)
    if "grad_psw" in c:
        torch.testing.assert_close(gpsw.float().cpu(), torch.from_numpy(c["grad_psw"]), **TOL[c["dtype"]])


def test_stored_reference_mixed_width(cuda_device):
    dev = cuda_device
    z = np.load(os.path.join(GOLDEN, "reference_mixed_exact_fp32.npz"))
    w, st = torch.from_numpy(z["weights"]).to(dev), torch.from_numpy(z["state"]).to(dev)
    to, tdo, do = (torch.from_numpy(z[k]).to(dev) for k in ("table_offsets", "table_dim_offsets", "dim_offsets"))
    idx, off = torch.from_numpy(z["indices"]).to(dev), torch.from_numpy(z["offsets"]).to(dev)
    total_D = int(z["dim_offsets"][-1])
    out = tbe.forward_mixed_D(w, to, do, total_D, idx, off, None, 5, 1, False)
    torch.testing.assert_close(out.cpu(), torch.from_numpy(z["out"]), **TOL["fp32"])
    tbe.backward_exact_adagrad_mixed_D(torch.from_numpy(z["grad"]).to(dev), w, to, tdo, do, total_D, idx, off, None, st,
                                       float(z["lr"]), float(z["eps"]), False, 1)
    torch.testing.assert_close(w.cpu(), torch.from_numpy(z["weights_after"]), **TOL["fp32"])
    torch.testing.assert_close(st.cpu(), torch.from_numpy(z["state_after"]), rtol=1e-5, atol=1e-5)


def test_stored_reference_construct_offsets(cuda_device):
    z = np.load(os.path.join(GOLDEN, "reference_construct_offsets.npz"))
    out = tbe.construct_offsets(torch.from_numpy(z["begin"]).to(cuda_device), torch.from_numpy(z["totals"]).to(cuda_device))
    assert np.array_equal(out.cpu().numpy(), z["lengths_out"])


# ------------------------------------------------------------------ live, side by side
@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(build_ref.OUT):
        pytest.skip("the reference extension has not been built into oracle/_ref/ (python oracle/build_ref.py)")
    return build_ref.load()


def _live_case(dev, T, E, D, B, dtype, seed, dist="uniform", lengths="ragged", Lmean=20, unique=False):
    rng = np.random.default_rng(seed)
    if lengths == "ragged":
        L = np.clip(rng.poisson(Lmean, size=(T, B)), 0, 100)
    else:
        L = np.full((T, B), Lmean)
    offsets = np.concatenate([[0], np.cumsum(L.reshape(-1))]).astype(np.int32)
    N = int(offsets[-1])
    if unique:
        per_table = L.sum(axis=1)
        assert per_table.max() <= E
        indices = np.concatenate([rng.permutation(E)[:n] for n in per_table]).astype(np.int32)
    elif dist == "zipf":
        indices = (rng.zipf(1.05, size=N).astype(np.int64) % E).astype(np.int32)
    else:
        indices = rng.integers(0, E, size=N).astype(np.int32)
    w = torch.from_numpy(rng.uniform(-0.5, 0.5, size=(T * E, D)).astype(np.float32)).to(dtype).to(dev)
    go = torch.from_numpy(rng.standard_normal(size=(B, T, D)).astype(np.float32) * 0.1).to(dtype).to(dev)
    psw = torch.from_numpy(rng.uniform(0.5, 1.5, size=N).astype(np.float32)).to(dtype).to(dev)
    st = torch.from_numpy(rng.uniform(0, 0.5, size=T * E).astype(np.float32)).to(dev)
    to = (torch.arange(T, dtype=torch.int32) * E).to(dev)
    return dict(w=w, go=go, psw=psw, state=st, to=to, idx=torch.from_numpy(indices).to(dev),
                off=torch.from_numpy(offsets).to(dev), Lmax=int(L.max()), tol=TOL["fp16" if dtype == torch.float16 else "fp32"])


@pytest.mark.parametrize("dtype,D", [(torch.float32, 128), (torch.float16, 128), (torch.float16, 36), (torch.float32, 320)])
@pytest.mark.parametrize("weighted", [False, True])
def test_live_forward(cuda_device, ref, dtype, D, weighted):
    c = _live_case(cuda_device, T=6, E=20000, D=D, B=256, dtype=dtype, seed=D, dist="zipf")
    psw = c["psw"] if weighted else None
    expect = ref.forward(c["w"], c["to"], c["idx"], c["off"], psw, c["Lmax"], 1, False)
    got = tbe.forward(c["w"], c["to"], c["idx"], c["off"], psw, c["Lmax"], 1, False)
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), expect.float(), **c["tol"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("dist", ["uniform", "zipf"])
def test_live_exact_rowwise_adagrad_with_repeats(cuda_device, ref, dtype, dist):
    """The reference's exact kernel sorts and sums repeated rows like this library's does, so skewed
    inputs with runs of hundreds of equal rows are comparable (table_batched_embeddings_cuda.cu:1499-1587)."""
    c = _live_case(cuda_device, T=4, E=50000, D=128, B=512, dtype=dtype, seed=3, dist=dist)
    w_ref, s_ref = c["w"].clone(), c["state"].clone()
    ref.backward_exact_adagrad(c["go"], w_ref, c["to"], c["idx"], c["off"], None, s_ref, 0.05, 0.1, False, 1)
    w, s = c["w"].clone(), c["state"].clone()
    tbe.backward_exact_adagrad(c["go"], w, c["to"], c["idx"], c["off"], None, s, 0.05, 0.1, False, 1)
    torch.cuda.synchronize()
    assert not torch.equal(w, c["w"])
    torch.testing.assert_close(s, s_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(w.float(), w_ref.float(), **c["tol"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_live_sgd_unique_rows(cuda_device, ref, dtype):
    c = _live_case(cuda_device, T=4, E=50000, D=128, B=512, dtype=dtype, seed=4, unique=True)
    w_ref = c["w"].clone()
    ref.backward_sgd(c["go"], w_ref, c["to"], c["idx"], c["off"], 0.05, c["Lmax"], 1, False)
    w = c["w"].clone()
    tbe.backward_sgd(c["go"], w, c["to"], c["idx"], c["off"], 0.05, c["Lmax"], 1, False)
    torch.cuda.synchronize()
    torch.testing.assert_close(w.float(), w_ref.float(), **c["tol"])


@pytest.mark.parametrize("weighted", [False, True])
def test_live_approx_rowwise_adagrad_unique_rows(cuda_device, ref, weighted):
    c = _live_case(cuda_device, T=3, E=50000, D=64, B=256, dtype=torch.float32, seed=5, unique=True)
    psw = c["psw"] if weighted else None
    w_ref, s_ref = c["w"].clone(), c["state"].clone()
    g_ref = ref.backward_approx_adagrad(c["go"], w_ref, c["to"], c["idx"], c["off"], psw, s_ref, 0.05, 0.1, c["Lmax"], False, 1)
    w, s = c["w"].clone(), c["state"].clone()
    g = tbe.backward_approx_adagrad(c["go"], w, c["to"], c["idx"], c["off"], psw, s, 0.05, 0.1, c["Lmax"], False, 1)
    torch.cuda.synchronize()
    torch.testing.assert_close(s, s_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(w, w_ref, **c["tol"])
    if weighted:
        torch.testing.assert_close(g, g_ref, **c["tol"])
    else:
        assert g is None and g_ref is None
