"""GPU parity of the pooled forward against the CPU oracle, through libtbe_b200.so."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import _lib, workloads
from sparse_ads_baselines_b200 import table_batched_embeddings as tbe

from tbe_testlib import assert_close, forward_scale, make_case, to_device

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _run_forward(c, pooling="sum", weighted=False):
    return tbe.forward(c["weights_d"], c["table_offsets_d"], c["indices_d"], c["offsets_d"],
                       c["psw_d"] if weighted else None, 200, 1, False, pooling_mode=pooling)


# D spans: one vector per row, sub-warp groups, exactly one warp, multi-chunk rows, non-power-of-two
# vector counts, and fp16 rows that are only 8-byte aligned (D % 8 == 4).
@pytest.mark.parametrize("D", [4, 8, 12, 20, 64, 100, 128, 256, 260, 512, 2048])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("pooling,weighted", [("sum", False), ("mean", False), ("sum", True)])
def test_forward_matches_embeddingbag(cuda_device, D, dtype, pooling, weighted):
    c = to_device(make_case(T=3, E=50, D=D, B=9, Lmax=40, dtype=dtype, seed=D, weighted=weighted), cuda_device)
    out = _run_forward(c, pooling, weighted)
    assert out.shape == (c["B"], c["T"], D) and out.dtype == dtype
    ref = oracle.forward(c["weights"], c["table_offsets"], c["indices"], c["offsets"],
                         c["psw"] if weighted else None, pooling, compute_dtype=torch.float32)
    assert_close(out, ref, dtype, scale=forward_scale(c, pooling, weighted))


def test_forward_fp64(cuda_device):
    c = to_device(make_case(T=2, E=30, D=12, B=5, Lmax=7, dtype=torch.float64, seed=0, weighted=True), cuda_device)
    out = _run_forward(c, "sum", True)
    ref = oracle.forward(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["psw"], "sum")
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("T,B,L", [(1, 1, 1), (4, 32, 32), (2, 5, 33), (1, 3, 200), (7, 1, 0)])
def test_forward_reference_test_shapes(cuda_device, T, B, L):
    """Fixed-L cases in the ranges of the reference's test_forward
    (test_table_batched_embeddings.py:115-122), plus L > 32 and all-empty bags."""
    for dtype in (torch.float32, torch.float16):
        c = to_device(make_case(T=T, E=10_000, D=64, B=B, Lmax=L, dtype=dtype, seed=T * 100 + B, fixed_L=L), cuda_device)
        out = _run_forward(c)
        ref = oracle.forward(c["weights"], c["table_offsets"], c["indices"], c["offsets"], compute_dtype=torch.float32)
        assert_close(out, ref, dtype, scale=forward_scale(c))


def test_forward_many_bags_covers_persistent_loop(cuda_device):
    """More bags than resident warps, ragged lengths, so every warp walks several bags through the
    prefetch pipeline."""
    c = to_device(make_case(T=8, E=1000, D=128, B=4096, Lmax=12, dtype=torch.float16, seed=11), cuda_device)
    out = _run_forward(c)
    ref = oracle.forward(c["weights"], c["table_offsets"], c["indices"], c["offsets"], compute_dtype=torch.float32)
    assert_close(out, ref, torch.float16)


@pytest.mark.parametrize("unroll", [2, 4, 8])
def test_forward_result_independent_of_tuning(cuda_device, unroll):
    """Results must not depend on launch hints (table_batched_embeddings_benchmark.py:179-206)."""
    c = to_device(make_case(T=4, E=500, D=128, B=64, Lmax=50, dtype=torch.float16, seed=5), cuda_device)
    base = _run_forward(c)
    try:
        _lib.call("tbe_set_tuning", b"fwd_unroll", unroll)
        _lib.call("tbe_set_tuning", b"fwd_threads", 128)
        other = _run_forward(c)
    finally:
        _lib.call("tbe_set_tuning", b"fwd_unroll", 0)
        _lib.call("tbe_set_tuning", b"fwd_threads", 0)
    ref = oracle.forward(c["weights"], c["table_offsets"], c["indices"], c["offsets"], compute_dtype=torch.float32)
    assert_close(other, ref, torch.float16)
    assert_close(base, ref, torch.float16)


@pytest.mark.parametrize("name", sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "tiny_*.npz"))))
def test_forward_golden(cuda_device, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dtype = torch.float16 if str(z["dtype"]) == "fp16" else torch.float32
    T, E = int(z["T"]), int(z["E"])
    w = torch.from_numpy(z["weights"]).to(dtype).to(cuda_device)
    to = torch.tensor([t * E for t in range(T)], dtype=torch.int32, device=cuda_device)
    psw = torch.from_numpy(z["psw"]).to(dtype).to(cuda_device) if "psw" in z.files else None
    out = tbe.forward(w, to, torch.from_numpy(z["indices"]).to(cuda_device), torch.from_numpy(z["offsets"]).to(cuda_device),
                      psw, 200, 1, False, pooling_mode=str(z["pooling"]))
    assert_close(out, torch.from_numpy(z["out"]), dtype)


def test_forward_cfg1_golden(cuda_device):
    z = np.load(os.path.join(GOLDEN, "cfg1.npz"))
    w = workloads.WORKLOADS["cfg1"]
    indices, offsets = workloads.make_inputs(w)
    weights = torch.from_numpy(workloads.make_weights(w)).to(cuda_device)
    to = torch.arange(w.T, dtype=torch.int32, device=cuda_device) * w.E
    out = tbe.forward(weights, to, torch.from_numpy(indices).to(cuda_device), torch.from_numpy(offsets).to(cuda_device),
                      None, 200, 4, False)
    torch.testing.assert_close(out.cpu(), torch.from_numpy(z["out"]), rtol=1e-5, atol=1e-7)


def test_forward_errors(cuda_device):
    c = to_device(make_case(T=2, E=10, D=8, B=2, Lmax=3, dtype=torch.float32, seed=0), cuda_device)
    with pytest.raises(RuntimeError, match="multiple of 4"):
        tbe.forward(torch.zeros(20, 6, device=cuda_device), c["table_offsets_d"], c["indices_d"], c["offsets_d"], None,
                    200, 1, False)
    with pytest.raises(RuntimeError, match="int32"):
        tbe.forward(c["weights_d"], c["table_offsets_d"], c["indices_d"].long(), c["offsets_d"], None, 200, 1, False)
    with pytest.raises(RuntimeError, match="BT_block_size"):
        tbe.forward(c["weights_d"], c["table_offsets_d"], c["indices_d"], c["offsets_d"], None, 200, 0, False)
    with pytest.raises(RuntimeError):
        tbe.forward(c["weights_d"], c["table_offsets_d"], c["indices_d"], c["offsets_d"],
                    torch.ones(c["N"], device=cuda_device), 200, 1, False, pooling_mode="mean")


def test_check_inputs(cuda_device):
    c = to_device(make_case(T=2, E=10, D=8, B=3, Lmax=4, dtype=torch.float32, seed=1, empty_bags=False), cuda_device)
    rows = torch.tensor([10, 10], dtype=torch.int32, device=cuda_device)
    tbe.check_inputs(c["indices_d"], c["offsets_d"], rows)
    bad = c["indices_d"].clone()
    bad[2] = 10
    with pytest.raises(_lib.TBEError, match="outside table"):
        tbe.check_inputs(bad, c["offsets_d"], rows)
    off = c["offsets_d"].clone()
    off[2] = off[1] - 1
    with pytest.raises(_lib.TBEError, match="decrease"):
        tbe.check_inputs(c["indices_d"], off, rows)


def test_construct_offsets(cuda_device):
    """The reference's test_construct_offsets (test_table_batched_embeddings.py:61-112): fused offsets
    reproduce every per-table bag extent exactly."""
    rng = np.random.default_rng(0)
    for T, B, L in [(1, 1, 2), (5, 7, 9), (128, 128, 16), (3, 1, 128)]:
        Ls = rng.integers(1, L, size=(T, B))
        begin = np.concatenate([np.zeros((T, 1), dtype=np.int64), np.cumsum(Ls, axis=1)[:, :-1]], axis=1).astype(np.int32)
        totals = Ls.sum(axis=1).astype(np.int32)
        out = tbe.construct_offsets(torch.from_numpy(begin).to(cuda_device), torch.from_numpy(totals).to(cuda_device))
        assert out.dtype == torch.int32
        assert np.array_equal(out.cpu().numpy(), oracle.construct_offsets(begin, totals))
        fused = torch.cumsum(out, dim=0).cpu().numpy()
        assert np.array_equal(np.diff(fused), Ls.reshape(-1))


def test_forward_full_size_cfg2_checksum(cuda_device):
    """Config 2 at full size (T=64, E=1M, D=128 fp16, B=2048, L=38).  The oracle cannot run this in
    seconds, so parity uses size-independent properties: (1) a sample of bags recomputed on the CPU
    from the same rows, (2) the checksum sum_d sum_bags out == sum over lookups of row sums,
    computed by an independent gather in fp64."""
    w = workloads.WORKLOADS["cfg2"]
    indices, offsets = workloads.make_inputs(w)
    dev = cuda_device
    gen = torch.Generator(device=dev).manual_seed(0)
    weights = torch.empty(w.T * w.E, w.D, dtype=torch.float16, device=dev)
    for t in range(w.T):  # U(-0.01, 0.01) without a 33 GB fp32 temporary
        weights[t * w.E:(t + 1) * w.E] = (torch.rand(w.E, w.D, device=dev, generator=gen) * 0.02 - 0.01).half()
    to = torch.arange(w.T, dtype=torch.int32, device=dev) * w.E
    idx_d, off_d = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
    out = tbe.forward(weights, to, idx_d, off_d, None, 200, 2, False)
    assert out.shape == (w.B, w.T, w.D)
    # (1) sampled bags
    rng = np.random.default_rng(1)
    for bag in rng.integers(0, w.T * w.B, size=64):
        t, b = divmod(int(bag), w.B)
        rows = torch.from_numpy(indices[offsets[bag]:offsets[bag + 1]].astype(np.int64)).to(dev) + t * w.E
        ref = weights[rows].float().sum(dim=0)
        torch.testing.assert_close(out[b, t].float(), ref, rtol=1e-2, atol=1e-3)
    # (2) checksum of checksums, per table
    row_sums = weights.float().sum(dim=1).double()  # [T*E]
    for t in range(0, w.T, 7):
        lo, hi = int(offsets[t * w.B]), int(offsets[(t + 1) * w.B])
        expect = row_sums[idx_d[lo:hi].long() + t * w.E].sum().item()
        got = out[:, t].double().sum().item()
        assert abs(got - expect) <= 2e-3 * max(1.0, abs(expect)) + 0.5  # fp16 output rounding of 2048*128 values
