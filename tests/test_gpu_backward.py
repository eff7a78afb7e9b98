"""GPU parity of the fused backward (exact SGD, exact rowwise Adagrad) and of its integer
bookkeeping against the CPU oracle, through libtbe_b200.so."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import _lib, workloads
from sparse_ads_baselines_b200 import table_batched_embeddings as tbe

from tbe_testlib import assert_close, make_case, to_device

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _sgd(c, lr, pooling="sum", grad=None):
    w = c["weights_d"].clone()
    tbe.backward_sgd(c["grad_d"] if grad is None else grad, w, c["table_offsets_d"], c["indices_d"], c["offsets_d"],
                     lr, 200, 1, False, pooling_mode=pooling)
    return w


def _adagrad(c, state, lr, eps, pooling="sum"):
    w = c["weights_d"].clone()
    s = state.clone()
    tbe.backward_exact_adagrad(c["grad_d"], w, c["table_offsets_d"], c["indices_d"], c["offsets_d"], None, s, lr, eps,
                               False, 1, pooling_mode=pooling)
    return w, s


def test_sort_segments_exact(cuda_device):
    """Sorted row ids, the bag of every sorted entry and the run starts equal the oracle's stable sort
    exactly (integers)."""
    for seed, (T, E, B, Lmax) in enumerate([(1, 1, 1, 1), (3, 17, 5, 6), (4, 100, 64, 20), (2, 5, 300, 3), (5, 70000, 33, 9)]):
        c = to_device(make_case(T=T, E=E, D=4, B=B, Lmax=Lmax, dtype=torch.float32, seed=seed), cuda_device)
        rows, bags, starts = tbe.sort_segments(c["table_offsets_d"], c["indices_d"], c["offsets_d"], T * E)
        r0, b0, s0 = oracle.sort_segments(c["table_offsets"], c["indices"], c["offsets"])
        assert np.array_equal(rows.cpu().numpy(), r0)
        assert np.array_equal(bags.cpu().numpy(), b0)
        assert np.array_equal(starts.cpu().numpy(), s0)


def test_sort_segments_empty_input(cuda_device):
    to = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    off = torch.zeros(2 * 3 + 1, dtype=torch.int32, device=cuda_device)
    idx = torch.zeros(0, dtype=torch.int32, device=cuda_device)
    rows, bags, starts = tbe.sort_segments(to, idx, off, 10)
    assert rows.numel() == 0 and bags.numel() == 0 and starts.numel() == 0


def _table_sort_case(rng, T, E, B, Lmax, hot):
    """Ragged bags (empty ones included); with ``hot`` most lookups of a table hit a few rows, so one
    bucket of the table-segmented sort outgrows a CTA and takes the queued path."""
    lengths = rng.integers(0, Lmax + 1, size=(T, B))
    lengths[rng.random((T, B)) < 0.1] = 0
    offsets = oracle.offsets_from_lengths(lengths)
    N = int(offsets[-1])
    indices = rng.integers(0, E, size=N).astype(np.int32)
    if hot:
        pick = rng.random(N) < 0.8
        indices[pick] = rng.integers(0, min(E, 3), size=int(pick.sum())).astype(np.int32)
    return indices, offsets.astype(np.int32)


@pytest.mark.parametrize("T,E,B,Lmax,hot", [
    (1, 1, 1, 1, False),
    (3, 17, 5, 6, False),              # a bucket is one row: nothing to sort inside it
    (2, 1000, 4096, 16, False),        # several slices and tiles per table
    (2, 1000, 4096, 16, True),         # oversize buckets (~24,000 pairs: sorted in a cluster's shared memory)
    (1, 5000, 8192, 40, True),         # a bucket of ~120,000 pairs: beyond the cluster, passes through global memory
    (40, 3000, 1024, 30, True),        # more queued buckets than resident clusters
    (5, 70000, 2048, 40, False),       # many buckets per table, rows not a power of two
    (5, 70000, 2048, 40, True),
    (70, 300000, 64, 30, False),       # more tables than one slice each can fill
    (1, 2 ** 20, 3000, 50, False),
    (3, 2 ** 20 + 1, 1500, 50, True),  # index bits roll over to 21
    (1, 2 ** 24, 4096, 20, False),     # 1024 buckets of 2^14 rows: the most the narrow kernel variants take
    (1, 2 ** 24 + 1, 4096, 20, False), # one more row: the wide variants (up to 4096 buckets per table)
    (1, 2 ** 26 + 1, 4096, 20, False), # more than 4096 buckets: falls back to the device radix sort
    (2, 2 ** 20, 16384, 240, False),   # ~1.6 lookups per row: 2048 buckets of 512 rows, the wide variants
    (300, 5000, 8, 12, False),         # more tables than resident CTAs: one slice per table
])
def test_table_segmented_sort_exact(cuda_device, T, E, B, Lmax, hot):
    """With max_rows_per_table the plan comes from the table-segmented two-level sort; rows, bags and
    run starts must equal the oracle's stable sort exactly, and the device radix sort's."""
    rng = np.random.default_rng(T * 1000 + B + int(hot))
    indices, offsets = _table_sort_case(rng, T, E, B, Lmax, hot)
    dev = cuda_device
    to_np = np.arange(T, dtype=np.int64) * E
    to = torch.from_numpy(to_np.astype(np.int32)).to(dev)
    idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
    r0, b0, s0 = oracle.sort_segments(list(to_np), indices, offsets)
    for sort_mode in (0, 1):
        _lib.call("tbe_set_tuning", b"bwd_sort", sort_mode)
        try:
            rows, bags, starts = tbe.sort_segments(to, idx, off, T * E, max_rows_per_table=E)
        finally:
            _lib.call("tbe_set_tuning", b"bwd_sort", 0)
        assert np.array_equal(rows.cpu().numpy(), r0), sort_mode
        assert np.array_equal(bags.cpu().numpy(), b0), sort_mode
        assert np.array_equal(starts.cpu().numpy(), s0), sort_mode


@pytest.mark.parametrize("bucket,hot", [(8, False), (8, True), (64, False), (300, False), (2048, False)])
def test_table_segmented_sort_bucket_sizes(cuda_device, bucket, hot):
    """The bucket-size knob changes the geometry (buckets per table, CTA variants: 8 pairs per bucket
    means 1563 buckets per table, the wide variants), never the result."""
    rng = np.random.default_rng(bucket)
    T, E, B = 4, 50000, 1024
    indices, offsets = _table_sort_case(rng, T, E, B, 24, hot)
    dev = cuda_device
    to_np = np.arange(T, dtype=np.int64) * E
    to = torch.from_numpy(to_np.astype(np.int32)).to(dev)
    idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
    r0, b0, s0 = oracle.sort_segments(list(to_np), indices, offsets)
    _lib.call("tbe_set_tuning", b"sort_bucket", bucket)
    try:
        rows, bags, starts = tbe.sort_segments(to, idx, off, T * E, max_rows_per_table=E)
    finally:
        _lib.call("tbe_set_tuning", b"sort_bucket", 0)
    assert np.array_equal(rows.cpu().numpy(), r0)
    assert np.array_equal(bags.cpu().numpy(), b0)
    assert np.array_equal(starts.cpu().numpy(), s0)


def test_sgd_same_bits_with_either_sort(cuda_device):
    """The two plans order every run identically, so the updated weights agree bit for bit."""
    c = to_device(make_case(T=6, E=3000, D=64, B=512, Lmax=30, dtype=torch.float16, seed=11), cuda_device)
    out = []
    for sort_mode in (0, 1):
        _lib.call("tbe_set_tuning", b"bwd_sort", sort_mode)
        try:
            out.append(_sgd(c, 0.05))
        finally:
            _lib.call("tbe_set_tuning", b"bwd_sort", 0)
    assert torch.equal(out[0], out[1])


@pytest.mark.parametrize("dtype,pooling", [(torch.float16, "sum"), (torch.float32, "mean")])
def test_same_bits_with_tickets_or_a_fixed_stride(cuda_device, dtype, pooling):
    """The apply kernel's warps take their tiles of the sorted entries either with a fixed stride or
    from a ticket counter (the default once the pooled gradient outgrows L2); which warp processes a
    tile must not show in the result.  ~300,000 lookups: more tiles than resident warps."""
    c = to_device(make_case(T=8, E=20000, D=128, B=2048, Lmax=36, dtype=dtype, seed=21), cuda_device)
    state = torch.rand(8 * 20000, device=cuda_device)
    out = []
    for mode in (1, 2):
        _lib.call("tbe_set_tuning", b"bwd_stride", mode)
        try:
            out.append((_sgd(c, 0.05, pooling), *_adagrad(c, state, 0.05, 0.1, pooling)))
        finally:
            _lib.call("tbe_set_tuning", b"bwd_stride", 0)
    for a, b in zip(*out):
        assert torch.equal(a, b)
    ref = oracle.sgd_step(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], 0.05, pooling,
                          compute_dtype=torch.float32)
    assert_close(out[1][0], ref, dtype)


@pytest.mark.parametrize("D", [4, 8, 12, 64, 100, 128, 256, 260, 2048])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("pooling", ["sum", "mean"])
def test_sgd_with_repeated_rows(cuda_device, D, dtype, pooling):
    """E is small so rows repeat within and across bags: the update must equal w - lr * dense(grad)
    (test_table_batched_embeddings.py:191-193 without its no-repeat restriction)."""
    c = to_device(make_case(T=3, E=40, D=D, B=8, Lmax=12, dtype=dtype, seed=D + 1), cuda_device)
    w1 = _sgd(c, 0.05, pooling)
    ref = oracle.sgd_step(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], 0.05, pooling,
                          compute_dtype=torch.float32)
    assert_close(w1, ref, dtype)


def test_sgd_unique_rows_reference_test(cuda_device):
    """The reference's own SGD test: unique rows per table, lr = 0.05
    (test_table_batched_embeddings.py:163-216)."""
    for dtype in (torch.float32, torch.float16):
        c = to_device(make_case(T=4, E=10_000, D=64, B=32, Lmax=32, dtype=dtype, seed=3, fixed_L=32, unique=True),
                      cuda_device)
        w1 = _sgd(c, 0.05)
        ref = oracle.sgd_step(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], 0.05)
        assert_close(w1, ref, dtype)


@pytest.mark.parametrize("D", [4, 64, 128, 260, 1024])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("pooling", ["sum", "mean"])
def test_exact_rowwise_adagrad(cuda_device, D, dtype, pooling):
    """state = sum_d dense_grad^2 and w - lr*grad/(sqrt(state)+eps) with lr = 0.5, eps = 0.2 and
    E = 100 with replacement, as in the reference's test (test_table_batched_embeddings.py:219-318)."""
    c = to_device(make_case(T=5, E=100, D=D, B=16, Lmax=10, dtype=dtype, seed=D + 7, fixed_L=10), cuda_device)
    state0 = torch.rand(c["T"] * c["E"], device=cuda_device)
    w1, s1 = _adagrad(c, state0, 0.5, 0.2, pooling)
    rw, rs = oracle.exact_rowwise_adagrad_step(c["weights"], state0.cpu(), c["table_offsets"], c["indices"],
                                               c["offsets"], c["grad"], 0.5, 0.2, pooling)
    st = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(s1.cpu(), rs, **st)
    assert_close(w1, rw, dtype)


@pytest.mark.parametrize("opt", ["sgd", "adagrad"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_long_segments(cuda_device, opt, dtype):
    """A handful of rows receive hundreds of lookups each: exercises the queued long-run kernel, both
    with the default threshold and with a tiny one."""
    c = to_device(make_case(T=2, E=3, D=128, B=400, Lmax=4, dtype=dtype, seed=21, empty_bags=False), cuda_device)
    c["grad_d"] = (c["grad_d"] * 0.01).contiguous()
    c["grad"] = c["grad_d"].cpu()
    for thresh in (0, 5):
        try:
            _lib.call("tbe_set_tuning", b"long_segment", thresh)
            if opt == "sgd":
                w1 = _sgd(c, 0.05)
                ref = oracle.sgd_step(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], 0.05,
                                      compute_dtype=torch.float32)
            else:
                s0 = torch.zeros(6, device=cuda_device)
                w1, s1 = _adagrad(c, s0, 0.5, 0.2)
                ref, rs = oracle.exact_rowwise_adagrad_step(c["weights"], s0.cpu(), c["table_offsets"], c["indices"],
                                                            c["offsets"], c["grad"], 0.5, 0.2)
                torch.testing.assert_close(s1.cpu(), rs, rtol=2e-3, atol=1e-3)
        finally:
            _lib.call("tbe_set_tuning", b"long_segment", 0)
        assert_close(w1, ref, dtype)


@pytest.mark.parametrize("opt", ["sgd", "adagrad"])
@pytest.mark.parametrize("dtype,D,pooling", [(torch.float32, 128, "mean"), (torch.float16, 128, "sum"), (torch.float32, 260, "sum")])
def test_hot_rows_are_split_over_several_ctas(cuda_device, opt, dtype, D, pooling):
    """Rows with thousands of lookups: the queued run is cut into parts that different CTAs sum, and
    the CTA finishing the last part folds them in part order.  Results must match the oracle, be
    bit-identical from call to call, and agree with the one-CTA-per-run path (knob split_runs = 1)."""
    T, E, B, L = 2, 3, 3000, 2   # ~2,000 lookups per row: 7 parts of 256 entries
    c = to_device(make_case(T=T, E=E, D=D, B=B, Lmax=L, dtype=dtype, seed=31, fixed_L=L), cuda_device)
    c["grad_d"] = (c["grad_d"] * 0.01).contiguous()
    c["grad"] = c["grad_d"].cpu()
    s0 = torch.rand(T * E, device=cuda_device) * 0.1

    def run():
        if opt == "sgd":
            w = c["weights_d"].clone()
            tbe.backward_sgd(c["grad_d"], w, c["table_offsets_d"], c["indices_d"], c["offsets_d"], 0.05, 200, 1, False,
                             pooling_mode=pooling)
            return w, None
        return _adagrad(c, s0, 0.5, 0.2, pooling=pooling)

    w1, s1 = run()
    w2, s2 = run()
    assert torch.equal(w1, w2) and (s1 is None or torch.equal(s1, s2))
    try:
        _lib.call("tbe_set_tuning", b"split_runs", 1)
        w3, s3 = run()
    finally:
        _lib.call("tbe_set_tuning", b"split_runs", 0)
    tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(w1.float(), w3.float(), **tol)
    if opt == "sgd":
        ref = oracle.sgd_step(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], 0.05, pooling,
                              compute_dtype=torch.float32)
    else:
        ref, rs = oracle.exact_rowwise_adagrad_step(c["weights"], s0.cpu(), c["table_offsets"], c["indices"],
                                                    c["offsets"], c["grad"], 0.5, 0.2, pooling)
        torch.testing.assert_close(s1.cpu(), rs, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(w1.float().cpu(), ref.float(), **tol)


def test_backward_is_deterministic(cuda_device):
    c = to_device(make_case(T=4, E=30, D=128, B=256, Lmax=10, dtype=torch.float16, seed=9), cuda_device)
    a = _sgd(c, 0.1)
    for _ in range(3):
        assert torch.equal(a, _sgd(c, 0.1))


def test_strided_grad_output(cuda_device):
    """The all-to-all backward hands over a [B][T][D] view of a [T][B][D] buffer
    (sparse_embedding_cuda_ops.py:113-115); strides are honoured without a copy."""
    c = to_device(make_case(T=3, E=50, D=64, B=10, Lmax=6, dtype=torch.float32, seed=4), cuda_device)
    tbd = c["grad_d"].transpose(0, 1).contiguous()  # [T][B][D]
    view = tbd.transpose(0, 1)
    assert not view.is_contiguous()
    w1 = _sgd(c, 0.05, grad=view)
    ref = oracle.sgd_step(c["weights"], c["table_offsets"], c["indices"], c["offsets"], c["grad"], 0.05)
    assert_close(w1, ref, torch.float32)


def test_untouched_rows_are_bit_identical(cuda_device):
    c = to_device(make_case(T=2, E=1000, D=32, B=4, Lmax=3, dtype=torch.float16, seed=2), cuda_device)
    w1 = _sgd(c, 0.05)
    rows, _, starts = oracle.sort_segments(c["table_offsets"], c["indices"], c["offsets"])
    touched = torch.zeros(2000, dtype=torch.bool)
    touched[torch.from_numpy(rows[starts].astype(np.int64))] = True
    assert torch.equal(w1.cpu()[~touched], c["weights"][~touched])


def test_stochastic_rounding_is_unbiased_and_within_one_ulp(cuda_device):
    """fp16 stochastic rounding (table_batched_embeddings_cuda.cu:564-578) is not bit-comparable with
    any CPU oracle; check it brackets the exact value and is unbiased on average."""
    T, E, D, B = 1, 64, 128, 64
    c = to_device(make_case(T=T, E=E, D=D, B=B, Lmax=1, dtype=torch.float16, seed=8, fixed_L=1, unique=True), cuda_device)
    c["grad_d"] = (c["grad_d"] * 1e-3).contiguous()
    c["grad"] = c["grad_d"].cpu()
    s0 = torch.ones(E, device=cuda_device)
    exact_w, _ = oracle.exact_rowwise_adagrad_step(c["weights"].float(), s0.cpu(), c["table_offsets"], c["indices"],
                                                   c["offsets"], c["grad"].float(), 0.5, 0.2)
    acc = torch.zeros(E, D, dtype=torch.float64)
    trials = 64
    for _ in range(trials):
        w = c["weights_d"].clone()
        tbe.backward_exact_adagrad(c["grad_d"], w, c["table_offsets_d"], c["indices_d"], c["offsets_d"], None,
                                   s0.clone(), 0.5, 0.2, True, 1)
        wc = w.cpu().float()
        ulp = torch.maximum(exact_w.abs(), torch.tensor(2.0 ** -14)) * 2.0 ** -10
        assert torch.all((wc - exact_w).abs() <= ulp * 1.01 + 1e-7)
        acc += wc.double()
    bias = (acc / trials - exact_w.double()).abs().mean().item()
    rn_err = (c["weights"].float() - exact_w).abs().mean().item()
    assert bias < 0.5 * (2.0 ** -11) * exact_w.abs().mean().item() + 1e-6, (bias, rn_err)


@pytest.mark.parametrize("name", sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "tiny_*.npz"))))
def test_backward_golden(cuda_device, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    opt = str(z["optimizer"])
    if opt == "approx_rowwise_adagrad":
        pytest.skip("covered by test_gpu_approx.py")
    dtype = torch.float16 if str(z["dtype"]) == "fp16" else torch.float32
    T, E = int(z["T"]), int(z["E"])
    dev = cuda_device
    w = torch.from_numpy(z["weights"]).to(dtype).to(dev)
    go = torch.from_numpy(z["grad"]).to(dtype).to(dev)
    to = torch.tensor([t * E for t in range(T)], dtype=torch.int32, device=dev)
    idx, off = torch.from_numpy(z["indices"]).to(dev), torch.from_numpy(z["offsets"]).to(dev)
    rows, bags, starts = tbe.sort_segments(to, idx, off, T * E)
    assert np.array_equal(rows.cpu().numpy(), z["sorted_rows"])
    assert np.array_equal(bags.cpu().numpy(), z["sorted_bags"])
    assert np.array_equal(starts.cpu().numpy(), z["segment_starts"])
    if opt == "sgd":
        tbe.backward_sgd(go, w, to, idx, off, float(z["lr"]), 200, 1, False, pooling_mode=str(z["pooling"]))
    else:
        s = torch.from_numpy(z["state0"]).to(dev)
        tbe.backward_exact_adagrad(go, w, to, idx, off, None, s, float(z["lr"]), float(z["eps"]), False, 1,
                                   pooling_mode=str(z["pooling"]))
        torch.testing.assert_close(s.cpu(), torch.from_numpy(z["state_after"]), rtol=1e-3, atol=1e-4)
    assert_close(w, torch.from_numpy(z["weights_after"]), dtype)


def test_cfg1_forward_backward_sgd(cuda_device):
    """Config 1 end to end: T=4, E=10000, D=64 fp32, B=128, L=10, uniform indices, sum pooling,
    exact SGD lr=0.1, seed 0, against per-table EmbeddingBag on the CPU and the stored fixture."""
    z = np.load(os.path.join(GOLDEN, "cfg1.npz"))
    w = workloads.WORKLOADS["cfg1"]
    indices, offsets = workloads.make_inputs(w)
    weights = torch.from_numpy(workloads.make_weights(w))
    grad = torch.from_numpy(workloads.make_grad(w))
    to = [t * w.E for t in range(w.T)]
    dev = cuda_device
    wd = weights.to(dev)
    tod = torch.tensor(to, dtype=torch.int32, device=dev)
    idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
    out = tbe.forward(wd, tod, idx, off, None, 200, 4, False)
    tbe.backward_sgd(grad.to(dev), wd, tod, idx, off, w.lr, 200, 4, False)
    torch.testing.assert_close(out.cpu(), oracle.forward(weights, to, indices, offsets), rtol=1e-5, atol=1e-7)
    ref = oracle.sgd_step(weights, to, indices, offsets, grad, w.lr)
    torch.testing.assert_close(wd.cpu(), ref, rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(wd.cpu().double().view(w.T, -1).sum(dim=1).numpy(), z["weights_sum"], rtol=1e-7)
    np.testing.assert_allclose(wd.cpu()[torch.from_numpy(z["sample_rows"])].numpy(), z["sample_values"], rtol=1e-5,
                               atol=1e-7)


def test_workspace_too_small_is_reported(cuda_device):
    c = to_device(make_case(T=2, E=10, D=8, B=4, Lmax=3, dtype=torch.float32, seed=0, empty_bags=False), cuda_device)
    ws = torch.empty(256, dtype=torch.uint8, device=cuda_device)
    rc = _lib.lib().tbe_backward_sgd(c["grad_d"].data_ptr(), c["T"] * c["D"], c["D"], c["weights_d"].data_ptr(),
                                     c["table_offsets_d"].data_ptr(), c["indices_d"].data_ptr(),
                                     c["offsets_d"].data_ptr(), c["T"], c["B"], c["D"], c["N"], c["T"] * c["E"],
                                     _lib.TBE_F32, _lib.TBE_POOL_SUM, 0.1, 0, 0, ws.data_ptr(), ws.numel(), None)
    assert rc == -2 and b"workspace" in _lib.lib().tbe_last_error_string()


def test_full_size_target_step_properties(cuda_device):
    """The headline shapes at full size (T=64, E=1M, D=128 fp16, B=2048, L=38, fwd + exact SGD).
    Properties that do not need the oracle at this size: (1) run count from the device equals the
    host's unique count, sorted keys ascending; (2) only looked-up rows change; (3) a sample of
    updated rows equals w - lr * sum of their bags' gradients recomputed independently; (4) running
    the step with lr then -lr restores the weights to within fp16 rounding."""
    w = workloads.WORKLOADS["target"]
    dev = cuda_device
    indices, offsets = workloads.make_inputs(w)
    gen = torch.Generator(device=dev).manual_seed(0)
    weights = torch.empty(w.T * w.E, w.D, dtype=torch.float16, device=dev)
    for t in range(w.T):
        weights[t * w.E:(t + 1) * w.E] = (torch.rand(w.E, w.D, device=dev, generator=gen) * 0.02 - 0.01).half()
    grad = (torch.randn(w.B, w.T, w.D, device=dev, generator=gen) * 0.01).half()
    to = torch.arange(w.T, dtype=torch.int32, device=dev) * w.E
    idx, off = torch.from_numpy(indices).to(dev), torch.from_numpy(offsets).to(dev)
    # the table-segmented sort (the plan backward_sgd uses below) against the device radix sort
    rows, bags, starts = tbe.sort_segments(to, idx, off, w.T * w.E, max_rows_per_table=w.E)
    rows_r, bags_r, starts_r = tbe.sort_segments(to, idx, off, w.T * w.E)
    assert torch.equal(rows, rows_r) and torch.equal(bags, bags_r) and torch.equal(starts, starts_r)
    del rows_r, bags_r, starts_r
    assert starts.numel() == workloads.count_unique_rows(indices, offsets, w.T, w.B, w.E)
    assert bool((rows[1:] >= rows[:-1]).all())
    before = weights.clone()
    tbe.backward_sgd(grad, weights, to, idx, off, w.lr, 200, 2, False)
    touched = torch.zeros(w.T * w.E, dtype=torch.bool, device=dev)
    touched[rows[starts.long()].long()] = True
    for t in range(w.T):  # table by table to bound temporary memory
        sl = slice(t * w.E, (t + 1) * w.E)
        changed = (weights[sl] != before[sl]).any(dim=1)
        assert not bool((changed & ~touched[sl]).any())
    # (3) sampled runs
    starts_c, rows_c, bags_c = starts.cpu().numpy(), rows.cpu().numpy(), bags.cpu().numpy()
    rng = np.random.default_rng(0)
    for u in rng.integers(0, len(starts_c), size=64):
        s = starts_c[u]
        e = starts_c[u + 1] if u + 1 < len(starts_c) else len(rows_c)
        r = int(rows_c[s])
        g = torch.zeros(w.D, dtype=torch.float32, device=dev)
        for bag in bags_c[s:e]:
            t, b = divmod(int(bag), w.B)
            g += grad[b, t].float()
        expect = (before[r].float() - w.lr * g).half()
        torch.testing.assert_close(weights[r].float(), expect.float(), rtol=2e-3, atol=1e-5)
    # (4) round trip, compared table by table to bound temporary memory
    tbe.backward_sgd(grad, weights, to, idx, off, -w.lr, 200, 2, False)
    worst = 0.0
    for t in range(w.T):
        sl = slice(t * w.E, (t + 1) * w.E)
        worst = max(worst, (weights[sl].float() - before[sl].float()).abs().max().item())
    assert worst <= 2.0 ** -16
