"""The allocation-free SGD backward (tbe_backward_sgd_noalloc), called through the C ABI.

Some users of libtbe_b200.so cannot give the backward a scratch buffer because they cannot allocate
device memory: an FFI host without a device allocator, or a serving process that may not call
cudaMalloc while it handles requests.  For them the library carries its own fixed scratch array.
This file checks that entry point against tbe_backward_sgd (caller-owned workspace) and against the
CPU oracle on the same inputs, twice in a row -- the second call finds the first call's leftovers
in the shared array -- that batches above the documented limit are refused, and that a batch of
exactly the limit fits the built-in array.  The file name keeps it last in
collection order, so a run that stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import _lib

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-5, atol=1e-6), torch.float16: dict(rtol=1e-2, atol=1e-2)}


def _inputs(device, dtype, T, E, D, B, Lmax, seed):
    rng = np.random.default_rng(seed)
    lengths = rng.integers(0, Lmax + 1, size=T * B)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    indices = rng.integers(0, E, size=int(offsets[-1])).astype(np.int32)  # E small: rows repeat
    weights = torch.from_numpy(rng.uniform(-1, 1, size=(T * E, D)).astype(np.float32)).to(dtype).to(device)
    grad = torch.from_numpy(rng.standard_normal(size=(B, T, D)).astype(np.float32)).to(dtype).to(device)
    table_offsets = (torch.arange(T, dtype=torch.int32) * E).to(device)
    return weights, grad, table_offsets, torch.from_numpy(indices).to(device), torch.from_numpy(offsets).to(device)


def _with_workspace(lib, weights, grad, to, idx, off, T, E, D, B, dt, lr, stream):
    w = weights.clone()
    nbytes = lib.tbe_backward_workspace_bytes(idx.numel(), T * E)
    assert nbytes > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    rc = lib.tbe_backward_sgd(grad.data_ptr(), T * D, D, w.data_ptr(), to.data_ptr(), idx.data_ptr(), off.data_ptr(),
                              T, B, D, idx.numel(), T * E, dt, _lib.TBE_POOL_SUM, lr, E, 0, ws.data_ptr(), nbytes,
                              stream)
    assert rc == 0, lib.tbe_last_error_string()
    return w


def _without_allocation(lib, weights, grad, to, idx, off, T, E, D, B, dt, lr, stream):
    w = weights.clone()
    rc = lib.tbe_backward_sgd_noalloc(grad.data_ptr(), T * D, D, w.data_ptr(), to.data_ptr(), idx.data_ptr(),
                                      off.data_ptr(), T, B, D, idx.numel(), T * E, dt, _lib.TBE_POOL_SUM, lr, E,
                                      stream)
    assert rc == 0, lib.tbe_last_error_string()
    return w


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_noalloc_matches_workspace_entry_point_twice(cuda_device, dtype):
    lib = _lib.lib()
    assert lib.tbe_noalloc_scratch_bytes() >= 1 << 20
    dt = _lib.TBE_F16 if dtype == torch.float16 else _lib.TBE_F32
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    # two different batches back to back: the second call runs on top of the first call's scratch
    for seed, (T, E, D, B, Lmax) in enumerate([(3, 40, 64, 33, 12), (5, 7, 128, 64, 40)]):
        weights, grad, to, idx, off = _inputs(cuda_device, dtype, T, E, D, B, Lmax, seed)
        expect = _with_workspace(lib, weights, grad, to, idx, off, T, E, D, B, dt, 0.05, stream)
        got = _without_allocation(lib, weights, grad, to, idx, off, T, E, D, B, dt, 0.05, stream)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float().cpu(), expect.float().cpu(), **TOL[dtype])
        assert torch.equal(got, expect)  # same kernels, same order of summation: the same bits
        assert not torch.equal(got, weights)  # the update really happened
        # and both agree with the oracle: w - lr * dense gradient, repeated rows summed
        ref = oracle.sgd_step(weights.cpu(), [t * E for t in range(T)], idx.cpu().numpy(), off.cpu().numpy(),
                              grad.cpu(), 0.05, compute_dtype=torch.float32)
        # (each row here sums ~100 gradient rows in another order than the oracle: absolute 1e-5)
        torch.testing.assert_close(got.float().cpu(), ref.float(), rtol=TOL[dtype]["rtol"], atol=max(TOL[dtype]["atol"], 1e-5))


def test_noalloc_limit_fits_the_builtin_array(cuda_device):
    """A batch of exactly TBE_NOALLOC_MAX_LOOKUPS lookups must fit the fixed array (the scratch size
    depends on the sort library's temporary storage), and runs."""
    lib = _lib.lib()
    limit = 524288
    T, E, D, B = 4, 50_000, 32, 1024
    L = limit // (T * B)
    assert T * B * L == limit
    assert 0 < lib.tbe_backward_workspace_bytes(limit, T * E) <= lib.tbe_noalloc_scratch_bytes()
    rng = np.random.default_rng(3)
    indices = rng.integers(0, E, size=limit).astype(np.int32)
    offsets = (np.arange(T * B + 1, dtype=np.int64) * L).astype(np.int32)
    weights = torch.from_numpy(rng.uniform(-1, 1, size=(T * E, D)).astype(np.float32)).to(cuda_device)
    grad = torch.from_numpy(rng.standard_normal(size=(B, T, D)).astype(np.float32)).to(cuda_device)
    to = (torch.arange(T, dtype=torch.int32) * E).to(cuda_device)
    idx, off = torch.from_numpy(indices).to(cuda_device), torch.from_numpy(offsets).to(cuda_device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    got = _without_allocation(lib, weights, grad, to, idx, off, T, E, D, B, _lib.TBE_F32, 0.05, stream)
    torch.cuda.synchronize()
    ref = oracle.sgd_step(weights.cpu(), [t * E for t in range(T)], indices, offsets, grad.cpu(), 0.05)
    torch.testing.assert_close(got.cpu(), ref, rtol=1e-5, atol=1e-5)


def test_noalloc_rejects_batches_above_the_limit(cuda_device):
    lib = _lib.lib()
    buf = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    p = buf.data_ptr()
    too_many = 524288 + 1
    rc = lib.tbe_backward_sgd_noalloc(p, 4, 4, p, p, p, p, 1, 1, 4, too_many, 16, _lib.TBE_F32, _lib.TBE_POOL_SUM, 0.1,
                                      0, None)
    assert rc == -2
    msg = lib.tbe_last_error_string().decode()
    assert "524288" in msg and "limit" in msg
