"""The fused table-sharded exchange checked on ONE GPU through the C ABI.

``tbe_forward_sharded`` and ``tbe_all2all_push`` take one destination pointer per rank; nothing in
them cares whether a pointer is peer-mapped.  Here every emulated rank's buffers live on the same
device, the ranks' calls run one after the other on one stream, and every destination is compared
with the layout contract of the reference's all-to-all (forward_all2all_nccl,
sparse_embedding_cuda.cpp:471-533: out_j[b', r*T/W + t] = in_r[j*B/W + b', t]; backward
All2AllFunction.backward, sparse_embedding_cuda_ops.py:104-117) -- bit for bit against the
unsharded kernel's own pooled rows (the exchange is a copy), and within tolerance against the oracle.
The last test runs a whole table-sharded SGD step the way sharded.py wires it (plan on a side
stream, gradient pushed into the owners' buffers, fused backward) against the oracle.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import _lib

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-5, atol=1e-5), torch.float16: dict(rtol=1e-2, atol=1e-2)}


def _rank_case(rank, Tl, E, D, B, Lmax, dtype):
    rng = np.random.default_rng(4000 + rank)
    lengths = rng.integers(0, Lmax + 1, size=(Tl, B))
    offsets = oracle.offsets_from_lengths(lengths)
    indices = rng.integers(0, E, size=int(offsets[-1])).astype(np.int32)
    weights = torch.from_numpy(rng.uniform(-1, 1, size=(Tl * E, D)).astype(np.float32)).to(dtype)
    return indices, offsets, weights


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _dt(dtype):
    return _lib.TBE_F16 if dtype == torch.float16 else _lib.TBE_F32


def _sharded_forward(dev, cases, world, Tl, E, D, B, dtype, pooling=_lib.TBE_POOL_SUM):
    """Runs every emulated rank's tbe_forward_sharded into `world` local buffers; also returns the
    unsharded kernel's [B][Tl][D] rows per rank."""
    Bl = B // world
    outs = [torch.full((Bl, Tl * world, D), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    to = (torch.arange(Tl, dtype=torch.int32) * E).to(dev)
    local = []
    for r, (idx, off, w) in enumerate(cases):
        wd, idx_d, off_d = w.to(dev), torch.from_numpy(idx).to(dev), torch.from_numpy(off).to(dev)
        _lib.call("tbe_forward_sharded", wd.data_ptr(), to.data_ptr(), idx_d.data_ptr(), off_d.data_ptr(), None,
                  _ptrs(outs), world, Tl, B, D, Tl * world, Tl * r, _dt(dtype), pooling, _stream(dev))
        plain = torch.empty(B, Tl, D, dtype=dtype, device=dev)
        _lib.call("tbe_forward", wd.data_ptr(), to.data_ptr(), idx_d.data_ptr(), off_d.data_ptr(), None,
                  plain.data_ptr(), Tl, B, D, _dt(dtype), pooling, _stream(dev))
        local.append(plain)
    torch.cuda.synchronize()
    return outs, local


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.float16, 128), (torch.float16, 36)])
def test_forward_sharded_layout(cuda_device, world, dtype, D):
    Tl, E, B, Lmax = 3, 50, 4 * world, 6
    cases = [_rank_case(r, Tl, E, D, B, Lmax, dtype) for r in range(world)]
    outs, local = _sharded_forward(cuda_device, cases, world, Tl, E, D, B, dtype)
    expect_copy = oracle.all_to_all_pooled([x.cpu() for x in local])
    to = [t * E for t in range(Tl)]
    expect = oracle.all_to_all_pooled([oracle.forward(w, to, i, o, compute_dtype=torch.float32) for (i, o, w) in cases])
    for j in range(world):
        got = outs[j].cpu()
        assert not torch.isnan(got.float()).any(), "a destination element was never written"
        assert torch.equal(got, expect_copy[j]), "rank %d's buffer is not the exchanged copy" % j
        torch.testing.assert_close(got.float(), expect[j].float(), **TOL[dtype])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.float16, 128), (torch.float16, 36)])
def test_all2all_push_layout(cuda_device, world, dtype, D):
    dev = cuda_device
    Tl, Bl = 3, 5
    g = torch.Generator().manual_seed(world)
    grads = [torch.randn(Bl, Tl * world, D, generator=g).to(dtype) for _ in range(world)]
    dsts = [torch.full((Bl * world, Tl, D), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    for j in range(world):
        src = grads[j].to(dev)
        _lib.call("tbe_all2all_push", src.data_ptr(), _ptrs(dsts), world, j, Bl, Tl * D * src.element_size(), _stream(dev))
    torch.cuda.synchronize()
    expect = oracle.all_to_all_pooled_backward(grads)
    for r in range(world):
        assert torch.equal(dsts[r].cpu(), expect[r]), "rank %d's incoming gradient is not the exchanged copy" % r


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_sharded_sgd_step_one_gpu(cuda_device, world, dtype):
    dev = cuda_device
    lib = _lib.lib()
    Tl, E, D, B, Lmax, lr = 3, 60, 64, 8 * world, 7, 0.05
    Bl = B // world
    cases = [_rank_case(r, Tl, E, D, B, Lmax, dtype) for r in range(world)]
    outs, _ = _sharded_forward(dev, cases, world, Tl, E, D, B, dtype)
    to_h = [t * E for t in range(Tl)]
    expect_out = oracle.all_to_all_pooled([oracle.forward(w, to_h, i, o, compute_dtype=torch.float32) for (i, o, w) in cases])
    for j in range(world):
        torch.testing.assert_close(outs[j].cpu().float(), expect_out[j].float(), **TOL[dtype])
    g = torch.Generator().manual_seed(11)
    grads = [torch.randn(Bl, Tl * world, D, generator=g).to(dtype) for _ in range(world)]
    grad_in = [torch.empty(B, Tl, D, dtype=dtype, device=dev) for _ in range(world)]
    # every rank's plan starts on a side stream while the pushes run on the main one, as in sharded.py
    to = (torch.arange(Tl, dtype=torch.int32) * E).to(dev)
    side = torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    dev_cases, plans = [], []
    for r, (idx, off, w) in enumerate(cases):
        wd, idx_d, off_d = w.to(dev).clone(), torch.from_numpy(idx).to(dev), torch.from_numpy(off).to(dev)
        nbytes = lib.tbe_backward_workspace_bytes(idx_d.numel(), Tl * E)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        dev_cases.append((wd, idx_d, off_d, ws, nbytes))
    side.wait_stream(main)
    for (wd, idx_d, off_d, ws, nbytes) in dev_cases:
        _lib.call("tbe_backward_plan", to.data_ptr(), idx_d.data_ptr(), off_d.data_ptr(), Tl, B, idx_d.numel(), Tl * E, E,
                  ws.data_ptr(), nbytes, ctypes.c_void_p(side.cuda_stream))
    done = torch.cuda.Event()
    done.record(side)
    for j in range(world):
        src = grads[j].to(dev)
        _lib.call("tbe_all2all_push", src.data_ptr(), _ptrs(grad_in), world, j, Bl, Tl * D * src.element_size(), _stream(dev))
    main.wait_event(done)
    for r, (wd, idx_d, off_d, ws, nbytes) in enumerate(dev_cases):
        _lib.call("tbe_backward_sgd", grad_in[r].data_ptr(), Tl * D, D, wd.data_ptr(), to.data_ptr(), idx_d.data_ptr(),
                  off_d.data_ptr(), Tl, B, D, idx_d.numel(), Tl * E, _dt(dtype), _lib.TBE_POOL_SUM, lr, E, 1,
                  ws.data_ptr(), nbytes, _stream(dev))
    torch.cuda.synchronize()
    expect_gin = oracle.all_to_all_pooled_backward(grads)
    for r, (idx, off, w) in enumerate(cases):
        assert torch.equal(grad_in[r].cpu(), expect_gin[r])
        expect_w = oracle.sgd_step(w, to_h, idx, off, expect_gin[r], lr, compute_dtype=torch.float32)
        torch.testing.assert_close(dev_cases[r][0].cpu().float(), expect_w.float(), **TOL[dtype])


def test_nccl_path_transposed_gradient_view(cuda_device):
    """The NCCL exchange hands the backward a transposed view ([W][B/W][Tl][D] seen as [B][Tl][D] is
    contiguous, but the reference's layout before its transpose copy is [B/W][W*Tl][D]): the backward
    takes any (stride_b, stride_t), so a column block of a wider gradient needs no copy."""
    dev = cuda_device
    Tl, E, D, B, lr, world = 2, 40, 32, 12, 0.1, 3
    idx, off, w = _rank_case(0, Tl, E, D, B, 5, torch.float32)
    wide = torch.randn(B, Tl * world, D, generator=torch.Generator().manual_seed(5))
    r = 1
    view = wide[:, r * Tl:(r + 1) * Tl]  # [B][Tl][D] with stride_b = world*Tl*D
    wd, idx_d, off_d, wide_d = w.to(dev).clone(), torch.from_numpy(idx).to(dev), torch.from_numpy(off).to(dev), wide.to(dev)
    to = (torch.arange(Tl, dtype=torch.int32) * E).to(dev)
    nbytes = _lib.lib().tbe_backward_workspace_bytes(idx_d.numel(), Tl * E)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.call("tbe_backward_sgd", wide_d.data_ptr() + r * Tl * D * 4, world * Tl * D, D, wd.data_ptr(), to.data_ptr(),
              idx_d.data_ptr(), off_d.data_ptr(), Tl, B, D, idx_d.numel(), Tl * E, _lib.TBE_F32, _lib.TBE_POOL_SUM, lr, E,
              0, ws.data_ptr(), nbytes, _stream(dev))
    torch.cuda.synchronize()
    expect = oracle.sgd_step(w, [0, E], idx, off, view.contiguous(), lr)
    torch.testing.assert_close(wd.cpu(), expect, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_row_sharded_exchange_one_gpu(cuda_device, world, dtype):
    """Row-wise sharding: every emulated rank looks up the global batch over its own row slice and
    stores the partial rows into slot `rank` of the owners' staging buffers (tbe_forward_sharded with
    advanced pointers); tbe_reduce_slots sums the slots; tbe_allgather_push gathers the gradient."""
    dev = cuda_device
    T, E, D, Bl, Lmax = 3, 40, 64, 4, 6
    B = Bl * world
    cases = [_rank_case(50 + r, T, E, D, B, Lmax, dtype) for r in range(world)]  # (indices, offsets, row slice)
    es = 2 if dtype == torch.float16 else 4
    stage = [torch.full((world, Bl, T, D), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    to = (torch.arange(T, dtype=torch.int32) * E).to(dev)
    for r, (idx, off, w) in enumerate(cases):
        wd, idx_d, off_d = w.to(dev), torch.from_numpy(idx).to(dev), torch.from_numpy(off).to(dev)
        dst = (ctypes.c_void_p * world)(*[s_.data_ptr() + r * Bl * T * D * es for s_ in stage])
        _lib.call("tbe_forward_sharded", wd.data_ptr(), to.data_ptr(), idx_d.data_ptr(), off_d.data_ptr(), None, dst,
                  world, T, B, D, T, 0, _dt(dtype), _lib.TBE_POOL_SUM, _stream(dev))
    outs = []
    for j in range(world):
        out = torch.empty(Bl, T, D, dtype=dtype, device=dev)
        _lib.call("tbe_reduce_slots", stage[j].data_ptr(), out.data_ptr(), world, Bl * T * D, _dt(dtype), _stream(dev))
        outs.append(out)
    torch.cuda.synchronize()
    to_h = [t * E for t in range(T)]
    partial = [oracle.forward(w, to_h, i, o, compute_dtype=torch.float32) for (i, o, w) in cases]
    expect = oracle.reduce_scatter_pooled(partial)
    for j in range(world):
        assert not torch.isnan(stage[j].float()).any()
        torch.testing.assert_close(outs[j].cpu().float(), expect[j].float(), **TOL[dtype])
    # the gradient slices, gathered on every rank
    g = torch.Generator().manual_seed(9)
    grads = [torch.randn(Bl, T, D, generator=g).to(dtype) for _ in range(world)]
    gathered = [torch.full((B, T, D), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    for j in range(world):
        src = grads[j].to(dev)
        _lib.call("tbe_allgather_push", src.data_ptr(), _ptrs(gathered), world, j, src.numel() * es, _stream(dev))
    torch.cuda.synchronize()
    expect_g = oracle.all_gather_pooled_backward(grads)
    for r in range(world):
        assert torch.equal(gathered[r].cpu(), expect_g[r])


@pytest.mark.parametrize("world,Tl,Bl,Lmax", [(2, 3, 4, 5), (4, 1, 7, 40), (8, 2, 3, 0), (3, 5, 64, 70)])
def test_regroup_bags_matches_oracle(cuda_device, world, Tl, Bl, Lmax):
    """Phase 3 of the index all-to-all: the [W][T/W][B/W] bags a rank received, regrouped to
    [T/W][B] order by tbe_permute_bags, equal the oracle's index all-to-all for that rank."""
    from sparse_ads_baselines_b200 import input_pipeline
    T = Tl * world
    feats = []
    for r in range(world):
        rng = np.random.default_rng(700 + r)
        lens = rng.integers(0, Lmax + 1, size=T * Bl)
        off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        feats.append((rng.integers(0, 10 ** 6, size=int(off[-1])).astype(np.int32), off))
    want = oracle.index_all_to_all([f[0] for f in feats], [f[1] for f in feats], T)
    for r in range(world):
        # what rank r receives: from every rank j, the [Tl][Bl] bags of r's tables, table-major
        blocks, lens = [], []
        for j in range(world):
            off = feats[j][1].astype(np.int64)
            lo, hi = off[r * Tl * Bl], off[(r + 1) * Tl * Bl]
            blocks.append(feats[j][0][lo:hi])
            lens.append(np.diff(off[r * Tl * Bl:(r + 1) * Tl * Bl + 1]))
        recv_idx = torch.from_numpy(np.concatenate(blocks).astype(np.int32)).to(cuda_device)
        recv_len = torch.from_numpy(np.stack(lens).astype(np.int32).reshape(world, Tl, Bl)).to(cuda_device)
        idx, off = input_pipeline.regroup_bags(recv_idx, recv_len)
        assert np.array_equal(off.cpu().numpy(), want[r][1])
        assert np.array_equal(idx.cpu().numpy(), want[r][0])
