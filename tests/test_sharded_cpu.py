"""Host logic of the table-sharded exchange on CPU ranks (gloo, world size 2 and 4): the library
all-to-all path of sharded.py against the layout contract of forward_all2all_nccl
(sparse_embedding_cuda.cpp:471-533) restated in the oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tbe_oracle as oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_inputs(rank, B, Tl, D):
    # every rank can regenerate every rank's tensor (the reference's same-seed trick,
    # test_sparse_embedding_cuda.py:145-150)
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randn(B, Tl, D, generator=g)


def _worker(rank, world, port, B, Tl, D, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparse_ads_baselines_b200 import sharded
        ins = [_rank_inputs(r, B, Tl, D) for r in range(world)]
        expect = oracle.all_to_all_pooled(ins)[rank]
        got = sharded.pooled_all_to_all(ins[rank])
        assert got.shape == (B // world, Tl * world, D)
        assert torch.equal(got, expect), "forward exchange layout"
        # backward: every rank holds a gradient for its batch slice over all tables
        grads = [_rank_inputs(50 + r, B // world, Tl * world, D) for r in range(world)]
        expect_b = oracle.all_to_all_pooled_backward(grads)[rank]
        got_b = sharded.pooled_all_to_all_backward(grads[rank])
        assert got_b.shape == (B, Tl, D)
        assert torch.equal(got_b, expect_b), "backward exchange layout"
        # autograd wiring: d(sum(out * g)) / d(in) is the backward exchange of g
        x = ins[rank].clone().requires_grad_(True)
        y = sharded._NcclExchange.apply(x, None)
        y.backward(grads[rank])
        assert torch.equal(x.grad, expect_b), "autograd of the exchange"
        # row-wise sharding: reduce-scatter forward, all-gather backward (test_sparse_embedding_cuda.py:138-171)
        parts = [_rank_inputs(200 + r, B, Tl, D) for r in range(world)]
        xr = parts[rank].clone().requires_grad_(True)
        yr = sharded._NcclRowExchange.apply(xr, None)
        torch.testing.assert_close(yr.detach(), oracle.reduce_scatter_pooled(parts)[rank], rtol=1e-6, atol=1e-6)
        gr = [_rank_inputs(300 + r, B // world, Tl, D) for r in range(world)]
        yr.backward(gr[rank])
        assert torch.equal(xr.grad, oracle.all_gather_pooled_backward(gr)[rank]), "all-gather of the gradient"
        # index all-to-all (phases 1-2 on CPU tensors): data-parallel features -> my tables' features
        import numpy as np
        from sparse_ads_baselines_b200 import input_pipeline
        T_all, Bl_, Lmax = 2 * world, 3, 4
        feats = []
        for r in range(world):
            rng = np.random.default_rng(900 + r)
            lens = rng.integers(0, Lmax + 1, size=T_all * Bl_)
            off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            feats.append((rng.integers(0, 1000, size=int(off[-1])).astype(np.int32), off))
        recv_idx, recv_len = input_pipeline.exchange_indices(torch.from_numpy(feats[rank][0]), torch.from_numpy(feats[rank][1]),
                                                              T_all)
        Tl_ = T_all // world
        assert tuple(recv_len.shape) == (world, Tl_, Bl_)
        # regroup on the host the way tbe_permute_bags does on the device
        src_off = np.concatenate([[0], np.cumsum(recv_len.numpy().reshape(-1))])
        pieces, lens_out = [], []
        for t in range(Tl_):
            for j in range(world):
                for b in range(Bl_):
                    sb = (j * Tl_ + t) * Bl_ + b
                    pieces.append(recv_idx.numpy()[src_off[sb]:src_off[sb + 1]])
                    lens_out.append(src_off[sb + 1] - src_off[sb])
        want_idx, want_off = oracle.index_all_to_all([f[0] for f in feats], [f[1] for f in feats], T_all)[rank]
        assert np.array_equal(np.concatenate(pieces) if pieces else np.zeros(0), want_idx), "index all-to-all"
        assert np.array_equal(np.concatenate([[0], np.cumsum(lens_out)]), want_off), "offsets after the index all-to-all"
        # B not divisible by the world size is refused (sparse_embedding_cuda.cpp:500)
        try:
            sharded.pooled_all_to_all(torch.zeros(B + 1, Tl, D))
        except AssertionError:
            pass
        else:
            raise AssertionError("indivisible batch accepted")
    except Exception as e:  # report instead of hanging the other ranks
        failures.put("rank %d: %r" % (rank, e))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B,Tl,D", [(2, 8, 3, 4), (4, 8, 2, 6), (2, 2, 1, 1)])
def test_exchange_layout_on_gloo_ranks(world, B, Tl, D):
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, Tl, D, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    assert not hung, "a rank did not finish"
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)


def test_world_size_one_is_identity():
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(_free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        from sparse_ads_baselines_b200 import sharded
        x = torch.randn(4, 3, 2)
        # every collective is an identity at world size 1 (sparse_embedding_cuda.cpp:492-494)
        assert sharded.pooled_all_to_all(x) is x
        assert sharded.pooled_all_to_all_backward(x) is x
    finally:
        dist.destroy_process_group()
