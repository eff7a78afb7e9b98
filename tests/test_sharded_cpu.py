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
