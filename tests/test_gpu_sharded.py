"""Table-sharded TBE on 2 (or 4) GPUs: the fused peer-store exchange and the NCCL exchange against
the single-process oracle.  Needs at least two GPUs; child processes, one per GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import tbe_oracle as oracle

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_case(rank, Tl, E, D, B, Lmax, dtype):
    rng = np.random.default_rng(1000 + rank)
    lengths = rng.integers(0, Lmax + 1, size=(Tl, B))
    offsets = oracle.offsets_from_lengths(lengths)
    indices = rng.integers(0, E, size=int(offsets[-1])).astype(np.int32)
    weights = torch.from_numpy(rng.uniform(-1, 1, size=(Tl * E, D)).astype(np.float32)).to(dtype)
    return indices, offsets, weights


def _worker(rank, world, port, exchange, dtype_name, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sparse_ads_baselines_b200 import table_batched_embeddings_ops as ops
        from sparse_ads_baselines_b200.sharded import TableShardedEmbeddingBags
        dtype = torch.float16 if dtype_name == "fp16" else torch.float32
        Tl, E, D, B, Lmax, lr = 3, 50, 64, 8 * world, 5, 0.05
        cases = [_rank_case(r, Tl, E, D, B, Lmax, dtype) for r in range(world)]
        to = [t * E for t in range(Tl)]
        # oracle: every rank's local pooled rows, exchanged
        local = [oracle.forward(w, to, i, o, compute_dtype=torch.float32) for (i, o, w) in cases]
        expect_out = oracle.all_to_all_pooled(local)[rank]
        g = torch.Generator().manual_seed(7)
        grads = [torch.randn(B // world, Tl * world, D, generator=g).to(dtype) for _ in range(world)]
        grad_in = oracle.all_to_all_pooled_backward(grads)[rank]
        idx, off, w0 = cases[rank]
        expect_w = oracle.sgd_step(w0, to, idx, off, grad_in, lr, compute_dtype=torch.float32)

        m = TableShardedEmbeddingBags(Tl, E, D, B, optimizer=ops.Optimizer.SGD, learning_rate=lr,
                                      fp16=(dtype == torch.float16), exchange=exchange).to(dev)
        m.tbe.embedding_weights.data.copy_(w0.to(dev))
        idx_d, off_d = torch.from_numpy(idx).to(dev), torch.from_numpy(off).to(dev)
        tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
        for step in range(2):  # twice: buffers are reused across iterations
            m.tbe.embedding_weights.data.copy_(w0.to(dev))
            out = m(idx_d, off_d)
            assert tuple(out.shape) == (B // world, Tl * world, D)
            torch.testing.assert_close(out.detach().float().cpu(), expect_out.float(), **tol)
            out.backward(grads[rank].to(dev))
            torch.cuda.synchronize()
            torch.testing.assert_close(m.tbe.embedding_weights.detach().float().cpu(), expect_w.float(), **tol)
        # Two forwards in a row (an evaluation loop, or micro-batches before a backward): the first
        # output must still hold when the second has been produced -- peers write the other buffer --
        # and two backwards in a row must each see their own incoming gradient.
        cases2 = [_rank_case(100 + r, Tl, E, D, B, Lmax, dtype) for r in range(world)]
        local2 = [oracle.forward(w0_, to, i, o, compute_dtype=torch.float32) for (i, o, _), (_, _, w0_) in zip(cases2, cases)]
        expect_out2 = oracle.all_to_all_pooled(local2)[rank]
        idx2_d, off2_d = torch.from_numpy(cases2[rank][0]).to(dev), torch.from_numpy(cases2[rank][1]).to(dev)
        m.tbe.embedding_weights.data.copy_(w0.to(dev))
        out1 = m(idx_d, off_d)
        out2 = m(idx2_d, off2_d)
        torch.cuda.synchronize()
        dist.barrier()  # every rank's second forward has landed
        torch.testing.assert_close(out1.detach().float().cpu(), expect_out.float(), **tol)
        torch.testing.assert_close(out2.detach().float().cpu(), expect_out2.float(), **tol)
        out2.backward(grads[rank].to(dev))
        out1.backward(grads[rank].to(dev))
        torch.cuda.synchronize()
        w_mid = oracle.sgd_step(w0, to, cases2[rank][0], cases2[rank][1], grad_in, lr, compute_dtype=torch.float32)
        expect_w2 = oracle.sgd_step(w_mid, to, idx, off, grad_in, lr, compute_dtype=torch.float32)
        torch.testing.assert_close(m.tbe.embedding_weights.detach().float().cpu(), expect_w2.float(), **tol)
        with torch.no_grad():  # forward-only loop
            for _ in range(3):
                o = m(idx_d, off_d)
        m.check_exchange()
        # row-wise sharding on the same ranks: every rank holds E rows of each of Tl tables and looks
        # up the global batch with indices local to its slice; reduce-scatter forward, all-gather backward
        from sparse_ads_baselines_b200.sharded import RowShardedEmbeddingBags
        rcases = [_rank_case(500 + r, Tl, E, D, B, Lmax, dtype) for r in range(world)]
        partial = [oracle.forward(w_, to, i_, o_, compute_dtype=torch.float32) for (i_, o_, w_) in rcases]
        r_expect = oracle.reduce_scatter_pooled(partial)[rank]
        g3 = torch.Generator().manual_seed(70)
        rgrads = [torch.randn(B // world, Tl, D, generator=g3).to(dtype) for _ in range(world)]
        r_gin = oracle.all_gather_pooled_backward(rgrads)[rank]
        ridx, roff, rw0 = rcases[rank]
        r_expect_w = oracle.sgd_step(rw0, to, ridx, roff, r_gin, lr, compute_dtype=torch.float32)
        rm = RowShardedEmbeddingBags(Tl, E, D, B, optimizer=ops.Optimizer.SGD, learning_rate=lr,
                                     fp16=(dtype == torch.float16), exchange=exchange).to(dev)
        ridx_d, roff_d = torch.from_numpy(ridx).to(dev), torch.from_numpy(roff).to(dev)
        for step in range(2):
            rm.tbe.embedding_weights.data.copy_(rw0.to(dev))
            rout = rm(ridx_d, roff_d)
            assert tuple(rout.shape) == (B // world, Tl, D)
            torch.testing.assert_close(rout.detach().float().cpu(), r_expect.float(), **tol)
            rout.backward(rgrads[rank].to(dev))
            torch.cuda.synchronize()
            torch.testing.assert_close(rm.tbe.embedding_weights.detach().float().cpu(), r_expect_w.float(), **tol)
        rm.check_exchange()
        if exchange == "fused" and dtype_name == "fp32":
            # the index all-to-all in front of the lookup: data-parallel features in, my tables' out
            from sparse_ads_baselines_b200 import input_pipeline
            T_all, Bl_ = Tl * world, B // world
            feats = []
            for r in range(world):
                rng = np.random.default_rng(800 + r)
                lens = rng.integers(0, Lmax + 1, size=T_all * Bl_)
                off_r = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
                feats.append((rng.integers(0, E, size=int(off_r[-1])).astype(np.int32), off_r))
            got_idx, got_off = input_pipeline.indices_all_to_all(torch.from_numpy(feats[rank][0]).to(dev),
                                                                 torch.from_numpy(feats[rank][1]).to(dev), T_all)
            want_idx, want_off = oracle.index_all_to_all([f[0] for f in feats], [f[1] for f in feats], T_all)[rank]
            assert np.array_equal(got_off.cpu().numpy(), want_off) and np.array_equal(got_idx.cpu().numpy(), want_idx)
            out_p = m(got_idx, got_off)  # and the exchanged features drive the sharded lookup
            assert tuple(out_p.shape) == (B // world, Tl * world, D)
        if exchange == "nccl" and dtype_name == "fp32":
            # row-wise sharding collectives, after test_sparse_embedding_cuda.py:138-171: the same seed
            # on every rank regenerates every rank's tensor
            from sparse_ads_baselines_b200 import sparse_embedding_cuda_ops as se_ops
            for (b, t, d) in [(world, 1, 1), (2 * world, 8, 7), (4 * world, 3, 284)]:
                g2 = torch.Generator().manual_seed(42)
                parts = [torch.randn(b, t, d, generator=g2) for _ in range(world)]
                x = parts[rank].to(dev).requires_grad_(True)
                y = se_ops.ReduceScatterFunction.apply(x)
                bl = b // world
                torch.testing.assert_close(y.detach().cpu(), sum(parts)[rank * bl:(rank + 1) * bl], rtol=1e-5, atol=1e-5)
                gy = [torch.randn(bl, t, d, generator=g2) for _ in range(world)]
                y.backward(gy[rank].to(dev))
                torch.testing.assert_close(x.grad.cpu(), torch.cat(gy, dim=0), rtol=0, atol=0)
    except Exception as e:
        failures.put("rank %d: %r" % (rank, e))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "fused"])
@pytest.mark.parametrize("dtype_name", ["fp32", "fp16"])
def test_sharded_forward_backward(exchange, dtype_name):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, exchange, dtype_name, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not hung, "a rank did not finish: %s" % msgs
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs)


def _absent_rank_worker(rank, world, port, failures):
    """Rank 1 stays away from the second forward (a failure made on the host: it simply does not
    call).  Rank 0's bounded wait must run out and be reported by check_exchange; rank 1 keeps its
    process and buffers alive until rank 0 is done, so nothing ever touches freed peer memory."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    host_group = dist.new_group(backend="gloo")  # the ranks meet on the host at the end
    try:
        from sparse_ads_baselines_b200 import _lib
        from sparse_ads_baselines_b200.sharded import TableShardedEmbeddingBags
        Tl, E, D, B = 2, 50, 32, 8
        idx, off, _ = _rank_case(rank, Tl, E, D, B, 4, torch.float32)
        idx_d, off_d = torch.from_numpy(idx).to(dev), torch.from_numpy(off).to(dev)
        m = TableShardedEmbeddingBags(Tl, E, D, B, exchange="fused", sync_timeout_s=1.0).to(dev)
        with torch.no_grad():
            m(idx_d, off_d)
            m.check_exchange()  # the first step completes on both ranks
            if rank == 0:
                m(idx_d, off_d)  # rank 1 never launches this step
                try:
                    m.check_exchange()
                    failures.put("rank 0: the missing rank went unnoticed")
                except _lib.TBEError as e:
                    if e.status != -6 or "rank 1" not in str(e):
                        failures.put("rank 0: unexpected error %r" % e)
                assert torch.arange(4, device=dev).sum().item() == 6  # the context survived
        dist.barrier(group=host_group)
    except Exception as e:
        failures.put("rank %d: %r" % (rank, e))
    finally:
        dist.destroy_process_group()


def test_absent_rank_is_reported_not_waited_for():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not hung, "a rank did not finish: %s" % msgs
    assert not msgs, msgs
