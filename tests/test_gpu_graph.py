"""The library's calls inside a CUDA graph.

Every entry point enqueues kernels (and a few memsets / device-to-device copies) on the caller's
stream and never synchronises, so a forward + backward step can be captured once and replayed: the
launch-bound regime (config 1: T=4, B=128 -- a step is 7 kernels of a few microseconds) then costs
one graph launch instead of seven kernel launches plus the Python around them.  A replay reads the
CURRENT contents of the captured buffers: new indices of the same count go into the same tensors.
"""
import numpy as np
import pytest
import torch

from oracle import tbe_oracle as oracle
from sparse_ads_baselines_b200 import table_batched_embeddings as tbe
from tbe_testlib import make_case, to_device, assert_close

pytestmark = pytest.mark.gpu


def _fresh_indices(c, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, c["E"], size=c["N"]).astype(np.int32)


@pytest.mark.parametrize("optimizer", ["sgd", "exact_rowwise_adagrad"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_captured_step_replays_on_new_indices(cuda_device, optimizer, dtype):
    dev = cuda_device
    c = to_device(make_case(T=4, E=10_000, D=64, B=128, Lmax=0, dtype=dtype, seed=5, fixed_L=10), dev)
    w = c["weights_d"].clone()
    state = torch.full((c["T"] * c["E"],), 0.25, device=dev)
    idx, off, to, go = c["indices_d"].clone(), c["offsets_d"], c["table_offsets_d"], c["grad_d"]
    out = torch.empty(c["B"], c["T"], c["D"], dtype=dtype, device=dev)

    def step():
        tbe.forward(w, to, idx, off, None, 10, 1, False, out=out)
        if optimizer == "sgd":
            tbe.backward_sgd(go, w, to, idx, off, 0.05, 10, 1, False)
        else:
            tbe.backward_exact_adagrad(go, w, to, idx, off, None, state, 0.05, 0.1, False, 1)

    # warm up on a side stream (workspace allocation, cached host copies of the small tensors), then
    # undo its effect so that the oracle below starts from the same tables
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    w.copy_(c["weights_d"])
    state.fill_(0.25)

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    torch.cuda.synchronize(dev)
    w.copy_(c["weights_d"])  # (capturing does not run the kernels, but be explicit)
    state.fill_(0.25)

    w_ref, s_ref = c["weights"].clone(), torch.full((c["T"] * c["E"],), 0.25)
    for r in range(3):
        new_idx = _fresh_indices(c, 100 + r)
        idx.copy_(torch.from_numpy(new_idx).to(dev))
        graph.replay()
        torch.cuda.synchronize(dev)
        ref_out = oracle.forward(w_ref, c["table_offsets"], new_idx, c["offsets"], None, "sum", compute_dtype=torch.float32)
        assert_close(out, ref_out, dtype)
        if optimizer == "sgd":
            w_ref = oracle.sgd_step(w_ref, c["table_offsets"], new_idx, c["offsets"], c["grad"], 0.05,
                                    compute_dtype=torch.float32)
        else:
            w_ref, s_ref = oracle.exact_rowwise_adagrad_step(w_ref, s_ref, c["table_offsets"], new_idx, c["offsets"],
                                                             c["grad"], 0.05, 0.1)
        assert_close(w, w_ref, dtype)
    if optimizer != "sgd":
        torch.testing.assert_close(state.cpu(), s_ref, rtol=1e-5, atol=1e-5)


def test_captured_step_equals_eager_bit_for_bit(cuda_device):
    dev = cuda_device
    c = to_device(make_case(T=6, E=3000, D=128, B=256, Lmax=0, dtype=torch.float16, seed=9, fixed_L=20), dev)
    idx, off, to, go = c["indices_d"], c["offsets_d"], c["table_offsets_d"], c["grad_d"]
    w_eager = c["weights_d"].clone()
    out_eager = tbe.forward(w_eager, to, idx, off, None, 20, 1, False)
    tbe.backward_sgd(go, w_eager, to, idx, off, 0.05, 20, 1, False)
    torch.cuda.synchronize(dev)

    w = c["weights_d"].clone()
    out = torch.empty_like(out_eager)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        tbe.forward(w, to, idx, off, None, 20, 1, False, out=out)
        tbe.backward_sgd(go, w, to, idx, off, 0.05, 20, 1, False)
    graph.replay()
    torch.cuda.synchronize(dev)
    assert torch.equal(out, out_eager)
    assert torch.equal(w, w_eager)
