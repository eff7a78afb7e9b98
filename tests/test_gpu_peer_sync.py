"""tbe_peer_signal_wait on one GPU: the flag protocol that orders the fused exchange across ranks.

Every emulated rank's flag array lives on the same device, so a "peer" store is a local store; all
signals are enqueued before the first wait, so no kernel here ever waits for a kernel behind it in
the stream.  The timeout case polls a flag nothing sets, with a 20 ms limit: the kernel must return
by itself, report {TBE_ERR_TIMEOUT, peer, wanted, seen}, and leave the context usable.
"""
import ctypes

import pytest
import torch

from sparse_ads_baselines_b200 import _lib

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


@pytest.mark.parametrize("world", [1, 2, 8, 16])
def test_signal_then_wait_passes(cuda_device, world):
    dev = cuda_device
    flags = [torch.zeros(32, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    for step in (1, 2, 3):
        for r in range(world):  # every rank raises its slot on all peers ...
            _lib.call("tbe_peer_signal_wait", _ptrs(flags), None, world, r, step, 0, 0, None, _stream(dev))
        for r in range(world):  # ... and then finds all of its slots raised
            _lib.call("tbe_peer_signal_wait", None, flags[r].data_ptr(), world, r, 0, step, 10_000_000, status.data_ptr(),
                      _stream(dev))
        host = (ctypes.c_int32 * 4)()
        _lib.call("tbe_peer_status", status.data_ptr(), host, _stream(dev))
        for r in range(world):
            assert flags[r][:world].tolist() == [step] * world and flags[r][world:].sum().item() == 0
    # waiting for a step that has already passed returns at once (values only grow)
    _lib.call("tbe_peer_signal_wait", None, flags[0].data_ptr(), world, 0, 0, 1, 10_000_000, status.data_ptr(), _stream(dev))
    _lib.call("tbe_peer_status", status.data_ptr(), (ctypes.c_int32 * 4)(), _stream(dev))


def test_wait_runs_out_and_reports(cuda_device):
    dev = cuda_device
    world = 4
    flags = torch.zeros(32, dtype=torch.int32, device=dev)
    flags[:world] = torch.tensor([5, 5, 4, 5], dtype=torch.int32)  # rank 2 never reached step 5
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _lib.call("tbe_peer_signal_wait", None, flags.data_ptr(), world, 0, 0, 5, 20_000_000, status.data_ptr(), _stream(dev))
    stop.record()
    host = (ctypes.c_int32 * 4)()
    rc = _lib.lib().tbe_peer_status(status.data_ptr(), host, _stream(dev))
    assert rc == -6, rc
    assert list(host) == [-6, 2, 5, 4]
    msg = _lib.last_error()
    assert "rank 2" in msg and "step 5" in msg
    assert 15.0 < start.elapsed_time(stop) < 2000.0  # the limit was honoured, roughly
    # the context is still usable and later work runs
    x = torch.arange(10, device=dev).sum().item()
    assert x == 45


def test_argument_checks(cuda_device):
    lib = _lib.lib()
    flags = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    assert lib.tbe_peer_signal_wait(None, None, 2, 0, 1, 1, 1000, None, None) == -1
    assert lib.tbe_peer_signal_wait(None, flags.data_ptr(), 2, 0, 1, 1, 1000, None, None) == -1  # no status word
    assert lib.tbe_peer_signal_wait(None, flags.data_ptr(), 2, 0, 1, 1, 0, flags.data_ptr(), None) == -1  # no limit
    assert lib.tbe_peer_signal_wait(None, flags.data_ptr(), 17, 0, 1, 1, 1000, flags.data_ptr(), None) == -1
    assert lib.tbe_peer_signal_wait(None, flags.data_ptr(), 2, 2, 1, 1, 1000, flags.data_ptr(), None) == -1
