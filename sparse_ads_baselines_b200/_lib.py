"""ctypes binding of libtbe_b200.so (C ABI in include/tbe_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtbe_b200.so")

TBE_F32, TBE_F16, TBE_F64 = 0, 1, 2
TBE_POOL_SUM, TBE_POOL_MEAN = 0, 1
TBE_MAX_PEERS = 16

c_i32p = ctypes.POINTER(ctypes.c_int32)
_vp, _i64, _i32, _f32, _u64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_uint64

# name -> (restype, argtypes); every symbol declared in include/tbe_b200.h
SIGNATURES = {
    "tbe_abi_version": (_i32, []),
    "tbe_last_error_string": (ctypes.c_char_p, []),
    "tbe_kernel_launch_count": (_i64, []),
    "tbe_library_launch_count": (_i64, []),
    "tbe_set_tuning": (_i32, [ctypes.c_char_p, _i32]),
    "tbe_kernel_timing_enable": (_i32, [_i32]),
    "tbe_kernel_timing_read": (_i64, [ctypes.c_char_p, _i64]),
    "tbe_forward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tbe_forward_strided": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tbe_forward_mixed": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tbe_forward_sharded": (_i32, [_vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_vp), _i32, _i64, _i64, _i64, _i64,
                                   _i64, _i32, _i32, _vp]),
    "tbe_all2all_push": (_i32, [_vp, ctypes.POINTER(_vp), _i32, _i32, _i64, _i64, _vp]),
    "tbe_reduce_slots": (_i32, [_vp, _vp, _i32, _i64, _i32, _vp]),
    "tbe_allgather_push": (_i32, [_vp, ctypes.POINTER(_vp), _i32, _i32, _i64, _vp]),
    "tbe_peer_signal_wait": (_i32, [ctypes.POINTER(_vp), _vp, _i32, _i32, _i32, _i32, _i64, _vp, _vp]),
    "tbe_peer_status": (_i32, [_vp, ctypes.POINTER(ctypes.c_int32), _vp]),
    "tbe_backward_workspace_bytes": (_i64, [_i64, _i64]),
    "tbe_backward_plan": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "tbe_backward_sgd": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32,
                                _f32, _i64, _i32, _vp, _i64, _vp]),
    "tbe_noalloc_scratch_bytes": (_i64, []),
    "tbe_backward_sgd_noalloc": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32,
                                        _f32, _i64, _vp]),
    "tbe_backward_exact_rowwise_adagrad": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                                  _i64, _i32, _i32, _f32, _f32, _i32, _u64, _u64, _i64, _i32, _vp,
                                                  _i64, _vp]),
    "tbe_backward_approx_rowwise_adagrad": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                                   _i64, _i64, _i64, _i32, _f32, _f32, _i32, _u64, _u64, _i64,
                                                   _vp, _i64, _vp]),
    "tbe_sort_segments": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "tbe_construct_offsets": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "tbe_permute_bags": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "tbe_check_inputs": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tbe_alloc_managed": (_i32, [ctypes.POINTER(_vp), _i64]),
    "tbe_free_managed": (_i32, [_vp]),
    "tbe_alloc_host_mapped": (_i32, [ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i64]),
    "tbe_free_host_mapped": (_i32, [_vp]),
    "tbe_cache_workspace_bytes": (_i64, [_i64, _i64]),
    "tbe_cache_prefetch": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64,
                                  _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "tbe_cache_writeback": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "tbe_cache_stage_bytes": (_i64, [_i64, _i64, _i32, _i32]),
    "tbe_cache_prefetch_staged": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                         _i64, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _vp, _i64, _vp]),
    "tbe_cache_forward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tbe_cache_backward_sgd": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32,
                                      _i32, _f32, _vp, _i64, _vp]),
    "tbe_cache_flush": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp]),
}

_lock = threading.Lock()
_lib = None


class TBEError(RuntimeError):
    """A libtbe_b200 call returned a non-zero status."""

    def __init__(self, fn, status, message):
        super().__init__("%s failed with status %d: %s" % (fn, status, message))
        self.status = status


def lib():
    """Returns the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        "libtbe_b200.so is not built (expected at %s). Build it with "
                        "`python -m sparse_ads_baselines_b200.build`; there is no CPU or PyTorch fallback." % LIB_PATH)
                handle = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)  # AttributeError if the symbol is missing
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def last_error():
    return lib().tbe_last_error_string().decode("utf-8", "replace")


def check(fn_name, status):
    if status != 0:
        raise TBEError(fn_name, status, last_error())


def call(fn_name, *args):
    """Calls an int-returning entry point and raises TBEError on failure."""
    status = getattr(lib(), fn_name)(*args)
    if status != 0:
        raise TBEError(fn_name, status, last_error())


def kernel_timing_enable(on):
    call("tbe_kernel_timing_enable", int(bool(on)))


def kernel_timing_read():
    """{kernel name: (launches, total_ms)} since timing was enabled; synchronises."""
    buf = ctypes.create_string_buffer(1 << 16)
    n = lib().tbe_kernel_timing_read(buf, len(buf))
    if n < 0:
        raise TBEError("tbe_kernel_timing_read", n, last_error())
    out = {}
    for line in buf.value.decode().splitlines():
        name, count, ms = line.split()
        out[name] = (int(count), float(ms))
    return out
