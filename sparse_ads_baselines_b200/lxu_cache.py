"""LXU-cached table-batched embedding bags: the table lives in device-mapped pinned host memory and
a set-associative cache of its rows lives in HBM (LRU or LFU replacement).

The reference has nothing like it -- its tables that do not fit HBM are read over the host link on
every lookup (``EmbeddingLocation.HOST_MAPPED``, table_batched_embeddings_ops.py:159-167).  The
module keeps the call surface of ``TableBatchedEmbeddingBags``: ``forward(indices, offsets)``
returns ``[B, T, D]`` and ``backward`` applies exact SGD in place.  Results are identical to the
uncached module's; only where the rows are read from differs.
"""
import ctypes

import numpy as np
import torch
from torch import nn

from . import _lib
from . import table_batched_embeddings as tbe_ext

_POLICY = {"lru": 0, "lfu": 1}


class _CachedLookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, module, indices, offsets):
        m = module
        m._prefetch(indices, offsets)
        w = m.embedding_weights
        out = torch.empty((m.batch_of(offsets), m.num_tables, m.embedding_dim), dtype=w.dtype, device=indices.device)
        with torch.cuda.device(indices.device):
            _lib.call("tbe_cache_forward", m.cache_rows.data_ptr(), w.data_ptr(), m.table_offsets.data_ptr(),
                      indices.data_ptr(), offsets.data_ptr(), m._locations.data_ptr(), out.data_ptr(),
                      m.num_tables, m.batch_of(offsets), m.embedding_dim, tbe_ext._DTYPES[w.dtype],
                      tbe_ext._POOLING[m.pooling_mode], tbe_ext._stream(indices.device))
        ctx.module = m
        ctx.save_for_backward(indices, offsets)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        m = ctx.module
        indices, offsets = ctx.saved_tensors
        w = m.embedding_weights
        B = m.batch_of(offsets)
        if grad_output.stride(2) != 1:
            grad_output = grad_output.contiguous()
        with torch.cuda.device(indices.device):
            _lib.call("tbe_cache_backward_sgd", grad_output.data_ptr(), grad_output.stride(0), grad_output.stride(1),
                      m.cache_rows.data_ptr(), w.data_ptr(), m.dirty.data_ptr(), offsets.data_ptr(), m.num_tables, B,
                      m.embedding_dim, indices.numel(), w.size(0), m.num_sets, tbe_ext._DTYPES[w.dtype],
                      tbe_ext._POOLING[m.pooling_mode], float(m.learning_rate), m._workspace.data_ptr(),
                      m._workspace.numel(), tbe_ext._stream(indices.device))
        return None, None, None, None


class LXUCachedEmbeddingBags(nn.Module):
    """``num_tables`` tables of ``num_embeddings`` x ``embedding_dim`` in host memory behind a
    ``ways``-way set-associative HBM cache of ``cache_rows`` rows; fused exact SGD."""

    def __init__(self, num_tables, num_embeddings, embedding_dim, cache_rows, ways=4, policy="lru",
                 learning_rate=0.01, fp16=False, pooling_mode="sum", deferred_writeback=False, staged_fill=True,
                 stage_rows=131072):
        super().__init__()
        assert policy in _POLICY and pooling_mode in ("sum", "mean")
        assert ways in (1, 2, 4, 8, 16, 32) and cache_rows % ways == 0
        dtype = torch.float16 if fp16 else torch.float32
        device = torch.device("cuda", torch.cuda.current_device())
        total_rows = num_tables * num_embeddings
        self.num_tables, self.num_embeddings, self.embedding_dim = num_tables, num_embeddings, embedding_dim
        self.ways, self.num_sets, self.policy = ways, cache_rows // ways, policy
        self.learning_rate, self.pooling_mode = learning_rate, pooling_mode
        proto = torch.empty(1, device=device, dtype=dtype)
        # pinned host memory mapped into the device: the GPU reads and writes it directly
        table = tbe_ext.new_host_mapped_tensor(proto, (total_rows, embedding_dim))
        self._table_host_ptr = table._tbe_host_ptr  # the same memory as the CPU addresses it
        self.embedding_weights = nn.Parameter(table, requires_grad=False)
        self.register_buffer("table_offsets", torch.arange(num_tables, dtype=torch.int32, device=device) * num_embeddings)
        self.register_buffer("cache_rows", torch.zeros(cache_rows, embedding_dim, dtype=dtype, device=device),
                             persistent=False)
        self.register_buffer("tags", torch.full((cache_rows,), -1, dtype=torch.int32, device=device), persistent=False)
        self.register_buffer("last_use", torch.zeros(cache_rows, dtype=torch.int32, device=device), persistent=False)
        self.register_buffer("use_count", torch.zeros(cache_rows, dtype=torch.int32, device=device), persistent=False)
        self.register_buffer("dirty", torch.zeros(cache_rows, dtype=torch.uint8, device=device), persistent=False)
        self._anchor = nn.Parameter(torch.zeros(1, device=device))  # gives autograd a reason to call backward
        self.step = 0
        self._stats = torch.zeros(5, dtype=torch.int32, device=device)
        self._locations = None
        self._workspace = None
        # deferred write-backs (optional): dirty victims are staged in HBM by the prefetch and carried to
        # the host table on a side stream while the lookup runs; the next prefetch (and flush) wait for
        # them.  Off by default: SM-issued traffic to mapped host memory shares one ~25 GB/s link budget,
        # so the deferred stores only move the time from the fill kernel into the lookup they overlap.
        self.deferred_writeback = deferred_writeback and not staged_fill
        # staged fill (default): missed rows and dirty victims cross the host link as contiguous copies
        # through the copy engines, gathered / scattered in the host table by the library's worker
        # threads, instead of as SM-issued loads and stores of single rows; the prefetch then waits for
        # the stream once per step
        self.staged_fill = staged_fill
        self.stage_rows = int(stage_rows)
        self._stage_dev = None
        self._stage_host = None
        self._wb_rows = None
        self._wb_ids = None
        self._wb_stream = None
        self._wb_done = None
        self.totals = {"lookups": 0, "hit_lookups": 0, "rows": 0, "hit_rows": 0, "fetched": 0, "uncached": 0}

    def batch_of(self, offsets):
        return (offsets.numel() - 1) // self.num_tables

    def _prefetch(self, indices, offsets):
        tbe_ext._check_cuda("indices", indices, torch.int32)
        tbe_ext._check_cuda("offsets", offsets, torch.int32)
        w = self.embedding_weights
        N = indices.numel()
        dev = indices.device
        nbytes = _lib.lib().tbe_cache_workspace_bytes(N, w.size(0))
        if nbytes < 0:
            raise _lib.TBEError("tbe_cache_workspace_bytes", nbytes, _lib.last_error())
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(int(nbytes * 1.1) + 4096, dtype=torch.uint8, device=dev)
        if self._locations is None or self._locations.numel() < N:
            self._locations = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
        self.step += 1
        stage = min(N, self.cache_rows.size(0))
        if self.deferred_writeback and stage > 0:
            if self._wb_rows is None or self._wb_rows.size(0) < stage:
                self._wait_writeback(dev)  # the side stream may still be reading the old staging buffer
                self._wb_rows = torch.empty((stage, self.embedding_dim), dtype=w.dtype, device=dev)
                self._wb_ids = torch.empty(stage, dtype=torch.int32, device=dev)
            if self._wb_stream is None:
                self._wb_stream = torch.cuda.Stream(dev, priority=-1)
        defer = self.deferred_writeback and stage > 0
        if self.staged_fill and N > 0:
            if self._stage_dev is None:
                dt = tbe_ext._DTYPES[w.dtype]
                nd = _lib.lib().tbe_cache_stage_bytes(self.stage_rows, self.embedding_dim, dt, 0)
                nh = _lib.lib().tbe_cache_stage_bytes(self.stage_rows, self.embedding_dim, dt, 1)
                if nd < 0 or nh < 0:
                    raise _lib.TBEError("tbe_cache_stage_bytes", min(nd, nh), _lib.last_error())
                self._stage_dev = torch.empty(nd, dtype=torch.uint8, device=dev)
                self._stage_host = torch.empty(nh, dtype=torch.uint8).pin_memory()
            with torch.cuda.device(dev):
                _lib.call("tbe_cache_prefetch_staged", self.cache_rows.data_ptr(), self.tags.data_ptr(),
                          self.last_use.data_ptr(), self.use_count.data_ptr(), self.dirty.data_ptr(), w.data_ptr(),
                          self.table_offsets.data_ptr(), indices.data_ptr(), offsets.data_ptr(),
                          self._locations.data_ptr(), self._stats.data_ptr(), self.num_tables, self.batch_of(offsets),
                          self.embedding_dim, N, w.size(0), self.num_sets, self.ways, tbe_ext._DTYPES[w.dtype],
                          _POLICY[self.policy], self.step, self._table_host_ptr, self._stage_dev.data_ptr(),
                          self._stage_host.data_ptr(), self.stage_rows, self._workspace.data_ptr(),
                          self._workspace.numel(), tbe_ext._stream(dev))
            self._last_n = N
            return
        with torch.cuda.device(dev):
            main = torch.cuda.current_stream(dev)
            self._wait_writeback(dev)  # this step's fetches must see the previous step's write-backs
            _lib.call("tbe_cache_prefetch", self.cache_rows.data_ptr(), self.tags.data_ptr(), self.last_use.data_ptr(),
                      self.use_count.data_ptr(), self.dirty.data_ptr(), w.data_ptr(), self.table_offsets.data_ptr(),
                      indices.data_ptr(), offsets.data_ptr(), self._locations.data_ptr(), self._stats.data_ptr(),
                      self.num_tables, self.batch_of(offsets), self.embedding_dim, N, w.size(0), self.num_sets,
                      self.ways, tbe_ext._DTYPES[w.dtype], _POLICY[self.policy], self.step,
                      self._wb_rows.data_ptr() if defer else None, self._wb_ids.data_ptr() if defer else None,
                      self._workspace.data_ptr(), self._workspace.numel(), tbe_ext._stream(dev))
            if defer and N > 0:
                filled = torch.cuda.Event()
                filled.record(main)
                self._wb_stream.wait_event(filled)
                _lib.call("tbe_cache_writeback", self._wb_rows.data_ptr(), self._wb_ids.data_ptr(),
                          self._stats.data_ptr(), w.data_ptr(), self.embedding_dim, tbe_ext._DTYPES[w.dtype],
                          ctypes.c_void_p(self._wb_stream.cuda_stream))
                self._wb_done = torch.cuda.Event()
                self._wb_done.record(self._wb_stream)
        self._last_n = N

    def _wait_writeback(self, device):
        """The current stream waits for the write-backs staged by the last prefetch."""
        if self._wb_done is not None:
            torch.cuda.current_stream(device).wait_event(self._wb_done)
            self._wb_done = None

    def forward(self, indices, offsets):
        return _CachedLookup.apply(self._anchor, self, indices, offsets)

    def last_stats(self):
        """Counters of the last step (synchronises): distinct rows, rows fetched into the cache,
        lookups served by rows that were already cached, distinct rows already cached, distinct rows
        left uncached; plus the hit rate = cached lookups / lookups."""
        rows, fetched, hit_lookups, hit_rows, uncached = (int(x) for x in self._stats.tolist())
        n = getattr(self, "_last_n", 0)
        return {"lookups": n, "rows": rows, "fetched": fetched, "hit_lookups": hit_lookups, "hit_rows": hit_rows,
                "uncached": uncached, "hit_rate": hit_lookups / n if n else 0.0}

    def flush(self):
        """Writes every dirty cached row back to the host table (call before reading the table)."""
        w = self.embedding_weights
        with torch.cuda.device(w.device):
            self._wait_writeback(w.device)
            _lib.call("tbe_cache_flush", self.cache_rows.data_ptr(), w.data_ptr(), self.tags.data_ptr(),
                      self.dirty.data_ptr(), self.cache_rows.size(0), self.embedding_dim, tbe_ext._DTYPES[w.dtype],
                      tbe_ext._stream(w.device))

    def state_dict(self, *args, **kwargs):
        self.flush()
        torch.cuda.synchronize(self.embedding_weights.device)
        return super().state_dict(*args, **kwargs)
