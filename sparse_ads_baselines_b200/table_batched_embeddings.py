"""The functions of the reference's ``table_batched_embeddings`` extension module
(table_batched_embeddings.cpp:56-70), bound to libtbe_b200.so.

Same names, argument order and meaning as the reference's pybind11 module.  Tensors must live on a
CUDA device; ``L_max``, ``BT_block_size`` and ``shmem`` are launch hints of the reference's kernels
and are accepted and ignored (results never depend on them).  Everything is enqueued on the
current CUDA stream of the weights' device and nothing synchronises.  Keyword-only extras
(``pooling_mode``) default to the reference's behaviour.
"""
import ctypes
import threading

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.TBE_F32, torch.float16: _lib.TBE_F16, torch.float64: _lib.TBE_F64}
_POOLING = {"sum": _lib.TBE_POOL_SUM, "mean": _lib.TBE_POOL_MEAN}

_ws_lock = threading.Lock()
_workspaces = {}  # (device index, stream handle) -> uint8 tensor


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _check_cuda(name, t, dtype=None):
    _require(isinstance(t, torch.Tensor), "%s must be a tensor" % name)
    _require(t.is_cuda, "%s must be a CUDA tensor (this library has no CPU path)" % name)
    if dtype is not None:
        _require(t.dtype == dtype, "%s must have dtype %s, got %s" % (name, dtype, t.dtype))


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _workspace(device, nbytes):
    """A cached scratch buffer per (device, stream); grows, never shrinks."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    with _ws_lock:
        buf = _workspaces.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = None
            _workspaces.pop(key, None)  # release the old buffer before asking for a larger one
            headroom = 1.25 if nbytes < (1 << 30) else 1.0  # small batches vary in size; huge ones take what they need
            buf = torch.empty(int(nbytes * headroom) + 4096, dtype=torch.uint8, device=device)
            _workspaces[key] = buf
        return buf


def release_workspaces():
    """Drops every cached backward workspace."""
    with _ws_lock:
        _workspaces.clear()


def _geometry(weights, table_offsets, offsets):
    T = table_offsets.numel()
    _require(T > 0, "table_offsets must not be empty")
    _require(weights.dim() == 2, "weights must be [total_rows, D]")
    D = weights.size(1)
    _require(D > 0 and D % 4 == 0, "embedding dimension must be a positive multiple of 4, got %d" % D)
    _require((offsets.numel() - 1) % T == 0, "offsets must have T*B+1 entries")
    B = (offsets.numel() - 1) // T
    _require(B > 0, "batch size must be > 0")
    return T, B, D


def _check_lookup_args(weights, table_offsets, indices, offsets):
    _check_cuda("weights", weights)
    _require(weights.dtype in _DTYPES, "weights must be float16, float32 or float64")
    _require(weights.is_contiguous(), "weights must be contiguous")
    _check_cuda("table_offsets", table_offsets, torch.int32)
    _check_cuda("indices", indices, torch.int32)
    _check_cuda("offsets", offsets, torch.int32)
    for name, t in (("table_offsets", table_offsets), ("indices", indices), ("offsets", offsets)):
        _require(t.device == weights.device, "%s is on %s but weights are on %s" % (name, t.device, weights.device))
        _require(t.is_contiguous(), "%s must be contiguous" % name)


def forward(weights, table_offsets, indices, offsets, indice_weights, L_max, BT_block_size, shmem, *,
            pooling_mode="sum", out=None):
    """Pooled lookup: returns ``[B, T, D]`` (reference: batched_embedding_forward_cuda,
    table_batched_embeddings_cuda.cu:253-316)."""
    _check_lookup_args(weights, table_offsets, indices, offsets)
    T, B, D = _geometry(weights, table_offsets, offsets)
    _require(BT_block_size != 0, "BT_block_size must not be 0")
    _require(pooling_mode in _POOLING, "pooling_mode must be 'sum' or 'mean'")
    psw = None
    if indice_weights is not None:
        _check_cuda("indice_weights", indice_weights, weights.dtype)
        _require(indice_weights.numel() == indices.numel(), "indice_weights must have one entry per index")
        psw = indice_weights.contiguous()
    with torch.cuda.device(weights.device):
        if out is None:
            out = torch.empty((B, T, D), dtype=weights.dtype, device=weights.device)
        else:
            _require(out.shape == (B, T, D) and out.dtype == weights.dtype and out.is_contiguous()
                     and out.device == weights.device, "out must be a contiguous [B, T, D] tensor like weights")
        _lib.call("tbe_forward", weights.data_ptr(), table_offsets.data_ptr(), indices.data_ptr(),
                  offsets.data_ptr(), psw.data_ptr() if psw is not None else None, out.data_ptr(),
                  T, B, D, _DTYPES[weights.dtype], _POOLING[pooling_mode], _stream(weights.device))
    return out


def _grad_view(grad_output, B, T, D, weights):
    _check_cuda("grad_output", grad_output, weights.dtype)
    _require(tuple(grad_output.shape) == (B, T, D), "grad_output must be [B, T, D] = [%d, %d, %d], got %s"
             % (B, T, D, tuple(grad_output.shape)))
    _require(grad_output.device == weights.device, "grad_output must be on the weights' device")
    if grad_output.stride(2) != 1 and D > 1:
        grad_output = grad_output.contiguous()
    return grad_output


def _workspace_bytes(N, total_rows):
    nbytes = _lib.lib().tbe_backward_workspace_bytes(N, total_rows)
    if nbytes < 0:
        raise _lib.TBEError("tbe_backward_workspace_bytes", nbytes, _lib.last_error())
    return nbytes


def _backward_workspace(weights, N, total_rows):
    return _workspace(weights.device, _workspace_bytes(N, total_rows))


def _max_rows_per_table(table_offsets, total_rows):
    """Row count of the largest table (lets the sort skip the table bits).  Reads ``table_offsets``
    back once per tensor OBJECT and version -- a host synchronisation on the first call only.  The
    value is kept on the tensor itself: an address can be handed to another tensor by the allocator,
    an attribute cannot."""
    cached = getattr(table_offsets, "_tbe_max_rows", None)
    key = (table_offsets._version, int(total_rows), table_offsets.numel())
    if cached is not None and cached[0] == key:
        return cached[1]
    offs = table_offsets.detach().cpu().tolist() + [int(total_rows)]
    diffs = [b - a for a, b in zip(offs[:-1], offs[1:])]
    v = max(diffs) if diffs and min(diffs) >= 0 else 0
    try:
        table_offsets._tbe_max_rows = (key, v)
    except AttributeError:  # a tensor subclass without a __dict__
        pass
    return v


_side_streams = {}


def _side_stream(device):
    s = _side_streams.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device, priority=-1)  # its short kernels go ahead of the long gathers
        _side_streams[device.index] = s
    return s


class BackwardPlan:
    """The index-only half of a backward (sorted lookups), built ahead of time on a side stream."""

    def __init__(self, workspace, event, N, total_rows, max_rows):
        self.workspace, self.event = workspace, event
        self.N, self.total_rows, self.max_rows = N, total_rows, max_rows


def backward_plan(table_offsets, indices, offsets, total_rows, workspace=None):
    """Starts sorting the lookups of ``(indices, offsets)`` on a side stream and returns a
    :class:`BackwardPlan`; pass it as ``plan=`` to a ``backward_*`` call for the same inputs.
    Nothing here depends on the gradient, so it overlaps with the forward or with an exchange.
    ``workspace`` (a uint8 CUDA tensor of at least ``tbe_backward_workspace_bytes``) lets a caller
    that builds one plan per step reuse one buffer: the side stream first waits for everything
    already enqueued on the current stream, which includes the backward that last read the buffer."""
    _check_cuda("table_offsets", table_offsets, torch.int32)
    _check_cuda("indices", indices, torch.int32)
    _check_cuda("offsets", offsets, torch.int32)
    dev = indices.device
    T = table_offsets.numel()
    B = (offsets.numel() - 1) // T
    N = indices.numel()
    max_rows = _max_rows_per_table(table_offsets, total_rows)
    with torch.cuda.device(dev):
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        nbytes = _workspace_bytes(N, total_rows)
        if workspace is None:
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        else:
            _require(workspace.is_cuda and workspace.dtype == torch.uint8 and workspace.numel() >= nbytes,
                     "workspace must be a uint8 CUDA tensor of at least %d bytes" % nbytes)
            ws = workspace
        # the side stream reads tensors that were allocated on the main stream: tell the allocator,
        # so that dropping the autograd graph without a backward cannot recycle them under the sort
        for t in (ws, indices, offsets, table_offsets):
            t.record_stream(side)
        side.wait_stream(main)
        _lib.call("tbe_backward_plan", table_offsets.data_ptr(), indices.data_ptr(), offsets.data_ptr(), T, B, N,
                  total_rows, max_rows, ws.data_ptr(), ws.numel(), ctypes.c_void_p(side.cuda_stream))
        event = torch.cuda.Event()
        event.record(side)
    return BackwardPlan(ws, event, N, total_rows, max_rows)


def _plan_or_workspace(plan, weights, table_offsets, N):
    """(workspace, max_rows, plan_ready) for a backward call; waits for a prebuilt plan."""
    total_rows = weights.size(0)
    if plan is None:
        return _backward_workspace(weights, N, total_rows), _max_rows_per_table(table_offsets, total_rows), 0
    _require(plan.N == N and plan.total_rows == total_rows, "the backward plan was built for other inputs")
    torch.cuda.current_stream(weights.device).wait_event(plan.event)
    return plan.workspace, plan.max_rows, 1


def backward_sgd(grad_output, weights, table_offsets, indices, offsets, learning_rate, L_max, BT_block_size, shmem,
                 *, pooling_mode="sum", plan=None):
    """In-place exact SGD on ``weights`` (reference: batched_embedding_backward_sgd_cuda,
    table_batched_embeddings_cuda.cu:383-435; here repeated rows are summed, not raced)."""
    _check_lookup_args(weights, table_offsets, indices, offsets)
    T, B, D = _geometry(weights, table_offsets, offsets)
    _require(BT_block_size > 0, "BT_block_size must be > 0")
    grad_output = _grad_view(grad_output, B, T, D, weights)
    N = indices.numel()
    with torch.cuda.device(weights.device):
        ws, max_rows, ready = _plan_or_workspace(plan, weights, table_offsets, N)
        _lib.call("tbe_backward_sgd", grad_output.data_ptr(), grad_output.stride(0), grad_output.stride(1),
                  weights.data_ptr(), table_offsets.data_ptr(), indices.data_ptr(), offsets.data_ptr(),
                  T, B, D, N, weights.size(0), _DTYPES[weights.dtype], _POOLING[pooling_mode],
                  float(learning_rate), max_rows, ready, ws.data_ptr(), ws.numel(), _stream(weights.device))
    return None


def _philox_inputs(device, increment):
    """(seed, offset) from the device's default generator, advancing it like a random op would."""
    gen = torch.cuda.default_generators[device.index]
    seed = gen.initial_seed()
    offset = gen.get_offset()
    gen.set_offset(offset + ((increment + 3) // 4) * 4)
    return seed & 0xFFFFFFFFFFFFFFFF, offset


def backward_exact_adagrad(grad_output, weights, table_offsets, indices, offsets, indice_weights, optimizer_state,
                           learning_rate, eps, stochastic_rounding, BT_block_size, *, pooling_mode="sum",
                           plan=None):
    """In-place exact rowwise Adagrad (reference: batched_embedding_backward_adagrad_exact_cuda,
    table_batched_embeddings_cuda.cu:1589-1705).  Like the reference, per-sample weights are not
    supported by this optimizer."""
    _check_lookup_args(weights, table_offsets, indices, offsets)
    T, B, D = _geometry(weights, table_offsets, offsets)
    _require(BT_block_size > 0, "BT_block_size must be > 0")
    _require(indice_weights is None, "exact rowwise Adagrad does not support per-sample weights")
    _check_cuda("optimizer_state", optimizer_state)
    _require(optimizer_state.numel() == weights.size(0) and optimizer_state.is_contiguous(),
             "optimizer_state must be a contiguous [total_rows] tensor")
    state_arg = optimizer_state
    if optimizer_state.dtype != torch.float32:  # see backward_approx_adagrad
        optimizer_state = state_arg.float()
    grad_output = _grad_view(grad_output, B, T, D, weights)
    N = indices.numel()
    seed, offset = (0, 0)
    if stochastic_rounding and weights.dtype == torch.float16:
        seed, offset = _philox_inputs(weights.device, 2 * ((D + 31) // 32))
    with torch.cuda.device(weights.device):
        ws, max_rows, ready = _plan_or_workspace(plan, weights, table_offsets, N)
        _lib.call("tbe_backward_exact_rowwise_adagrad", grad_output.data_ptr(), grad_output.stride(0),
                  grad_output.stride(1), weights.data_ptr(), table_offsets.data_ptr(), indices.data_ptr(),
                  offsets.data_ptr(), optimizer_state.data_ptr(), T, B, D, N, weights.size(0),
                  _DTYPES[weights.dtype], _POOLING[pooling_mode], float(learning_rate), float(eps),
                  int(bool(stochastic_rounding)), seed, offset, max_rows, ready, ws.data_ptr(), ws.numel(),
                  _stream(weights.device))
        if optimizer_state is not state_arg:
            state_arg.copy_(optimizer_state)
    return None


def backward_approx_adagrad(grad_output, weights, table_offsets, indices, offsets, indice_weights, optimizer_state,
                            learning_rate, eps, L_max, stochastic_rounding, BT_block_size):
    """In-place approximate rowwise Adagrad; returns the gradient of ``indice_weights`` or None
    (reference: batched_embedding_backward_adagrad_approx_cuda,
    table_batched_embeddings_cuda.cu:706-793)."""
    _check_lookup_args(weights, table_offsets, indices, offsets)
    T, B, D = _geometry(weights, table_offsets, offsets)
    _require(BT_block_size > 0, "BT_block_size must be > 0")
    _check_cuda("optimizer_state", optimizer_state)
    _require(optimizer_state.numel() == weights.size(0) and optimizer_state.is_contiguous(),
             "optimizer_state must be a contiguous [total_rows] tensor")
    # the kernels keep the rowwise state in fp32; a module cast with .double() (gradient checks) has a
    # float64 buffer, which is converted around the call
    state_arg = optimizer_state
    if optimizer_state.dtype != torch.float32:
        optimizer_state = state_arg.float()
    grad_output = _grad_view(grad_output, B, T, D, weights)
    N = indices.numel()
    psw = grad_psw = None
    if indice_weights is not None:
        _check_cuda("indice_weights", indice_weights, weights.dtype)
        _require(indice_weights.numel() == N, "indice_weights must have one entry per index")
        psw = indice_weights.contiguous()
        grad_psw = torch.empty(indices.shape, dtype=grad_output.dtype, device=weights.device)
    seed, offset = (0, 0)
    if stochastic_rounding and weights.dtype == torch.float16:
        seed, offset = _philox_inputs(weights.device, 2 * ((D + 31) // 32))
    with torch.cuda.device(weights.device):
        ws = _backward_workspace(weights, N, weights.size(0))
        _lib.call("tbe_backward_approx_rowwise_adagrad", grad_output.data_ptr(), grad_output.stride(0),
                  grad_output.stride(1), weights.data_ptr(), table_offsets.data_ptr(), indices.data_ptr(),
                  offsets.data_ptr(), psw.data_ptr() if psw is not None else None,
                  grad_psw.data_ptr() if grad_psw is not None else None, optimizer_state.data_ptr(),
                  T, B, D, N, weights.size(0), _DTYPES[weights.dtype], float(learning_rate), float(eps),
                  int(bool(stochastic_rounding)), seed, offset,
                  _max_rows_per_table(table_offsets, weights.size(0)), ws.data_ptr(), ws.numel(),
                  _stream(weights.device))
        if optimizer_state is not state_arg:
            state_arg.copy_(optimizer_state)
    return grad_psw


# ---------------------------------------------------------------------------- mixed-D tables
# Tables of different width and height share one flat weights vector (reference:
# MixedDimTableBatchedEmbeddingBags, table_batched_embeddings_ops.py:324-434).  Each table is run
# through the uniform kernels as a one-table problem: its lookups are a contiguous slice of
# `indices`, its rows a contiguous slice of `weights`, and its pooled rows go straight into its
# columns of the [B, sum(D)] output (tbe_forward_strided) / are read from its columns of the
# gradient (strided backward), so nothing is copied.

def _host_list(t):
    """Host copy of a small index tensor, kept on the tensor object (per version): one
    synchronisation per distinct tensor, and no confusion when the allocator reuses an address."""
    cached = getattr(t, "_tbe_host_list", None)
    key = (t._version, t.numel())
    if cached is not None and cached[0] == key:
        return cached[1]
    v = [int(x) for x in t.detach().cpu().tolist()]
    try:
        t._tbe_host_list = (key, v)
    except AttributeError:
        pass
    return v


def _mixed_tables(weights, table_offsets, dim_offsets, indices, offsets):
    """Yields (t, weights_t [E_t, D_t], indices_t, offsets_t, lo, hi, col0, D_t) per table."""
    _check_cuda("weights", weights)
    _require(weights.dim() == 1 and weights.is_contiguous(), "mixed-D weights must be a flat contiguous vector")
    _check_cuda("indices", indices, torch.int32)
    _check_cuda("offsets", offsets, torch.int32)
    elem = _host_list(table_offsets)
    cols = _host_list(dim_offsets)
    T = len(cols) - 1
    _require(len(elem) == T + 1, "table_offsets and dim_offsets must both have T + 1 entries")
    _require((offsets.numel() - 1) % T == 0, "offsets must have T*B+1 entries")
    B = (offsets.numel() - 1) // T
    bounds = offsets[::B].cpu().tolist()  # first lookup of every table (+ the total); one synchronisation
    out = []
    for t in range(T):
        D = cols[t + 1] - cols[t]
        _require(D > 0 and D % 4 == 0, "every embedding dimension must be a positive multiple of 4")
        w_t = weights[elem[t]:elem[t + 1]].view(-1, D)
        lo, hi = int(bounds[t]), int(bounds[t + 1])
        out.append((t, w_t, indices[lo:hi], offsets[t * B:(t + 1) * B + 1] - lo, lo, hi, cols[t], D))
    return out, B, T


def forward_mixed_D(weights, table_offsets, dim_offsets, total_D, indices, offsets, indice_weights, L_max,
                    BT_block_size, shmem):
    """Pooled lookup over tables of different width in one launch: returns ``[B, total_D]``
    (reference: batched_embedding_forward_mixed_D_cuda, table_batched_embeddings_cuda.cu:945-1004).
    ``table_offsets`` are int64 element offsets ``[T+1]`` into the flat ``weights``, ``dim_offsets``
    int32 output columns ``[T+1]``, as MixedDimTableBatchedEmbeddingBags registers them."""
    _check_cuda("weights", weights)
    _require(weights.dim() == 1 and weights.is_contiguous(), "mixed-D weights must be a flat contiguous vector")
    _require(weights.dtype in _DTYPES, "weights must be float16, float32 or float64")
    _check_cuda("table_offsets", table_offsets, torch.int64)
    _check_cuda("dim_offsets", dim_offsets, torch.int32)
    _check_cuda("indices", indices, torch.int32)
    _check_cuda("offsets", offsets, torch.int32)
    elem, cols = _host_list(table_offsets), _host_list(dim_offsets)  # host copies, cached per tensor
    T = len(cols) - 1
    _require(len(elem) == T + 1, "table_offsets and dim_offsets must both have T + 1 entries")
    _require((offsets.numel() - 1) % T == 0, "offsets must have T*B+1 entries")
    B = (offsets.numel() - 1) // T
    _require(B > 0, "batch size must be > 0")
    dims = [cols[t + 1] - cols[t] for t in range(T)]
    _require(all(d > 0 and d % 4 == 0 for d in dims), "every embedding dimension must be a positive multiple of 4")
    _require(int(total_D) == cols[-1], "total_D must equal dim_offsets[-1]")
    es = weights.element_size()
    vb = 16 if all((d * es) % 16 == 0 for d in dims) and all((e * es) % 16 == 0 for e in elem) else 8
    dev = weights.device
    psw = None
    if indice_weights is not None:
        _check_cuda("indice_weights", indice_weights, weights.dtype)
        _require(indice_weights.numel() == indices.numel(), "indice_weights must have one entry per index")
        psw = indice_weights.contiguous()
    with torch.cuda.device(dev):
        out = torch.empty((B, int(total_D)), dtype=weights.dtype, device=dev)
        _lib.call("tbe_forward_mixed", weights.data_ptr(), table_offsets.data_ptr(), dim_offsets.data_ptr(),
                  indices.data_ptr(), offsets.data_ptr(), psw.data_ptr() if psw is not None else None, out.data_ptr(),
                  T, B, int(total_D), _DTYPES[weights.dtype], vb, _stream(dev))
    return out


def _mixed_groups(tables, table_offsets_tensor, elem):
    """Runs of consecutive tables of one width: ``(t0, t1, table_offsets_g)`` with the group's row
    offsets (int32, on the device, relative to the group's first row).  Tables of one width that
    follow each other share their layout with the uniform kernels -- rows of D elements back to
    back, gradient columns side by side -- so a run takes ONE sort and ONE update launch."""
    cache = getattr(table_offsets_tensor, "_tbe_mixed_groups", None)
    key = tuple(tb[7] for tb in tables)
    if cache is not None and cache[0] == key:
        return cache[1]
    groups, t0 = [], 0
    dev = table_offsets_tensor.device
    for t in range(1, len(tables) + 1):
        if t == len(tables) or tables[t][7] != tables[t0][7]:
            D = tables[t0][7]
            rows = [(elem[u] - elem[t0]) // D for u in range(t0, t)]
            groups.append((t0, t, torch.tensor(rows, dtype=torch.int32, device=dev)))
            t0 = t
    try:
        table_offsets_tensor._tbe_mixed_groups = (key, groups)
    except AttributeError:
        pass
    return groups


def _backward_mixed(exact, grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, total_D, indices,
                    offsets, indice_weights, optimizer_state, learning_rate, eps, stochastic_rounding):
    tables, B, T = _mixed_tables(weights, table_offsets, dim_offsets, indices, offsets)
    rows = _host_list(table_dim_offsets)
    elem = _host_list(table_offsets)
    _require(tuple(grad_output.shape) == (B, int(total_D)), "grad_output must be [B, total_D]")
    if grad_output.stride(1) != 1:
        grad_output = grad_output.contiguous()
    grad_psw = None
    if indice_weights is not None:
        grad_psw = torch.empty(indices.shape, dtype=grad_output.dtype, device=weights.device)
    for (t0, t1, to_g) in _mixed_groups(tables, table_offsets, elem):
        D, col0, lo, hi = tables[t0][7], tables[t0][6], tables[t0][4], tables[t1 - 1][5]
        Tg = t1 - t0
        w_g = weights[elem[t0]:elem[t1]].view(-1, D)
        idx_g = indices[lo:hi]
        off_g = tables[t0][3] if Tg == 1 else offsets[t0 * B:t1 * B + 1] - lo
        g_g = grad_output[:, col0:col0 + Tg * D].unflatten(1, (Tg, D))  # [B, Tg, D], sample stride total_D
        s_g = optimizer_state[rows[t0]:rows[t1]]
        if exact:
            backward_exact_adagrad(g_g, w_g, to_g, idx_g, off_g, None, s_g, learning_rate, eps, stochastic_rounding, 1)
        else:
            psw = indice_weights[lo:hi] if indice_weights is not None else None
            gp = backward_approx_adagrad(g_g, w_g, to_g, idx_g, off_g, psw, s_g, learning_rate, eps, 200,
                                         stochastic_rounding, 1)
            if gp is not None:
                grad_psw[lo:hi] = gp
    return grad_psw


def backward_approx_adagrad_mixed_D(grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, total_D,
                                    indices, offsets, indice_weights, optimizer_state, learning_rate, eps, L_max,
                                    stochastic_rounding, BT_block_size):
    """reference: batched_embedding_backward_adagrad_approx_mixed_D_cuda,
    table_batched_embeddings_cuda.cu:1076-1163."""
    return _backward_mixed(False, grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, total_D,
                           indices, offsets, indice_weights, optimizer_state, learning_rate, eps, stochastic_rounding)


def backward_exact_adagrad_mixed_D(grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, total_D,
                                   indices, offsets, indice_weights, optimizer_state, learning_rate, eps,
                                   stochastic_rounding, BT_block_size):
    """reference: batched_embedding_backward_adagrad_exact_mixed_D_cuda,
    table_batched_embeddings_cuda.cu:1350-1469 (per-sample weights unsupported, as there)."""
    _require(indice_weights is None, "exact rowwise Adagrad does not support per-sample weights")
    return _backward_mixed(True, grad_output, weights, table_offsets, table_dim_offsets, dim_offsets, total_D,
                           indices, offsets, None, optimizer_state, learning_rate, eps, stochastic_rounding)


def sort_segments(table_offsets, indices, offsets, total_rows, max_rows_per_table=0):
    """The backward's integer bookkeeping: ``(sorted_rows, sorted_bags, segment_starts)`` with
    ``segment_starts`` trimmed to the number of distinct rows (synchronises to read that count).
    ``max_rows_per_table`` > 0 (an upper bound on every table's row count, tables laid out in
    ascending order) selects the table-segmented sort the optimizer calls use."""
    _check_cuda("table_offsets", table_offsets, torch.int32)
    _check_cuda("indices", indices, torch.int32)
    _check_cuda("offsets", offsets, torch.int32)
    T = table_offsets.numel()
    B = (offsets.numel() - 1) // T
    N = indices.numel()
    dev = indices.device
    with torch.cuda.device(dev):
        rows = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
        bags = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
        starts = torch.empty(N + 1, dtype=torch.int32, device=dev)
        count = torch.zeros(1, dtype=torch.int32, device=dev)
        nbytes = _lib.lib().tbe_backward_workspace_bytes(N, total_rows)
        if nbytes < 0:
            raise _lib.TBEError("tbe_backward_workspace_bytes", nbytes, _lib.last_error())
        ws = _workspace(dev, nbytes)
        _lib.call("tbe_sort_segments", table_offsets.data_ptr(), indices.data_ptr(), offsets.data_ptr(),
                  T, B, N, total_rows, int(max_rows_per_table), rows.data_ptr(), bags.data_ptr(), starts.data_ptr(),
                  count.data_ptr(),
                  ws.data_ptr(), ws.numel(), _stream(dev))
        u = int(count.item())
    return rows[:N], bags[:N], starts[:u]


def construct_offsets(batch_offsets_per_table, total_indices_per_table):
    """``int32 [1 + T*B]`` with a leading 0 followed by every bag's length; the caller cumsums it
    (reference: construct_offsets, table_batched_embeddings_cuda.cu:1190-1213)."""
    _check_cuda("batch_offsets_per_table", batch_offsets_per_table, torch.int32)
    _check_cuda("total_indices_per_table", total_indices_per_table, torch.int32)
    _require(batch_offsets_per_table.dim() == 2, "batch_offsets_per_table must be [T, B]")
    T, B = batch_offsets_per_table.shape
    _require(total_indices_per_table.numel() == T, "total_indices_per_table must be [T]")
    dev = batch_offsets_per_table.device
    begin = batch_offsets_per_table.contiguous()
    totals = total_indices_per_table.contiguous()
    with torch.cuda.device(dev):
        out = torch.empty(1 + T * B, dtype=torch.int32, device=dev)
        _lib.call("tbe_construct_offsets", begin.data_ptr(), totals.data_ptr(), out.data_ptr(), T, B, _stream(dev))
    return out


def check_inputs(indices, offsets, rows_per_table):
    """Raises if indices/offsets violate the layout contract (synchronises)."""
    _check_cuda("indices", indices, torch.int32)
    _check_cuda("offsets", offsets, torch.int32)
    _check_cuda("rows_per_table", rows_per_table, torch.int32)
    T = rows_per_table.numel()
    _require((offsets.numel() - 1) % T == 0, "offsets must have T*B+1 entries")
    B = (offsets.numel() - 1) // T
    with torch.cuda.device(indices.device):
        _lib.call("tbe_check_inputs", indices.data_ptr(), offsets.data_ptr(), rows_per_table.data_ptr(), T, B,
                  indices.numel(), _stream(indices.device))


class _RawCudaBuffer:
    """Owns an allocation made by libtbe_b200 and exposes it through __cuda_array_interface__."""

    def __init__(self, device_ptr, nbytes, free_fn, free_arg, typestr, shape):
        self._free_fn, self._free_arg = free_fn, free_arg
        self.device_ptr, self.nbytes = device_ptr, nbytes
        self.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": typestr, "data": (device_ptr, False), "version": 2, "strides": None,
        }

    def __del__(self):
        if self._free_fn is not None:
            try:
                getattr(_lib.lib(), self._free_fn)(ctypes.c_void_p(self._free_arg))
            except Exception:
                pass
            self._free_fn = None


_TYPESTR = {torch.float16: "<f2", torch.float32: "<f4", torch.float64: "<f8", torch.int32: "<i4", torch.int64: "<i8",
            torch.uint8: "|u1"}


def _numel(sizes):
    n = 1
    for s in sizes:
        n *= int(s)
    return n


def new_managed_tensor(proto, sizes):
    """A tensor of ``proto``'s dtype on ``proto``'s device backed by managed memory that prefers
    host residency and is mapped into the device (reference: new_managed_tensor,
    table_batched_embeddings_cuda.cu:864-871)."""
    _check_cuda("proto", proto)
    sizes = tuple(int(s) for s in sizes)
    nbytes = max(_numel(sizes) * proto.element_size(), 1)
    with torch.cuda.device(proto.device):
        p = ctypes.c_void_p()
        _lib.call("tbe_alloc_managed", ctypes.byref(p), nbytes)
        holder = _RawCudaBuffer(p.value, nbytes, "tbe_free_managed", p.value, _TYPESTR[proto.dtype], sizes)
        return torch.as_tensor(holder, device=proto.device)


def new_host_mapped_tensor(proto, sizes):
    """A tensor on ``proto``'s device whose storage is pinned host memory mapped into the device
    (reference: new_host_mapped_tensor, table_batched_embeddings_cuda.cu:873-880)."""
    _check_cuda("proto", proto)
    sizes = tuple(int(s) for s in sizes)
    nbytes = max(_numel(sizes) * proto.element_size(), 1)
    with torch.cuda.device(proto.device):
        h, d = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.call("tbe_alloc_host_mapped", ctypes.byref(h), ctypes.byref(d), nbytes)
        holder = _RawCudaBuffer(d.value, nbytes, "tbe_free_host_mapped", h.value, _TYPESTR[proto.dtype], sizes)
        t = torch.as_tensor(holder, device=proto.device)
        t._tbe_host_ptr = h.value
        return t
