"""Helpers shared by the GPU parity tests: case construction and oracle comparison."""
import numpy as np
import torch

from oracle import tbe_oracle as oracle

FP32_TOL = dict(rtol=1e-5, atol=1e-6)   # fp32 pooled outputs / updated weights
FP16_TOL = dict(rtol=1e-2, atol=1e-2)   # fp16


def tol(dtype):
    return FP16_TOL if dtype == torch.float16 else FP32_TOL


def make_case(T, E, D, B, Lmax, dtype, seed, fixed_L=None, weighted=False, unique=False, empty_bags=True):
    """Random inputs in the reference tests' style (uniform indices; E small -> repeated rows)."""
    rng = np.random.default_rng(seed)
    if fixed_L is not None:
        lengths = np.full((T, B), fixed_L)
    else:
        lengths = rng.integers(0 if empty_bags else 1, Lmax + 1, size=(T, B))
    offsets = oracle.offsets_from_lengths(lengths)
    N = int(offsets[-1])
    if unique:
        assert fixed_L is not None and B * fixed_L <= E
        indices = np.concatenate([rng.permutation(E)[:B * fixed_L] for _ in range(T)]).astype(np.int32)
    else:
        indices = rng.integers(0, E, size=N).astype(np.int32)
    weights = torch.from_numpy(rng.uniform(-1, 1, size=(T * E, D)).astype(np.float32)).to(dtype)
    grad = torch.from_numpy(rng.standard_normal(size=(B, T, D)).astype(np.float32)).to(dtype)
    psw = torch.from_numpy(rng.standard_normal(size=N).astype(np.float32)).to(dtype) if weighted else None
    return dict(T=T, E=E, D=D, B=B, N=N, indices=indices, offsets=offsets, weights=weights, grad=grad, psw=psw,
                table_offsets=[t * E for t in range(T)], dtype=dtype)


def to_device(case, device):
    d = dict(case)
    d["weights_d"] = case["weights"].to(device)
    d["grad_d"] = case["grad"].to(device)
    d["indices_d"] = torch.from_numpy(case["indices"]).to(device)
    d["offsets_d"] = torch.from_numpy(case["offsets"]).to(device)
    d["table_offsets_d"] = torch.tensor(case["table_offsets"], dtype=torch.int32, device=device)
    d["psw_d"] = case["psw"].to(device) if case["psw"] is not None else None
    return d


def assert_close(actual, expected, dtype, scale=None):
    """Default: elementwise rtol/atol of the dtype.  With ``scale`` (the same sum taken over absolute
    values, i.e. the condition of the summation) the bound is |actual - expected| <= rtol * scale:
    "1e-5 relative" for fp32 and 1e-2 for fp16 in the sense that matters when terms cancel."""
    a, e = actual.detach().cpu().double(), expected.detach().cpu().double()
    if scale is None:
        torch.testing.assert_close(a.float(), e.float(), msg=None, **tol(dtype))
        return
    bound = tol(dtype)["rtol"] * scale.detach().cpu().double() + 1e-30
    worst = ((a - e).abs() / bound).max().item() if a.numel() else 0.0
    assert worst <= 1.0, "error is %.3g x the allowed %g relative bound" % (worst, tol(dtype)["rtol"])


def forward_scale(case, pooling="sum", weighted=False):
    """sum_l |w_l| * |row_l| per output element (divided by L for mean pooling)."""
    psw = case["psw"].abs() if (weighted and case["psw"] is not None) else None
    return oracle.forward(case["weights"].abs().float(), case["table_offsets"], case["indices"], case["offsets"], psw,
                          pooling)
