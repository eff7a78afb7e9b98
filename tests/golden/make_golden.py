"""Generates the golden fixtures in this directory from the CPU oracle (oracle/tbe_oracle.py).

    python tests/golden/make_golden.py

The reference ships no golden vectors and its CUDA extension cannot be built or imported here,
so these vectors come from the same per-table torch.nn.EmbeddingBag computation the reference's
tests use as their oracle.  Inputs are seeded; small cases store inputs and outputs in full, the
config-1 case stores the pooled output, per-table checksums of the updated weights and a sample of
updated rows (its inputs are regenerated from the seed by the workload generators).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import tbe_oracle as oracle  # noqa: E402
from sparse_ads_baselines_b200 import workloads  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def tiny_case(name, T, E, D, B, Lmax, dtype, pooling, optimizer, weighted, seed):
    rng = np.random.default_rng(seed)
    lengths = rng.integers(0, Lmax + 1, size=(T, B))
    offsets = oracle.offsets_from_lengths(lengths)
    N = int(offsets[-1])
    indices = rng.integers(0, E, size=N).astype(np.int32)  # E small -> repeated rows are certain
    tdt = torch.float16 if dtype == "fp16" else torch.float32
    weights = torch.from_numpy(rng.uniform(-1, 1, size=(T * E, D)).astype(np.float32)).to(tdt)
    grad = torch.from_numpy(rng.standard_normal(size=(B, T, D)).astype(np.float32)).to(tdt)
    psw = torch.from_numpy(rng.standard_normal(size=N).astype(np.float32)).to(tdt) if weighted else None
    table_offsets = [t * E for t in range(T)]
    out = oracle.forward(weights, table_offsets, indices, offsets, psw, pooling, compute_dtype=torch.float32)
    rec = dict(T=T, E=E, D=D, B=B, indices=indices, offsets=offsets, weights=weights.float().numpy(),
               grad=grad.float().numpy(), out=out.float().numpy(), dtype=dtype, pooling=pooling,
               optimizer=optimizer)
    if psw is not None:
        rec["psw"] = psw.float().numpy()
    lr, eps = 0.05, 0.2
    rec["lr"], rec["eps"] = lr, eps
    state0 = torch.from_numpy(rng.uniform(0, 1, size=T * E).astype(np.float32))
    rec["state0"] = state0.numpy()
    if optimizer == "sgd":
        w1 = oracle.sgd_step(weights, table_offsets, indices, offsets, grad, lr, pooling, compute_dtype=torch.float32)
        rec["weights_after"] = w1.float().numpy()
    elif optimizer == "exact_rowwise_adagrad":
        w1, s1 = oracle.exact_rowwise_adagrad_step(weights, state0, table_offsets, indices, offsets, grad, lr, eps,
                                                   pooling)
        rec["weights_after"], rec["state_after"] = w1.float().numpy(), s1.numpy()
    elif optimizer == "approx_rowwise_adagrad":
        w1, s1, gp = oracle.approx_rowwise_adagrad_step(weights, state0, table_offsets, indices, offsets, grad, lr,
                                                        eps, psw)
        rec["weights_after"], rec["state_after"] = w1.float().numpy(), s1.numpy()
        if gp is not None:
            rec["grad_psw"] = gp.float().numpy()
    rows, bags, starts = oracle.sort_segments(table_offsets, indices, offsets)
    rec["sorted_rows"], rec["sorted_bags"], rec["segment_starts"] = rows, bags, starts
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print(name, "N=%d U=%d" % (N, len(starts)))


def cfg1_case():
    w = workloads.WORKLOADS["cfg1"]
    indices, offsets = workloads.make_inputs(w)
    weights = torch.from_numpy(workloads.make_weights(w))
    grad = torch.from_numpy(workloads.make_grad(w))
    table_offsets = [t * w.E for t in range(w.T)]
    out = oracle.forward(weights, table_offsets, indices, offsets)
    w1 = oracle.sgd_step(weights, table_offsets, indices, offsets, grad, w.lr)
    rows, bags, starts = oracle.sort_segments(table_offsets, indices, offsets)
    touched = rows[starts]
    sample = touched[:: max(1, len(touched) // 256)][:256]
    rec = dict(out=out.numpy(),
               weights_sum=w1.double().view(w.T, -1).sum(dim=1).numpy(),
               weights_sqsum=w1.double().pow(2).view(w.T, -1).sum(dim=1).numpy(),
               sample_rows=sample.astype(np.int64), sample_values=w1[torch.from_numpy(sample.astype(np.int64))].numpy(),
               num_unique=np.int64(len(starts)), N=np.int64(len(indices)),
               indices_head=indices[:64], sorted_rows_head=rows[:256], segment_starts_head=starts[:256])
    np.savez_compressed(os.path.join(HERE, "cfg1.npz"), **rec)
    print("cfg1 N=%d U=%d" % (len(indices), len(starts)))


if __name__ == "__main__":
    torch.manual_seed(0)
    tiny_case("tiny_fp32_sum_sgd", T=3, E=17, D=8, B=5, Lmax=6, dtype="fp32", pooling="sum", optimizer="sgd",
              weighted=False, seed=1)
    tiny_case("tiny_fp16_sum_sgd", T=2, E=11, D=16, B=7, Lmax=9, dtype="fp16", pooling="sum", optimizer="sgd",
              weighted=False, seed=2)
    tiny_case("tiny_fp32_mean_adagrad", T=4, E=13, D=12, B=6, Lmax=7, dtype="fp32", pooling="mean",
              optimizer="exact_rowwise_adagrad", weighted=False, seed=3)
    tiny_case("tiny_fp16_sum_adagrad", T=2, E=9, D=128, B=9, Lmax=40, dtype="fp16", pooling="sum",
              optimizer="exact_rowwise_adagrad", weighted=False, seed=4)
    tiny_case("tiny_fp32_weighted_approx", T=3, E=19, D=20, B=4, Lmax=5, dtype="fp32", pooling="sum",
              optimizer="approx_rowwise_adagrad", weighted=True, seed=5)
    cfg1_case()
