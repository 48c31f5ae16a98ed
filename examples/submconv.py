"""Minimal use of the submanifold conv (mirrors the reference's examples/submconv.py):
build a sparse shell, run the conv forward and backward, reuse the neighbour cache."""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from flexgemm_b200 import workloads
from flexgemm_b200.ops import spconv

RES, C = 128, 256
dev = torch.device("cuda")
spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
coords, feats, weight, bias, shape = workloads.make_problem(RES, C, C, torch.float16, seed=0)
coords, feats = coords.to(dev), feats.to(dev).requires_grad_(True)
weight, bias = weight.to(dev).requires_grad_(True), bias.to(dev).requires_grad_(True)

out, cache = spconv.sparse_submanifold_conv3d(feats, coords, shape, weight, bias)          # builds the neighbour cache
out2, _ = spconv.sparse_submanifold_conv3d(out.detach(), coords, shape, weight, bias, cache)  # reuses it
out.sum().backward()
print("out", tuple(out.shape), "grad_feats", tuple(feats.grad.shape), "grad_weight", tuple(weight.grad.shape),
      "pairs", int(cache["valid_signal_i"].shape[0]))
