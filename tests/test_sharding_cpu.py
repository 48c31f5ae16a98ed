"""Host-side logic of the sample-sharded path, with two gloo ranks on CPU.
The per-rank compute is supplied by the CPU oracle (the CUDA kernels need a
GPU); what is under test is the partitioning, the batch re-basing and the
single fp32 all-reduce."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flexgemm_b200 import sharding
from oracle import submconv_oracle as orc


def test_assign_samples_lpt():
    parts = sharding.assign_samples([5, 9, 3, 7, 1], 2)
    assert sorted(sum(parts, [])) == [0, 1, 2, 3, 4]
    loads = [sum([5, 9, 3, 7, 1][i] for i in p) for p in parts]
    assert max(loads) == 13
    assert sharding.assign_samples([4, 4, 4, 4], 4) == [[0], [1], [2], [3]]
    assert sharding.assign_samples([3], 2) == [[0], []]
    assert abs(sharding.load_balance_bound([10, 10, 10, 16], 4) - 46 / 16) < 1e-12


def test_local_shard_rebases_batch():
    coords = torch.from_numpy(orc.shell_coords(8, batch=3, scales=(1.0, 0.8, 0.9)))
    feats = torch.arange(coords.shape[0], dtype=torch.float32)[:, None].repeat(1, 2)
    seen = []
    for r in range(2):
        c, f, shape, rows = sharding.local_shard(coords, feats, (3, 2, 8, 8, 8), r, 2)
        assert torch.equal(f[:, 0].long(), rows)
        assert torch.equal(c[:, 1:], coords[rows][:, 1:])
        assert c[:, 0].max().item() == shape[0] - 1 and c[:, 0].min().item() == 0
        seen.append(rows)
    assert torch.equal(torch.sort(torch.cat(seen)).values, torch.arange(coords.shape[0]))
    with pytest.raises(ValueError):
        sharding.sample_ranges(coords.flip(0), 3)


def _oracle_local(grad_out, feats, cache, w, has_bias):
    Co, V, Ci = w.shape
    gin, gw, gb = orc.conv_backward(grad_out, feats, cache["neighbor_map"], w.reshape(Co, 3, 3, 3, Ci), has_bias)
    return gin, gw.reshape(Co, V, Ci).float(), (gb.float() if has_bias else None)


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        coords, feats, weight, bias, shape = orc.make_problem(8, 8, 8, "float32", seed=4, batch=3, scales=(1.0, 0.7, 0.85))
        g = torch.Generator().manual_seed(9)
        grad_out = torch.randn(coords.shape[0], 8, generator=g)
        c, f, lshape, rows = sharding.local_shard(coords, feats, shape, rank, world)
        cache = {"neighbor_map": orc.neighbor_map(c.numpy(), lshape)}
        out = orc.conv_forward(f, cache["neighbor_map"], weight, bias)
        gin, gw, gb = sharding.sharded_backward(grad_out[rows], f, cache, weight, bias, local_grads=_oracle_local)
        torch.save({"rows": rows, "out": out, "gin": gin, "gw": gw, "gb": gb}, os.path.join(tmp, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_matches_unsharded(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    coords, feats, weight, bias, shape = orc.make_problem(8, 8, 8, "float32", seed=4, batch=3, scales=(1.0, 0.7, 0.85))
    g = torch.Generator().manual_seed(9)
    grad_out = torch.randn(coords.shape[0], 8, generator=g)
    nbr = orc.neighbor_map(coords.numpy(), shape)
    out = orc.conv_forward(feats, nbr, weight, bias)
    gin, gw, gb = orc.conv_backward(grad_out, feats, nbr, weight)
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(2)]
    full_out, full_gin = torch.empty_like(out), torch.empty_like(gin)
    for p in parts:
        full_out[p["rows"]] = p["out"]
        full_gin[p["rows"]] = p["gin"]
        assert torch.allclose(p["gw"], gw, atol=1e-4) and torch.allclose(p["gb"], gb, atol=1e-4)
    assert torch.equal(parts[0]["gw"], parts[1]["gw"])
    assert torch.allclose(full_out, out, atol=1e-5) and torch.allclose(full_gin, gin, atol=1e-5)
