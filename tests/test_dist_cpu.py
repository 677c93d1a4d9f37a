"""Host-side logic of the multi-GPU mode on CPU ranks (gloo, world size 2): every rank derives the same
token-balanced partition from the lengths alone, works on its own contiguous shard without any
collective, and the verification gather reassembles the batch in order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nestedtensor_b200 import sharding, workloads
from oracle import ntref


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = workloads.config1()
        lengths = w.sizes[:, 0].tolist()
        parts = sharding.token_balanced_partition(lengths, world)
        a, b = parts[rank]
        shard = w.slice(a, b)
        # the "hot path" of this rank on its shard alone (CPU stand-in: the oracle); padded to the GLOBAL
        # maximum so that the shards concatenate into the global dense tensor
        gmax = int(w.sizes[:, 0].max())
        local = torch.stack([ntref.pad_tensor_to_shape(t, [gmax, 256], 0.0) for t in shard.tensors()])
        # verification gather of the ragged inputs and of the dense outputs
        buf, sizes = sharding.gather_ragged(shard.buffer, shard.sizes)
        dense, _ = sharding.gather_ragged(local.reshape(-1), torch.tensor([[local.numel()]], dtype=torch.int64))
        ok = torch.equal(buf, w.buffer) and torch.equal(sizes, w.sizes)
        want = ntref.to_padded_tensor(w.tensors(), 0.0)
        ok = ok and torch.equal(dense.reshape(want.shape), want)
        results[rank] = (ok, parts, int(shard.sizes[:, 0].sum()))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_verification_gather():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == world
    assert all(results[r][0] for r in range(world))
    assert results[0][1] == results[1][1]                      # same partition on every rank
    toks = [results[r][2] for r in range(world)]
    assert abs(toks[0] - toks[1]) <= 128                       # within one sequence of balance


def test_partition_properties_random():
    g = torch.Generator().manual_seed(0)
    for _ in range(50):
        n = int(torch.randint(0, 40, (1,), generator=g))
        world = int(torch.randint(1, 9, (1,), generator=g))
        L = torch.randint(0, 50, (n,), generator=g).tolist()
        parts = sharding.token_balanced_partition(L, world)
        assert len(parts) == world and parts[0][0] == 0 and parts[-1][1] == n
        assert all(a <= b for a, b in parts) and all(p[1] == q[0] for p, q in zip(parts, parts[1:]))
