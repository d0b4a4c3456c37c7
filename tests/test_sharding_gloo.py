"""World-size-2 and -3 CPU tests (gloo) of the multi-rank path: every rank builds only its own
(batch x head) shard of a workload, computes on it, and the gathered result must equal the
single-process result.  The compute here is the float64 oracle; what is under test is the
sharding, the per-head seeded generation and the verification gather."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jvp_flash_attention_b200 import sharding, workloads
from oracle import jvp_attention_oracle as orc

TOTAL_HEADS = 5  # deliberately not divisible by the world sizes
L = 64


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = sharding.local_heads(TOTAL_HEADS)
        assert (lo, hi) == workloads.shard_range(TOTAL_HEADS, rank, world)
        if hi > lo:
            w = workloads.make_workload("c5_bf16_long", L=L, heads=(lo, hi))
            t = w.tensors
            o, to = orc.sdpa_jvp(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"])
            shard = torch.stack([o[0], to[0]], dim=1).float()  # (n_local, 2, L, D)
        else:
            shard = torch.zeros(0, 2, L, 128)
        full = sharding.gather_heads(shard, TOTAL_HEADS)
        assert full.shape[0] == TOTAL_HEADS
        if rank == 0:
            torch.save(full, os.path.join(out_dir, f"gathered_w{world}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_heads_gather_to_the_single_process_result(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = torch.load(tmp_path / f"gathered_w{world}.pt")
    w = workloads.make_workload("c5_bf16_long", L=L, heads=(0, TOTAL_HEADS))
    t = w.tensors
    o, to = orc.sdpa_jvp(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"])
    ref = torch.stack([o[0], to[0]], dim=1).float()
    assert torch.equal(got, ref)


def test_gather_without_process_group_is_identity():
    x = torch.arange(6.0).reshape(3, 2)
    assert sharding.gather_heads(x, 3) is x
    assert sharding.local_heads(7) == (0, 7)


def test_more_ranks_than_heads_leaves_surplus_ranks_empty():
    spans = [workloads.shard_range(2, r, 4) for r in range(4)]
    assert spans == [(0, 1), (1, 2), (2, 2), (2, 2)]
