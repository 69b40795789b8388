"""The multi-GPU path on the CPU: (batch, head) problems are partitioned over ranks with no data
exchange; world_size-2 gloo ranks each compute their slice (with the CPU oracle standing in for the
kernel) and the gathered result must equal the unsharded one.  Also covers the timing reduction
bench.py uses (max over ranks)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tfg_flashattention_b200 import workloads


@pytest.mark.parametrize("total,world", [(256, 8), (100, 8), (100, 3), (5, 8), (48, 1), (0, 4)])
def test_shard_heads_partitions_exactly(total, world):
    slices = [workloads.shard_heads(total, world, r) for r in range(world)]
    covered = [i for s in slices for i in range(s.start, s.stop)]
    assert covered == list(range(total))                      # every head once, in order
    sizes = [s.stop - s.start for s in slices]
    assert max(sizes) - min(sizes) <= 1                       # balanced to within one head
    assert sizes == sorted(sizes, reverse=True)               # the extra heads go to the first ranks


def test_hundred_heads_over_eight_ranks():
    sizes = [workloads.shard_heads(100, 8, r) for r in range(8)]
    assert [s.stop - s.start for s in sizes] == [13, 13, 13, 13, 12, 12, 12, 12]


def test_workload_flops_and_bytes():
    w = workloads.config1()
    assert w.flops() == pytest.approx(6.44e9, rel=1e-2)
    assert w.bytes(with_lse=True) == pytest.approx(25.4e6, rel=1e-2)
    assert workloads.config3(4096, causal=False).flops() == pytest.approx(1.10e12, rel=1e-2)
    assert workloads.config4_attention().flops() == pytest.approx(1.07e11, rel=1e-2)
    assert workloads.config5(32768).flops() == pytest.approx(1.37e13, rel=1e-2)


def test_workload_generator_is_deterministic_and_sliceable():
    w = workloads.AttnWorkload("t", 2, 3, 40, seed=9, stress_k_rows=True)
    q, k, v = w.make_cpu()
    q2, k2, v2 = w.make_cpu()
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)
    qs, ks, vs = w.make_cpu(heads=slice(2, 5))
    assert torch.equal(qs[:, 0], q.reshape(6, 40, 64)[2:5])
    assert (k.norm(dim=-1) > 20).any()                       # some key rows were scaled x4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.attention_oracle import manual_attention
    w = workloads.AttnWorkload("t", 3, 5, 70, seed=12)
    sl = workloads.shard_heads(w.B * w.H, world, rank)
    q, k, v = w.make_cpu(heads=sl)                            # this rank's heads only
    o = manual_attention(q, k, v, causal=True)                # [n_local, 1, N, d]
    # gather for the check only: the data path itself has no collective
    bufs = [None] * world
    dist.all_gather_object(bufs, o)
    # the timing reduction of bench.py: max over ranks
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        torch.save({"o": torch.cat(bufs), "tmax": t.item()}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_sharded_run_equals_unsharded(tmp_path, world):
    out_path = str(tmp_path / "gathered.pt")
    mp.spawn(_rank_main, args=(world, _free_port(), out_path), nprocs=world, join=True)
    res = torch.load(out_path)
    from oracle.attention_oracle import manual_attention
    w = workloads.AttnWorkload("t", 3, 5, 70, seed=12)
    q, k, v = w.make_cpu()
    full = manual_attention(q, k, v, causal=True).reshape(w.B * w.H, 1, w.N, w.d)
    assert torch.equal(res["o"], full)                        # same arithmetic, bit for bit
    assert res["tmax"] == float(world)
