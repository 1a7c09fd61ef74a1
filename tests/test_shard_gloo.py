"""world_size-2 CPU test (gloo) of the multi-GPU path's host logic: every rank takes its
(batch, head) shard, computes it independently (here with the CPU oracle standing in for the
kernels), and an all_gather reassembles exactly the unsharded result."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import attention_oracle as orc
from flash_b200 import workloads
from flash_b200 import shard


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, q_out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        B, H, Hk, L, D = (2, 4, 2, 96, 16) if mode == "heads" else (2, 3, 3, 96, 16)
        q = torch.randn(B, H, L, D); k = torch.randn(B, Hk, L, D); v = torch.randn(B, Hk, L, D); do = torch.randn(B, H, L, D)
        ids = torch.from_numpy(workloads.doc_ids("c0", __import__("numpy").random.default_rng(1), B=B, L=L)[0])
        eq = ids[:, None, :].expand(B, H, L)
        full = orc.attention_forward_backward(q, k, v, do, True, None, eq, eq, 1)
        dim, qs, ks = shard.shard_slices(B, H, Hk, world, rank)
        assert dim == (1 if mode == "heads" else 0)
        tq, tk = (lambda x: shard.take_shard(x, dim, qs)), (lambda x: shard.take_shard(x, dim, ks))
        part = orc.attention_forward_backward(tq(q), tk(k), tk(v), tq(do), True, None, tq(eq), tq(eq), 1)
        got = [shard.gather_shards(x, dim) for x in part]
        err = max((a - b).abs().max().item() for a, b in zip(full, got))
        # throughput bookkeeping of the benchmark: units of all ranks over the slowest rank's time
        t = torch.tensor([1.0 + rank])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        q_out.put((rank, err, float(t)))
    finally:
        dist.destroy_process_group()


def _run(mode):
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, tmax in res:
        assert err < 1e-5 and tmax == 2.0


def test_shard_by_head_two_ranks():
    _run("heads")


def test_shard_by_batch_two_ranks():
    _run("batch")


def _failing_worker(rank, world, port, q_out):
    """Rank 1 fails on the host between steps, with nothing in flight: it raises before the gather. Rank 0
    learns of it when its next collective ends with an error after the (short) process-group timeout."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        x = torch.full((4,), float(rank))
        dist.all_reduce(x)  # a first, healthy step
        assert float(x[0]) == 1.0
        if rank == 1:
            raise RuntimeError("injected host-side failure of rank 1")
        try:
            shard.gather_shards(torch.zeros(1, 2, 8, 4), 1)
            q_out.put((rank, "gather returned although a rank was missing"))
        except Exception as exc:  # gloo reports the missing peer (connection closed or timed out)
            q_out.put((rank, "noticed: " + type(exc).__name__))
    except RuntimeError as exc:
        if rank == 1:
            q_out.put((rank, "raised: " + str(exc)))
            return
        raise
    finally:
        if rank == 0:
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def test_a_rank_that_fails_between_steps_is_noticed_by_the_others():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q_out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res[1].startswith("raised: injected")
    assert res[0].startswith("noticed:"), res[0]
