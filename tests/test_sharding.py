"""Host-side logic of the multi-GPU path: users are split into contiguous per-rank blocks
and results are gathered to rank 0 for verification.  Runs as two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from omnistack_rs_b200.serving import shard_range, gather_rows_to_rank0, ShardLiveness, collect_rows_via_store


def test_shard_range_covers_everything():
    for n, w in ((131072, 8), (10, 3), (2, 4), (0, 2)):
        spans = [shard_range(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _worker(rank, world, port, n_users, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    b, e = shard_range(n_users, world, rank)
    # stand-in for a rank's attention output: a checksum row per owned user
    local = torch.arange(b, e, dtype=torch.float32).unsqueeze(1) * torch.ones(1, 4)
    full = gather_rows_to_rank0(local, n_users)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)            # max-over-ranks timing reduction
    if rank == 0:
        q.put((full[:, 0].tolist(), float(t)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_gloo():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 11, q)) for r in range(2)]
    [p.start() for p in procs]
    users, tmax = q.get(timeout=120)
    [p.join(120) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    assert users == [float(i) for i in range(11)] and tmax == 2.0


def _serving_rank(rank, world, port, n_users, n_steps, leaves_after, q):
    """One CPU rank of a sharded serving loop.  Rank ``world - 1`` stops after step ``leaves_after`` -- between
    steps, with nothing in flight, and without telling anybody -- and the others must notice on the host, finish
    their own steps and deliver a result that names the shard nobody served."""
    from datetime import timedelta
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=60))
    live = ShardLiveness(store, rank, world)
    b, e = shard_range(n_users, world, rank)
    acc = torch.zeros(e - b, 2)
    gone = set()
    for step in range(n_steps):
        acc += torch.arange(b, e, dtype=torch.float32).unsqueeze(1) * torch.tensor([[1.0, float(step)]])
        live.beat(step)
        if rank == world - 1 and step == leaves_after:
            return                                           # the process ends here; no collective is pending
        gone.update(live.missing(step, timeout_s=3.0))
    out = collect_rows_via_store(store, rank, world, acc, n_users, missing=gone)
    if rank == 0:
        rows, spans = out
        q.put((rows[:, 0].tolist(), spans, sorted(gone)))
    else:
        store.set(f"done/{rank}", "1")
    if rank == 0:                                            # the store lives in rank 0: wait for the other survivors
        for r in range(1, world):
            if r not in gone:
                store.wait([f"done/{r}"])


def test_rank_leaves_between_steps_and_survivors_report_the_missing_shard():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, n_users, n_steps = 3, 10, 4
    procs = [ctx.Process(target=_serving_rank, args=(r, world, port, n_users, n_steps, 1, q)) for r in range(world)]
    [p.start() for p in procs]
    col0, spans, gone = q.get(timeout=180)
    [p.join(120) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    assert gone == [2] and spans == [shard_range(n_users, world, 2)]
    b2, e2 = shard_range(n_users, world, 2)
    want = [float(u * n_steps) if not (b2 <= u < e2) else 0.0 for u in range(n_users)]
    assert col0 == want
