"""Host-side logic of the multi-GPU path: users are split into contiguous per-rank blocks
and results are gathered to rank 0 for verification.  Runs as two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from omnistack_rs_b200.serving import shard_range, gather_rows_to_rank0


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
