"""Host-side sharding logic: slice arithmetic, and the world_size-2 aggregation over gloo."""
import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "craftax.cu_b200"))
from cfx.sharding import aggregate_throughput, env_slice, max_over_ranks  # noqa: E402


@pytest.mark.parametrize("n,world", [(262144, 1), (262144 * 8, 8), (96, 2), (160, 4), (32, 4), (2080, 3)])
def test_slices_tile_the_batch(n, world):
    prev = 0
    for r in range(world):
        a, b = env_slice(r, world, n)
        assert a == prev and b >= a and (b - a) % 32 == 0
        prev = b
    assert prev == n
    sizes = [env_slice(r, world, n)[1] - env_slice(r, world, n)[0] for r in range(world)]
    assert max(sizes) - min(sizes) <= 32


def test_slice_errors():
    with pytest.raises(ValueError):
        env_slice(0, 2, 100)
    with pytest.raises(ValueError):
        env_slice(2, 2, 64)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a, b = env_slice(rank, world, 2080)
    ms = 2.0 if rank == 0 else 5.0        # the slower rank sets the job time
    sps, t = aggregate_throughput(ms, (b - a) * 10, dist)
    both = max_over_ranks([ms, 7.0 - ms], dist)
    dist.barrier()
    q.put((rank, a, b, sps, t, both))
    dist.destroy_process_group()


def test_two_rank_aggregation_over_gloo():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, a0, b0, sps0, t0, m0), (r1, a1, b1, sps1, t1, m1) = res
    assert m0 == m1 == [5.0, 5.0]
    assert (a0, b1) == (0, 2080) and b0 == a1
    assert t0 == t1 == 5.0
    assert sps0 == sps1 == pytest.approx(2080 * 10 / 5e-3)


def test_single_process_aggregate():
    sps, t = aggregate_throughput(4.0, 1000)
    assert t == 4.0 and sps == pytest.approx(250000.0)
    assert max_over_ranks([1.5, 2.5]) == [1.5, 2.5]
