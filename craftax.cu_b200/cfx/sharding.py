"""Host-side sharding of the env batch over ranks: contiguous env-index slices, no
data-path collective (envs are independent, weights are replicated).  The only
communication is a barrier and a max-reduction of timings, done with torch.distributed
by the caller's process group (NCCL on GPUs, gloo in CPU tests)."""


def env_slice(rank, world, n_total, align=32):
    """Contiguous slice [start, stop) of rank `rank`; every slice is a multiple of `align`
    envs (the policy handle needs n % 32 == 0) and the slices tile [0, n_total)."""
    if n_total % align != 0:
        raise ValueError(f"n_total={n_total} must be a multiple of {align}")
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    units = n_total // align
    base, extra = divmod(units, world)
    start_u = rank * base + min(rank, extra)
    size_u = base + (1 if rank < extra else 0)
    return start_u * align, (start_u + size_u) * align


def _single(dist):
    return dist is None or not dist.is_initialized() or dist.get_world_size() == 1


def max_over_ranks(values, dist=None):
    """Element-wise maximum over ranks of a list of timings (the slowest rank sets the job
    time).  `dist` is an initialised torch.distributed module or None for a single process."""
    vals = [float(v) for v in values]
    if _single(dist) or not vals:
        return vals
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor(vals, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def aggregate_throughput(local_ms, local_env_steps, dist=None):
    """Whole-job env-steps/s = env-steps of all ranks / max over ranks of the elapsed time."""
    if _single(dist):
        return local_env_steps / (local_ms * 1e-3), local_ms
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    s = torch.tensor([float(local_env_steps)], dtype=torch.float64, device=dev)
    dist.all_reduce(s, op=dist.ReduceOp.SUM)
    t = max_over_ranks([local_ms], dist)[0]
    return s.item() / (t * 1e-3), t
