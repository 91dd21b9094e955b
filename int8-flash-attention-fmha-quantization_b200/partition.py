"""Partitioning of one attention problem over several GPUs.

Every (batch, head) pair is an independent problem (the reference maps one CTA to each,
src/fmha_i8.cu:43, inc/fmha_i8.cuh:59-60), and in the [B,H,S,D] layout any range of the flattened
batch*head axis is one contiguous byte range of Q, K, V and O.  So rank r of n takes heads
[r*BH/n, (r+1)*BH/n), holds only that slice of the four tensors plus the whole [B,S] mask, and calls
fmha_i8_sm100_infer_slice; nothing is exchanged on the data path.
"""


def slice_bounds(total_heads: int, rank: int, world: int):
    """(begin, count) of the contiguous head range of `rank`; counts differ by at most one."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, extra = divmod(total_heads, world)
    begin = rank * base + min(rank, extra)
    return begin, base + (1 if rank < extra else 0)


def max_over_ranks(value: float, group=None) -> float:
    """Job time of a step = the slowest rank's device time."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def exchange_reports(begin: int, count: int, ok: bool, detail: str = "", group=None):
    """Every rank tells every other rank which heads it was given and whether it computed them.
    Returns the list of (rank, begin, count, ok, detail), ordered by rank.  Host-side objects only."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return [(0, int(begin), int(count), bool(ok), str(detail))]
    world = dist.get_world_size(group)
    got = [None] * world
    dist.all_gather_object(got, (dist.get_rank(group), int(begin), int(count), bool(ok), str(detail)), group=group)
    return sorted(got, key=lambda t: t[0])


def coverage(reports, total_heads: int):
    """What a job that lost ranks still has: {"complete": bool, "heads_done": n, "heads_missing": [(begin, count), ...],
    "ranks_failed": [(rank, detail), ...]}.  A rank that failed (or never launched) contributes a hole, nothing else."""
    missing, failed, done = [], [], 0
    for rank, begin, count, ok, detail in reports:
        if ok:
            done += count
        else:
            missing.append((begin, count))
            failed.append((rank, detail))
    return {"complete": not missing and done == total_heads, "heads_done": done, "heads_missing": missing,
            "ranks_failed": failed}


def assemble_on_rank0(slice_out, begin: int, count: int, ok: bool, total_heads: int, detail: str = "", group=None):
    """Gathers the per-rank output slices (torch tensors [count, ...], on the device for an NCCL group, on the host
    for gloo) onto rank 0.  Returns (whole, coverage): `whole` is a tensor [total_heads, ...] on rank 0 (None
    elsewhere) in which the heads of failed ranks are zero; `coverage` (see coverage()) is returned on every rank.
    A rank whose computation failed passes ok=False (its tensor is ignored and may be None); nothing here waits
    for more than every rank's arrival, so a failed rank costs a hole in the result, not a hang."""
    import torch
    import torch.distributed as dist
    reports = exchange_reports(begin, count, ok, detail, group)
    cov = coverage(reports, total_heads)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return (slice_out if ok else None), cov
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    # equal-sized contributions: pad to the largest slice; failed ranks send zeros of the agreed shape
    shape_src = [None]
    shapes = [None] * world
    dist.all_gather_object(shapes, (tuple(slice_out.shape[1:]), str(slice_out.dtype)) if (ok and slice_out is not None) else None, group=group)
    good = [s for s in shapes if s is not None]
    if not good:
        return None, cov
    tail, dtype_name = good[0]
    dtype = getattr(torch, dtype_name.replace("torch.", ""))
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    max_count = max(c for _, _, c, _, _ in reports)
    send = torch.zeros((max_count,) + tuple(tail), dtype=dtype, device=dev)
    if ok and slice_out is not None:
        send[:count].copy_(slice_out.reshape((count,) + tuple(tail)))
    recv = [torch.empty_like(send) for _ in range(world)] if rank == 0 else None
    dist.gather(send, recv, dst=0, group=group)
    if rank != 0:
        return None, cov
    whole = torch.zeros((total_heads,) + tuple(tail), dtype=dtype, device=dev)
    for (r, b, c, good_r, _), part in zip(reports, recv):
        if good_r:
            whole[b:b + c].copy_(part[:c])
    return whole, cov
