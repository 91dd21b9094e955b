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
