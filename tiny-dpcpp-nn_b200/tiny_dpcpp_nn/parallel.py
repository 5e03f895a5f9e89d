"""Data-parallel helpers: the path shards over independent batch rows; the only exchange of a training
step is one all-reduce of the small fp32 weight-gradient buffer (no reference counterpart: the
reference's MPI benchmarks run independent replicas, benchmarks/common_benchmarks.h:53-54)."""
import torch


def shard_rows(n_rows, rank, world_size, multiple=8):
    """Row range [start, stop) of `rank`: equal shards rounded to the kernels' batch granularity
    (multiples of 8, SwiftNetMLP.h:293-302); the last rank takes the remainder."""
    per = (n_rows // world_size) // multiple * multiple
    start = rank * per
    stop = n_rows if rank == world_size - 1 else start + per
    return start, stop


def allreduce_sum_(tensor, group=None):
    """In-place sum over the ranks of `group` (NCCL on GPUs, gloo in the CPU tests)."""
    if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
        torch.distributed.all_reduce(tensor, group=group)
    return tensor
