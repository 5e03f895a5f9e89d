"""Data-parallel helpers: the path shards over independent batch rows; the only exchange of a training
step is one all-reduce of the small fp32 weight-gradient buffer (no reference counterpart: the
reference's MPI benchmarks run independent replicas, benchmarks/common_benchmarks.h:53-54)."""
import ctypes

import torch


def shard_rows(n_rows, rank, world_size, multiple=8):
    """Row range [start, stop) of `rank`.  Every rank gets the same number of rows, a multiple of the kernels'
    batch granularity (8, SwiftNetMLP.h:293-302): each rank's step normalises its loss by its own row count
    and the trainer averages the ranks' gradients with equal weights, which is the gradient of the global
    mean loss only for equal shards.  Raises (on every rank alike, before any collective is entered) when
    n_rows does not split that way, instead of leaving one rank with a different or empty shard."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    unit = multiple * world_size
    if n_rows <= 0 or n_rows % unit != 0:
        raise ValueError(f"{n_rows} rows do not split into {world_size} equal shards of a multiple of {multiple} rows; "
                         f"pad or trim the batch to a multiple of {unit}")
    per = n_rows // world_size
    return rank * per, (rank + 1) * per


def allreduce_sum_(tensor, group=None):
    """In-place sum over the ranks of `group` through torch.distributed (gloo in the CPU tests; on GPUs the
    trainer uses the library's own NCCL communicator instead, see create_dp_comm)."""
    if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
        torch.distributed.all_reduce(tensor, group=group)
    return tensor


def create_dp_comm(group):
    """A tnn_dp_comm (NCCL communicator owned by the library) over the ranks of the torch.distributed `group`:
    rank 0 draws the NCCL unique id, the group broadcasts its 128 bytes, every rank joins with the current CUDA
    device.  Returns the handle as a ctypes.c_void_p."""
    from . import _lib

    dist = torch.distributed
    lib = _lib.load()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    buf = (ctypes.c_ubyte * 128)()
    if rank == 0:
        _lib.check(lib.tnn_dp_get_unique_id(buf))
    box = [bytes(buf)]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
    idbuf = (ctypes.c_ubyte * 128).from_buffer_copy(box[0])
    h = ctypes.c_void_p()
    _lib.check(lib.tnn_dp_comm_create(idbuf, rank, world, ctypes.byref(h)))
    return h
