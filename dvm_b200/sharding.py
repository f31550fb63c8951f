"""Partitioning of the fused-operator workloads over the GPUs of one box.

The reference has no data / tensor parallelism of its own; its only multi-device feature is the in-kernel
collectives of the NPU backend (src/ops_c.cc), of which MatMul -> AllReduce (src/ops_c.cc:366-645) is the one on this
path.  Here every workload is cut along an independent leading dimension with no communication, and the K-split
MatMul exchanges fp32 partial products with one all-reduce.
"""
import numpy as np


def leading_range(extent, rank, world):
    """[begin, end) of `extent` owned by `rank`: contiguous blocks, sizes differing by at most one."""
    base, rem = divmod(int(extent), int(world))
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_leading(array, rank, world, axis=0):
    """The slice of `array` along `axis` that `rank` works on (a view)."""
    b, e = leading_range(array.shape[axis], rank, world)
    index = [slice(None)] * array.ndim
    index[axis] = slice(b, e)
    return array[tuple(index)]


def ksplit_operands(a, b, rank, world):
    """K-split of C = A @ B: rank r multiplies A[:, Kr] by B[Kr, :]; the partial products are summed by an all-reduce."""
    kb, ke = leading_range(a.shape[-1], rank, world)
    return np.ascontiguousarray(a[..., kb:ke]), np.ascontiguousarray(b[..., kb:ke, :])


def units_processed(per_rank_units, world, scaling):
    """Whole-job units of one step: every rank a full shard (weak) or one workload cut into `world` parts (strong)."""
    return per_rank_units * world if scaling == "weak" else per_rank_units
