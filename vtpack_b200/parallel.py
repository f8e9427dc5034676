"""Batch sharding across the GPUs of one node: one process per GPU, weights
replicated, no exchange inside the model (every kernel works on whole images), and one
all-gather of the logits after the classifier head.

The reference evaluates the same way (DistributedSampler shards + per-rank forward,
``main.py:217-233``, ``engine/utils.py:231-253``) but only all-reduces its meters; the
logits gather is what a serving front end needs.
"""
import os

import torch
import torch.distributed as dist


def init_from_env(backend=None):
    """Join the process group torchrun describes (RANK / WORLD_SIZE / LOCAL_RANK /
    MASTER_*).  Returns (rank, world_size, local_rank); a single process returns (0,1,0)
    without creating a group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world, local


def shard_range(total: int, rank: int, world: int):
    """Contiguous [start, end) of `total` images owned by `rank`; earlier ranks take the
    remainder, so sizes differ by at most one."""
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def gather_logits(local_logits: torch.Tensor, group=None) -> torch.Tensor:
    """All ranks receive the logits of the whole batch, ordered by rank.  Shards may
    differ in size by one image (they are padded to the largest for the collective)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_logits
    world = dist.get_world_size(group)
    n_local = torch.tensor([local_logits.shape[0]], dtype=torch.int64, device=local_logits.device)
    sizes = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(sizes, n_local, group=group)
    sizes = [int(s.item()) for s in sizes]
    n_max = max(sizes)
    if all(s == n_max for s in sizes):
        out = torch.empty(world * n_max, local_logits.shape[1], dtype=local_logits.dtype,
                          device=local_logits.device)
        dist.all_gather_into_tensor(out, local_logits.contiguous(), group=group)
        return out
    padded = torch.zeros(n_max, local_logits.shape[1], dtype=local_logits.dtype, device=local_logits.device)
    padded[:local_logits.shape[0]] = local_logits
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], 0)


def gather_logits_equal(local_logits: torch.Tensor, out: torch.Tensor, group=None, async_op=False):
    """Fast path for equal shards: one all_gather_into_tensor into a preallocated buffer
    (no size exchange, no host sync).  Returns the work handle when async_op."""
    return dist.all_gather_into_tensor(out, local_logits, group=group, async_op=async_op)
