"""Batch sharding across the GPUs of one box: one process per GPU.

The hot path has no cross-sample dependence (the outer ``ops.map`` over samples in
examples/stacked_rnn/stacked_lstm1.py:61, dilated_rnn.py:39-40, grid_rnn.py:144-145,
flash_attention.py:85-87), so rank r simply owns a contiguous slice of the batch
and weights are replicated.  No collective runs inside the recurrence; the only
exchange is one all-gather of the output shards.
"""
import torch
import torch.distributed as dist


def shard_range(n, rank, world):
    """Contiguous slice [lo, hi) of n batch entries owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world: %r/%r" % (rank, world))
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(t, dim, rank, world):
    lo, hi = shard_range(t.shape[dim], rank, world)
    return t.narrow(dim, lo, hi - lo).contiguous()


def gather_batch(local, dim, n_total, group=None):
    """All-gathers the batch shards (contiguous split of n_total along `dim`) into the full tensor
    on every rank.  NCCL over NVLink for CUDA tensors, gloo for CPU tensors."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    if n_total % world == 0 and dim == 0:
        out = local.new_empty([n_total] + list(local.shape[1:]))
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    # Uneven or inner-dimension split: pad every shard to the longest one, gather, trim.
    sizes = [shard_range(n_total, r, world) for r in range(world)]
    longest = max(hi - lo for lo, hi in sizes)
    padded = local
    if local.shape[dim] < longest:
        pad_shape = list(local.shape)
        pad_shape[dim] = longest - local.shape[dim]
        padded = torch.cat([local, local.new_zeros(pad_shape)], dim=dim)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p.narrow(dim, 0, hi - lo) for p, (lo, hi) in zip(parts, sizes)], dim=dim)
