"""Head sharding across the GPUs of one node.

Every quantisation group and every unit of kernel work belongs to one (batch, head), so attention
splits by head with no exchange on the forward path: rank r of W owns a contiguous range of heads,
prepares and attends to them on its own GPU, and the outputs are disjoint head slices.  Only a
caller that wants the whole [S,H,128] output on every rank pays for a collective (an all-gather of
the BF16 slices); it is never fused with a peer-memory load.

The reference has no distributed code; "H = 7" in its tables is the per-GPU share of a 56-head
model under 8-way head (Ulysses) parallelism (docs/performance.md:15 of the reference).
"""


def head_range(heads, world_size, rank):
    """Contiguous [start, stop) of heads owned by ``rank``; the first ``heads % world_size`` ranks get one more."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    if heads < 1 or world_size < 1:
        raise ValueError("heads and world_size must be positive")
    base, extra = divmod(heads, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_heads(tensor, world_size, rank):
    """The rank's contiguous copy of ``tensor[..., h0:h1, :]`` (head axis is -2)."""
    h0, h1 = head_range(tensor.shape[-2], world_size, rank)
    return tensor[..., h0:h1, :].contiguous()


def gather_heads(local, heads, group=None):
    """All-gather per-rank outputs ``[..., H_r, 128]`` into ``[..., H, 128]`` on every rank.

    Uses the default (or given) torch.distributed group: NCCL over NVLink for CUDA tensors, gloo for
    CPU tensors.  Ranks may own different head counts, so slices are padded to the largest count.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    widest = max(head_range(heads, world, r)[1] - head_range(heads, world, r)[0] for r in range(world))
    padded = local
    if local.shape[-2] != widest:
        pad = list(local.shape)
        pad[-2] = widest - local.shape[-2]
        padded = torch.cat([local, local.new_zeros(pad)], dim=-2)
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded.contiguous(), group=group)
    parts = []
    for r, piece in enumerate(pieces):
        h0, h1 = head_range(heads, world, r)
        parts.append(piece[..., : h1 - h0, :])
    return torch.cat(parts, dim=-2)


def attention_head_sharded(q, k, v, *, heads=None, group=None, gather=False, **kwargs):
    """Attention over this rank's heads.

    ``q, k, v`` hold either all heads (``heads=None``: the rank's slice is cut out here) or already
    only this rank's heads (``heads`` = the global head count).  Returns the local output, or the
    full ``[..., H, 128]`` tensor when ``gather`` is true.
    """
    import torch.distributed as dist

    from .api import attention

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if heads is None:
        heads = q.shape[-2]
        q, k, v = (shard_heads(t, world, rank) for t in (q, k, v))
    h0, h1 = head_range(heads, world, rank)
    if q.shape[-2] != h1 - h0:
        raise ValueError(f"rank {rank} expects {h1 - h0} heads, got {q.shape[-2]}")
    out = attention(q, k, v, **kwargs) if h1 > h0 else q.new_zeros(q.shape)
    return gather_heads(out, heads, group) if gather and world > 1 else out
