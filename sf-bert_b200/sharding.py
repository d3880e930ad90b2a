"""Host-side partition of the (batch, head) pairs of an attention problem across ranks.  Every pair
is an independent attention problem that shares only the read-only look-up tables (the reference
indexes them as grid.y / grid.z, blocksparse.h:250-251), so ranks never exchange anything inside
attention; the outputs are gathered afterwards.  No CUDA here: the module is exercised on CPU ranks."""


def partition_pairs(batch, heads, world_size, rank):
    """Contiguous slice [start, stop) of the batch*heads pairs (pair = b*heads + h) owned by `rank`.
    The first (batch*heads) % world_size ranks own one pair more."""
    if not (0 <= rank < world_size):
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    total = batch * heads
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def batch_slice(batch, world_size, rank):
    """Whole batch elements per rank (what bench.py and the encoder driver use: [B', L, H, d] stays contiguous)."""
    if batch % world_size:
        raise ValueError("batch %d does not divide over %d ranks" % (batch, world_size))
    per = batch // world_size
    return rank * per, (rank + 1) * per


def gather_outputs(local_out, world_size, dist=None):
    """All-gather of the per-rank outputs [B', L, H, d] into [world_size * B', L, H, d] (the one collective
    of the path; NCCL on GPUs, gloo in the CPU tests)."""
    import torch
    if world_size == 1:
        return local_out
    if dist is None:
        import torch.distributed as dist
    parts = [torch.empty_like(local_out) for _ in range(world_size)]
    dist.all_gather(parts, local_out.contiguous())
    return torch.cat(parts, dim=0)
