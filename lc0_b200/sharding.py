"""Batch partitioning for data-parallel evaluation with replicated weights.

The path has no exchange step: each GPU evaluates a contiguous slice of the batch and keeps its results
(the reference's `demux` backend does the same split above the backend, src/neural/backends/network_demux.cc:279-334).
"""


def split_batch(total, parts, step=1):
    """Contiguous (start, stop) slices of `total` positions for `parts` workers, slice sizes rounded to
    multiples of `step` (the workers' preferred batch step) except for the last non-empty slice."""
    if parts <= 0:
        raise ValueError("parts must be positive")
    if total < 0 or step <= 0:
        raise ValueError("bad total / step")
    units = -(-total // step)
    base, extra = divmod(units, parts)
    out, start = [], 0
    for r in range(parts):
        n = (base + (1 if r < extra else 0)) * step
        stop = min(total, start + n)
        out.append((start, stop))
        start = stop
    return out


def gather_max(value, dist=None):
    """Max of a per-rank float over all ranks (what the bench uses for its max-over-ranks timing)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
