"""View-parallel training step: host-side pieces that do not depend on the device.

The path shards by camera view (the reference loops over the views of a batch sequentially,
src/lib/rendering/PointRenderer.cu:741-745 and 1339-1344, and views only meet in the gradient buffers).  Every rank
holds a full replica of the point parameters, renders its own views, and the point gradients are summed over ranks
with one collective before the fused Adam step.  MyAdam leaves elements with a zero gradient untouched
(src/lib/models/MyAdam.cu:57-61); because the sum is taken first, "zero" means zero on every rank, which is the
single-process semantics of a batch that contains all views.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np


def shard_views(n_views: int, world: int, rank: int) -> List[int]:
    """Views of `rank`: contiguous blocks, sizes differing by at most one, every view owned exactly once."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world / rank")
    base, extra = divmod(n_views, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


class FlatGradLayout:
    """All point gradients in ONE contiguous fp32 buffer, so that a single collective sums them.

    Order and shapes are those of the gradients BlendPointCloudBackward returns
    (src/lib/rendering/PointRenderer.cu:1423-1426): texture [C,n_tex], confidence [1,n_tex], points [N,4],
    point_size [N,1], background [C]."""

    KEYS = ("texture", "confidence", "points", "point_size", "background")

    def __init__(self, n_points: int, n_tex: int, channels: int):
        self.shapes: Dict[str, Tuple[int, ...]] = {
            "texture": (channels, n_tex), "confidence": (1, n_tex), "points": (n_points, 4),
            "point_size": (n_points, 1), "background": (channels,)}
        self.offsets: Dict[str, int] = {}
        o = 0
        for k in self.KEYS:
            self.offsets[k] = o
            o += int(np.prod(self.shapes[k]))
        self.numel = o

    def views(self, flat):
        """Dict of views into `flat` (a 1-D torch tensor or numpy array of `numel` elements)."""
        if flat.shape[0] != self.numel:
            raise ValueError(f"flat buffer has {flat.shape[0]} elements, layout needs {self.numel}")
        out = {}
        for k in self.KEYS:
            n = int(np.prod(self.shapes[k]))
            seg = flat[self.offsets[k]:self.offsets[k] + n]
            out[k] = seg.view(self.shapes[k]) if hasattr(seg, "view") and not isinstance(seg, np.ndarray) else seg.reshape(self.shapes[k])
        return out


def allreduce_sum(flat, group=None):
    """Sum `flat` (torch tensor) over all ranks in place; a no-op without an initialised process group."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    return flat
