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


def slice_bounds(numel: int, world: int, rank: int, align: int = 4):
    """Flat elements [lo, hi) owned by `rank`: equal shares rounded to `align` elements (16-byte vectors)."""
    per = -(-numel // world)
    per = -(-per // align) * align
    lo = min(numel, rank * per)
    return lo, min(numel, lo + per)


class FusedPointOptimizer:
    """Gradient sum over ranks + MyAdam + parameter broadcast as one kernel over peer memory.

    All point parameters of the scene are re-homed into one flat buffer (`self.param_flat`), their gradients are
    written into another (`self.grad_flat`, use `self.grad_views` as the `out=` of PointRendererCache.backward); with
    more than one rank both buffers are symmetric-memory allocations, so every rank holds peer pointers to all of
    them.  `step()` = barrier, trips_fused_reduce_adam on this rank's slice, barrier.  Update semantics are MyAdam's
    (src/lib/models/MyAdam.cu:41-88) evaluated after the sum, i.e. those of a single process that saw all views.
    The optimizer state exists only for the owned slice.

    multicast: when the symmetric-memory allocations come with NVSwitch multicast addresses, the step can run
    trips_fused_reduce_adam_multicast instead (the switch sums the gradients and replicates the new weights).  There
    every GPU sends ALL of its gradient buffer into the switch for the reduction, whatever the number of ranks, while
    over peer pointers it serves (world - 1) / world of it and sends the new weights of its slice world - 1 times.
    Measured on config 3 (360 MB of parameters): 0.65 / 0.56 ms at 2 / 4 ranks through multicast against 0.37 / 0.51
    ms over peer pointers; by the byte counts the curves cross between 4 and 8 ranks.  multicast: None or False = peer
    pointers, True = multicast (an error where the allocation has no multicast address).  `self.mode` says which
    kernel runs."""

    def __init__(self, named_params, cache, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, lrs=None, group=None, multicast=None):
        import ctypes as C

        import torch
        import torch.distributed as dist

        from . import _lib
        self._C, self._lib, self.torch, self.dist = C, _lib, torch, dist
        self.cache = cache
        self.names = [n for n, _ in named_params]
        params = [p for _, p in named_params]
        dev = params[0].device
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.numel = sum(-(-p.numel() // 4) * 4 for p in params)  # every tensor starts on a 16-byte boundary
        self.handles = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm
            g = group if group is not None else dist.group.WORLD
            self.param_flat = symm.empty(self.numel, dtype=torch.float32, device=dev)
            self.grad_flat = symm.empty(self.numel, dtype=torch.float32, device=dev)
            hp, hg = symm.rendezvous(self.param_flat, g), symm.rendezvous(self.grad_flat, g)
            self.handles = (hp, hg)
            self.param_ptrs = [int(x) for x in hp.buffer_ptrs]
            self.grad_ptrs = [int(x) for x in hg.buffer_ptrs]
            self.param_mc = int(getattr(hp, "multicast_ptr", 0) or 0)
            self.grad_mc = int(getattr(hg, "multicast_ptr", 0) or 0)
        else:
            self.param_flat = torch.empty(self.numel, dtype=torch.float32, device=dev)
            self.grad_flat = torch.empty(self.numel, dtype=torch.float32, device=dev)
            self.param_ptrs = [self.param_flat.data_ptr()]
            self.grad_ptrs = [self.grad_flat.data_ptr()]
        self.param_flat.zero_()
        self.grad_flat.zero_()
        self.offsets, self.grad_views, segs = {}, {}, []
        o = 0
        with torch.no_grad():
            for name, p in zip(self.names, params):
                n = p.numel()
                view = self.param_flat[o:o + n].view(p.shape)
                view.copy_(p.data)
                p.data = view  # the module's parameter now lives in the flat buffer
                self.grad_views[name] = self.grad_flat[o:o + n].view(p.shape)
                self.offsets[name] = o
                seg_lr = (lrs or {}).get(name, lr)
                segs.append(_lib.TripsAdamSegment(o, seg_lr, betas[0], betas[1], eps, 0.0, 0.0, 0.0, 0.0, 3.4028234663852886e38))
                o += -(-n // 4) * 4
        self.segments = (_lib.TripsAdamSegment * len(segs))(*segs)
        self.lo, self.hi = slice_bounds(self.numel, self.world, self.rank)
        n_own = max(1, self.hi - self.lo)
        self.first_moments = torch.zeros(n_own, dtype=torch.float32, device=dev)
        self.second_moments = torch.zeros(n_own, dtype=torch.float32, device=dev)
        self.steps = torch.zeros(n_own, dtype=torch.int32, device=dev)
        self._gp = (C.c_void_p * self.world)(*self.grad_ptrs)
        self._pp = (C.c_void_p * self.world)(*self.param_ptrs)
        have_mc = self.world > 1 and bool(getattr(self, "param_mc", 0)) and bool(getattr(self, "grad_mc", 0))
        if multicast and not have_mc:
            raise RuntimeError("FusedPointOptimizer: multicast=True, but the symmetric-memory allocations have no multicast address")
        self.mode = "multimem" if (have_mc and multicast) else "peer"
        # all ranks must run the same kernel (a rank without a multicast address would otherwise read stale replicas)
        if self.world > 1:
            flag = torch.tensor([1 if self.mode == "multimem" else 0], device=dev, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            if int(flag.item()) == 0:
                self.mode = "peer"

    def barrier(self):
        if self.handles is not None:
            self.handles[1].barrier(channel=0)

    def step(self):
        """Every rank must call this after its backward pass wrote `grad_views`."""
        C, _lib, torch = self._C, self._lib, self.torch
        self.barrier()  # all gradients are complete and visible
        stream = C.c_void_p(torch.cuda.current_stream(self.param_flat.device).cuda_stream)
        if self.mode == "multimem":
            _lib.check(_lib.lib().trips_fused_reduce_adam_multicast(
                self.cache._h, C.c_void_p(self.grad_mc), C.c_void_p(self.param_mc), C.c_void_p(self.param_flat.data_ptr()), self.segments,
                len(self.segments), self.lo, self.hi, self.first_moments.data_ptr(), self.second_moments.data_ptr(),
                self.steps.data_ptr(), stream), self.cache._h)
        else:
            _lib.check(_lib.lib().trips_fused_reduce_adam(self.cache._h, self._gp, self._pp, self.world, self.rank, self.segments,
                                                         len(self.segments), self.lo, self.hi, self.first_moments.data_ptr(),
                                                         self.second_moments.data_ptr(), self.steps.data_ptr(), stream), self.cache._h)
        self.barrier()  # every replica holds the new parameters before anybody renders again
