"""MyAdam: the reference's custom Adam over point parameters (src/lib/models/MyAdam.{h,cu}) on the fused kernel.

Same surface as torch::optim::MyAdam: param groups with (lr, betas, eps, relative_weight_decay,
absolute_weight_decay, weight_clipping_magnitude, adabound), step(), shrinkInternalState(group, keep) and
appendToInternalState(group, new_size).  All tensors of all groups are updated by ONE kernel launch.
Semantics that differ from torch.optim.Adam and are kept: elements with a zero gradient are untouched, every
element has its own step counter, epsilon is added to sqrt(v) before the bias correction is applied to lr.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable

import torch

from . import _lib

_FLT_MAX = 3.4028234663852886e38


class MyAdam(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 relative_weight_decay: float = 0.0, absolute_weight_decay: float = 0.0,
                 weight_clipping_magnitude: float = 0.0, adabound: bool = False, cache=None):
        if lr < 0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if eps < 0:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0 <= betas[0] < 1.0:
            raise ValueError(f"Invalid beta parameter at index 0: {betas[0]}")
        if not 0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid beta parameter at index 1: {betas[1]}")
        if relative_weight_decay < 0 or absolute_weight_decay < 0:
            raise ValueError("Invalid weight decay value")
        defaults = dict(lr=lr, betas=betas, eps=eps, relative_weight_decay=relative_weight_decay,
                        absolute_weight_decay=absolute_weight_decay, weight_clipping_magnitude=weight_clipping_magnitude,
                        adabound=adabound)
        super().__init__(params, defaults)
        # `cache`: a PointRendererCache whose library context (stream-ordered scratch, stage timers) is shared
        self._ctx = None
        self._shared = cache

    def _context(self, device):
        if self._shared is not None:
            return self._shared._h
        if self._ctx is None:
            h = C.c_void_p()
            _lib.check(_lib.lib().trips_context_create(C.byref(h), device.index or 0))
            self._ctx = h
        return self._ctx

    def __del__(self):
        if getattr(self, "_ctx", None):
            try:
                _lib.lib().trips_context_destroy(self._ctx)
            except Exception:
                pass
            self._ctx = None

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        entries = []
        keep = []
        device = None
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Adam does not support sparse gradients")
                if p.dtype != torch.float32 or not p.is_cuda:
                    raise RuntimeError("MyAdam on the B200 kernel takes float32 CUDA parameters")
                if not p.is_contiguous():
                    raise RuntimeError("MyAdam needs contiguous parameters")
                device = p.device
                st = self.state[p]
                if len(st) == 0:
                    st["param_steps"] = torch.zeros(p.shape, dtype=torch.int32, device=p.device)
                    st["first_moments"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                    st["second_moments"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                    st["current_step"] = 0
                st["current_step"] += 1
                lo, hi = 0.0, _FLT_MAX
                if group["adabound"]:
                    # AdaBound bounds, MyAdam.cu:220-224
                    lo = 0.1 - 0.1 / ((1 - beta2) * st["current_step"] + 1)
                    hi = 0.1 + 0.1 / ((1 - beta2) * st["current_step"])
                g = p.grad.contiguous()
                keep.append(g)
                entries.append(_lib.TripsAdamTensor(p.data_ptr(), g.data_ptr(), st["first_moments"].data_ptr(),
                                                    st["second_moments"].data_ptr(), st["param_steps"].data_ptr(), p.numel(),
                                                    group["lr"], beta1, beta2, group["eps"], group["relative_weight_decay"],
                                                    group["absolute_weight_decay"], group["weight_clipping_magnitude"], lo, hi))
        if entries:
            arr = (_lib.TripsAdamTensor * len(entries))(*entries)
            ctx = self._context(device)
            stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            _lib.check(_lib.lib().trips_adam_step(ctx, arr, len(entries), stream), ctx)
        return loss

    @torch.no_grad()
    def shrinkInternalState(self, param_group_index: int, indices_to_keep: torch.Tensor):
        """Keep only the listed entries along the last dimension of every state tensor (MyAdam.cu:346-373)."""
        group = self.param_groups[param_group_index]
        for p in group["params"]:
            st = self.state.get(p)
            if not st:
                continue
            idx = indices_to_keep.reshape(-1).to(p.device).long()
            for k in ("first_moments", "second_moments", "param_steps"):
                st[k] = st[k].index_select(st[k].dim() - 1, idx).contiguous()

    @torch.no_grad()
    def appendToInternalState(self, param_group_index: int, new_size: int):
        """Zero-extend every state tensor along its last dimension to `new_size` (MyAdam.cu:376-415)."""
        group = self.param_groups[param_group_index]
        for p in group["params"]:
            st = self.state.get(p)
            if not st:
                continue
            for k in ("first_moments", "second_moments", "param_steps"):
                t = st[k]
                extra = new_size - t.shape[-1]
                pad = torch.zeros(t.shape[:-1] + (extra,), dtype=t.dtype, device=t.device)
                st[k] = torch.cat([t, pad], dim=-1).contiguous()

    def rebind(self, old_param: torch.Tensor, new_param: torch.Tensor):
        """Move the state of a replaced parameter tensor (the reference keys state by tensor identity, MyAdam.cu:184)."""
        if old_param in self.state:
            self.state[new_param] = self.state.pop(old_param)
        for group in self.param_groups:
            group["params"] = [new_param if q is old_param else q for q in group["params"]]


def UpdateOptimLR(optimizer: torch.optim.Optimizer, factor: float):
    """Scale the learning rate of every param group in place (MyAdam.h:91-118)."""
    for pg in optimizer.param_groups:
        pg["lr"] = pg["lr"] * factor
