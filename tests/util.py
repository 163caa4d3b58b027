"""Shared helpers of the parity tests: run one synthetic scene through the CPU oracle and through the CUDA library
(via the C ABI) and compare every intermediate."""
from __future__ import annotations

import numpy as np

import oracle
from trips_b200 import scenes


def oracle_frames(s: scenes.Scene, train=None, views=None, **param_kw):
    """One oracle.Frame per view."""
    train = s.train if train is None else train
    sa = oracle.SceneArrays.from_scene(s, index=param_kw.pop("index", None))
    p = oracle.make_params(s.num_layers, s.k_keep, train, **param_kw)
    frames = []
    for v in (range(s.n_views) if views is None else views):
        view = oracle.make_view(s.width, s.height, s.poses[v], s.intrinsics[v])
        frames.append(oracle.forward(sa, view, p))
    return sa, p, frames


def sort_lists(counts, offsets, frags):
    """Sort every per-pixel list by its 64-bit key (list order is unspecified; the content is what must match)."""
    out = frags.copy()
    long_lists = np.nonzero(counts > 1)[0]
    for p in long_lists:
        a, b = offsets[p], offsets[p] + counts[p]
        out[a:b] = np.sort(out[a:b])
    return out


def gpu_render(s: scenes.Scene, train=None, views=None, index=None, **render_kw):
    """Render with the CUDA library through the reference-shaped host API.  Returns (scene module, info, outputs)."""
    import torch
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.renderer import NeuralRenderInfo, PointRendererCache, RenderParams, BlendPointCloud
    train = s.train if train is None else train
    ns = NeuralScene.from_synthetic(s)
    if index is not None:
        ns.point_cloud_cuda.t_index = torch.from_numpy(np.ascontiguousarray(index, dtype=np.int32)).cuda().reshape(-1, 1)
    params = RenderParams(num_texture_channels=s.channels, k_keep=s.k_keep, **render_kw)
    info = NeuralRenderInfo(scene=ns, images=images_for(s, views), params=params, num_layers=s.num_layers, train=train,
                            cache=PointRendererCache())
    return ns, info, BlendPointCloud


def rel_err(a, b, floor=None):
    """max |a-b| / max(|b|, floor).  The floor defaults to 1 % of the largest reference magnitude: a bound of 1e-4 on
    this number means rtol = 1e-4 for every element that matters and atol = 1e-6 * max|b| for the near-zero ones
    (sums of fp32 atomics cannot do better than a few ulp of the tensor's scale)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    if b.size == 0:
        return 0.0
    if floor is None:
        floor = max(1e-30, 1e-2 * np.abs(b).max())
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor)))
