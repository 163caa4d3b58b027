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
    """Sort every per-pixel list by its 64-bit key (list order is unspecified; the content is what must match).
    Vectorised: one stable sort by key, then one stable sort by the list a fragment belongs to."""
    if frags.size == 0:
        return frags.copy()
    seg = np.repeat(np.arange(counts.size, dtype=np.int64), counts)
    assert seg.size == frags.size, "list lengths do not add up to the number of fragments"
    order = np.argsort(frags, kind="stable")
    order = order[np.argsort(seg[order], kind="stable")]
    return frags[order]


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


def strict_grad_report(a, b, rtol=1e-4):
    """Element-wise view of a gradient comparison: the share of elements with |a - b| <= rtol |b| (elements where both
    are exactly zero count as met), the worst absolute error in units of the tensor's largest magnitude, and the worst
    relative error among the elements above 1e-3 of that magnitude."""
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    if b.size == 0:
        return dict(share_strict=1.0, worst_abs_over_max=0.0, worst_rel_significant=0.0, n=0)
    scale = max(np.abs(b).max(), 1e-300)
    diff = np.abs(a - b)
    met = diff <= rtol * np.abs(b)
    sig = np.abs(b) > 1e-3 * scale
    return dict(share_strict=float(met.mean()), worst_abs_over_max=float(diff.max() / scale),
                worst_rel_significant=float((diff[sig] / np.abs(b[sig])).max()) if sig.any() else 0.0, n=int(b.size))


def parity_report(name, record):
    """Prints one JSON line per full-size parity case (visible with pytest -s / -rP) and, when TRIPS_PARITY_REPORT names
    a file, appends it there."""
    import json
    import os
    line = json.dumps({"case": name, **record})
    print("PARITY " + line)
    path = os.environ.get("TRIPS_PARITY_REPORT")
    if path:
        with open(path, "a") as fh:
            fh.write(line + "\n")
