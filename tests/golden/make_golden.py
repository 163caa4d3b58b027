"""Regenerates tests/golden/tiny_scene.npz: outputs of the CPU oracle on a tiny seeded scene.

    python tests/golden/make_golden.py

The reference has no fixtures for this path and cannot be built without its saiga submodule, so these vectors are
NOT reference outputs: they freeze the oracle's own results (after the known-answer tests in tests/test_oracle.py
passed) so that later edits of the oracle or of the shared math header cannot change results unnoticed, and they
give the GPU tests a fixture that does not depend on the oracle being rebuilt.  Scene: 400 points, 2 views 40x28,
3 layers, K = 16, seed 99."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def scene():
    from trips_b200 import scenes
    return scenes.tiny(n_points=400, seed=99, width=40, height=28, num_layers=3, k_keep=16, n_views=2, fx=40.0,
                       size_range=(0.01, 0.5))


def compute():
    import oracle
    from trips_b200 import scenes
    s = scene()
    sa = oracle.SceneArrays.from_scene(s)
    p = oracle.make_params(s.num_layers, s.k_keep, True)
    out = {}
    for b in range(s.n_views):
        f = oracle.forward(sa, oracle.make_view(s.width, s.height, s.poses[b], s.intrinsics[b]), p)
        depth, nl, rec = f.points()
        counts, offsets, frags = f.lists()
        nrec, pid, alpha = f.records()
        g = scenes.target_gradient(s, b)
        grads = f.backward(g)
        out.update({f"depth_{b}": depth, f"nlayers_{b}": nl, f"record_{b}": rec, f"counts_{b}": counts,
                    f"offsets_{b}": offsets, f"frags_{b}": frags, f"nrec_{b}": nrec, f"rec_pid_{b}": pid,
                    f"rec_alpha_{b}": alpha, f"pyramid_{b}": f.pyramid_flat()})
        for k, v in grads.items():
            # the fixture holds the five pinhole coefficients' gradients (the scene has no lens distortion, for which the
            # oracle returns eight more entries)
            out[f"grad_{k}_{b}"] = v[:5] if k == "intrinsics" else v
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_scene.npz")
    np.savez_compressed(path, **compute())
    print("wrote", path, os.path.getsize(path), "bytes")
