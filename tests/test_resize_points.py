"""trips_resize_points (device-side point removal / growth over all per-point tensors and the Adam state) against the
numpy restatement of the reference's index_select / cat semantics.  Bit-exact: the operation only moves values."""
import numpy as np
import pytest


def test_oracle_resize_points_known_answer(oracle_lib):
    a = np.arange(12, dtype=np.float32).reshape(6, 2)          # point-major [N, 2]
    b = np.arange(18, dtype=np.int32).reshape(3, 6)            # planar [3, N]
    pa, pb = oracle_lib.resize_points([(a, True, 0.0), (b, False, 7)], [4, 1], 6)
    assert pa.tolist() == [[0, 1], [4, 5], [6, 7], [10, 11], [0, 0], [0, 0]]
    assert pb.tolist() == [[0, 2, 3, 5, 7, 7], [6, 8, 9, 11, 7, 7], [12, 14, 15, 17, 7, 7]]
    assert oracle_lib.resize_points([(a, True, 0.0)], [], 6)[0].tolist() == a.tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("n,frac,grow", [(1, 0.0, 0), (5000, 0.3, 0), (5000, 0.0, 777), (40_001, 0.5, 1234), (8192, 1.0, 5), (4096, 1.0, 0)])
def test_resize_points_matches_numpy(cuda_lib, oracle_lib, n, frac, grow):
    import torch
    from trips_b200 import scenes
    from trips_b200.modules import NeuralScene
    from trips_b200.optim import MyAdam
    from trips_b200.renderer import PointRendererCache
    s = scenes.tiny(n_points=n, seed=n % 97, width=48, height=32, num_layers=2, n_views=1)
    dev = torch.device("cuda")
    ns = NeuralScene.from_synthetic(s, device=dev)
    pc, tex = ns.point_cloud_cuda, ns.texture
    cache = PointRendererCache(dev)
    opt = MyAdam([tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size], lr=1e-3, cache=cache)
    gen = torch.Generator(device=dev)
    gen.manual_seed(n)
    for p in (tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size):
        p.grad = torch.randn(p.shape, device=dev, generator=gen) * (torch.rand(p.shape, device=dev, generator=gen) < 0.7)
    opt.step()  # creates state; elements with zero gradient keep step 0
    rng = np.random.default_rng(n)
    remove = rng.permutation(n)[: int(round(frac * n))]
    n_new = n - remove.size + grow
    params = {"pos": (pc.t_position, True, 0.0), "size": (pc.t_point_size, True, 0.0), "tex": (tex.texture_raw, False, 0.5),
              "conf": (tex.confidence_raw, False, 0.5)}
    before, spec = {}, []
    for k, (p, pm, fill) in params.items():
        before[k] = p.detach().cpu().numpy().copy()
        spec.append((before[k], pm, fill))
        for sk in ("first_moments", "second_moments", "param_steps"):
            before[k + sk] = opt.state[p][sk].cpu().numpy().copy()
            spec.append((before[k + sk], pm, 0))
    want = oracle_lib.resize_points(spec, remove, n_new)
    kept = ns.ResizePoints(cache, torch.from_numpy(remove).to(dev) if remove.size else None, new_size=n_new, optimizers=[opt])
    assert kept == n - remove.size and cache.last_status() == 0
    got = []
    for k, (p, pm, fill) in params.items():
        got.append(p.detach().cpu().numpy())
        for sk in ("first_moments", "second_moments", "param_steps"):
            got.append(opt.state[p][sk].cpu().numpy())
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        assert np.array_equal(g.view(np.uint32), w.view(np.uint32))
    assert pc.t_index.shape == (n_new, 1) and int(pc.t_index[-1]) == n_new - 1 if n_new else True
    if n_new:  # the resized scene still trains: one more optimizer step on the new shapes
        for p in (tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size):
            p.grad = torch.ones_like(p)
        opt.step()
        assert int(opt.state[pc.t_position]["param_steps"].max()) >= 1


@pytest.mark.gpu
def test_resize_points_flags_bad_indices(cuda_lib):
    import ctypes as C

    import torch
    from trips_b200 import _lib
    from trips_b200.renderer import PointRendererCache
    dev = torch.device("cuda")
    cache = PointRendererCache(dev)
    src = torch.arange(40, dtype=torch.float32, device=dev).reshape(10, 4)
    dst = torch.empty((8, 4), device=dev)
    tab = (_lib.TripsPointTensor * 1)(_lib.TripsPointTensor(src.data_ptr(), dst.data_ptr(), 4, 4, 1, 0))
    f = cuda_lib.trips_resize_points
    dup = torch.tensor([3, 3], dtype=torch.int64, device=dev)
    assert f(cache._h, dup.data_ptr(), 2, 10, 8, tab, 1, None) == _lib.OK
    assert cache.last_status() & 16  # TRIPS_DEV_BAD_POINT_INDEX: index listed twice
    oob = torch.tensor([3, 10], dtype=torch.int64, device=dev)
    assert f(cache._h, oob.data_ptr(), 2, 10, 8, tab, 1, None) == _lib.OK
    assert cache.last_status() & 16
    assert f(cache._h, None, 2, 10, 8, tab, 1, None) == _lib.ERR_INVALID_ARG
    assert f(cache._h, dup.data_ptr(), 2, 10, 7, tab, 1, None) == _lib.ERR_INVALID_ARG  # n_new below the kept count
    bad = (_lib.TripsPointTensor * 1)(_lib.TripsPointTensor(src.data_ptr(), dst.data_ptr(), 4, 2, 1, 0))
    assert f(cache._h, None, 0, 10, 10, bad, 1, None) == _lib.ERR_INVALID_ARG  # 2-byte elements
