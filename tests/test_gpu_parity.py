"""GPU parity: the CUDA library (called through the C ABI) against the CPU oracle on identical seeded inputs.

Bars: per-point projection results, list lengths, offsets, fragment lists (as sorted sets), kept point ids and the
number of backward records are BIT-EXACT; alphas and pyramid values within 1e-5 relative; gradients within 1e-4
relative (relative to max(|reference|, 1 % of the largest reference magnitude of that tensor))."""
import numpy as np
import pytest

from trips_b200 import scenes
from util import gpu_render, oracle_frames, rel_err, sort_lists

pytestmark = pytest.mark.gpu

TOL_PYRAMID = 1e-5
TOL_GRAD = 1e-4


def _variants():
    v = {}
    v["base_L4_K16"] = (scenes.tiny(), {}, None)
    v["K8"] = (scenes.tiny(k_keep=8, seed=11), {}, None)
    v["L1"] = (scenes.tiny(num_layers=1, seed=12), {}, None)
    v["L8_odd_97x65"] = (scenes.tiny(num_layers=8, width=97, height=65, seed=13, size_range=(5e-3, 1.5)), {}, None)
    v["C3"] = (scenes.tiny(channels=3, seed=14), {}, None)
    v["C6"] = (scenes.tiny(channels=6, seed=15, n_points=1500), {}, None)
    v["C8"] = (scenes.tiny(channels=8, seed=16, n_points=1500), {}, None)
    v["C16"] = (scenes.tiny(channels=16, seed=17, n_points=1500), {}, None)
    s = scenes.tiny(seed=18, n_points=6000, size_range=(0.05, 0.6))
    s.confidence[:] = 1.0  # opaque points: transmittance falls below the cut-off, records end early
    v["saturating"] = (s, {}, None)
    v["drop_radius"] = (scenes.tiny(seed=19), dict(drop_out_points_by_radius=True, drop_out_radius_threshold=2.0), None)
    v["bg_Tn"] = (scenes.tiny(seed=20), dict(bg_uses_Tn=True), None)
    s = scenes.tiny(seed=21)
    rng = np.random.default_rng(5)
    v["index_permuted"] = (s, {}, rng.permutation(s.n_points).astype(np.int32))
    s = scenes.tiny(seed=22, n_points=3000)
    s.position[:, 2] += 100.0  # everything behind / outside every camera
    v["all_culled"] = (s, {}, None)
    v["three_views_long_lists"] = (scenes.tiny(seed=23, n_points=20000, width=64, height=48, n_views=3), {}, None)
    # lists of several hundred fragments: exercises the streaming top-K path used for lists longer than 192
    v["very_long_lists"] = (scenes.tiny(seed=24, n_points=60000, width=40, height=30, n_views=1, num_layers=3), {}, None)
    # a cloud stored in spatial order: blocks of 8192 consecutive points are compact, the ones beside the view are
    # skipped as a whole by the bounding-box test (the test function checks that some were)
    s = scenes.tiny(seed=30, n_points=50000, n_views=2)
    s.position[:, 0] *= 6.0
    order = np.argsort(s.position[:, 0], kind="stable")
    s.position[:] = s.position[order]
    s.point_size[:] = s.point_size[order]
    s.texture[:] = s.texture[:, order]
    s.confidence[:] = s.confidence.reshape(-1)[order].reshape(s.confidence.shape)
    v["sorted_cloud_block_culling"] = (s, {}, None)
    # every point stored twice (ids i and i + n/2): every list holds pairs of equal depths, which the point id orders
    s = scenes.tiny(seed=33, n_points=3000)
    h = s.n_points // 2
    s.position[h:2 * h] = s.position[:h]
    s.point_size[h:2 * h] = s.point_size[:h]
    v["duplicate_points_depth_ties"] = (s, {}, None)
    # ---- the reference's second forward pipeline (PointRenderer.cu:730-731), selected by its non-default flags ----
    strict = dict(render_points_in_all_lower_resolutions=False)
    v["second_strict_L8_odd_97x65"] = (scenes.tiny(num_layers=8, width=97, height=65, seed=41, size_range=(5e-3, 1.5)), dict(strict), None)
    v["second_combine_lists"] = (scenes.tiny(seed=42, size_range=(5e-3, 0.4)), dict(combine_lists=True), None)
    v["second_combine_strict_L6"] = (scenes.tiny(num_layers=6, seed=43, width=120, height=80, size_range=(5e-3, 1.0)),
                                     dict(strict, combine_lists=True), None)
    v["second_no_layer_point_size_L5"] = (scenes.tiny(seed=44, num_layers=5), dict(use_layer_point_size=False), None)
    s = scenes.tiny(seed=45, n_points=6000, size_range=(0.05, 0.6))
    s.confidence[:] = np.minimum(1.0, s.confidence * 3.0)  # alphas that sum past 1 within a few fragments
    v["second_saturated_accumulation"] = (s, dict(combine_lists=True, saturated_alpha_accumulation=True), None)
    s = scenes.tiny(seed=46, n_points=6000, size_range=(0.05, 0.6), channels=8)
    s.confidence[:] = np.minimum(1.0, s.confidence * 3.0)
    v["second_saturated_strict_C8_index"] = (s, dict(strict, saturated_alpha_accumulation=True),
                                             np.random.default_rng(9).permutation(s.n_points).astype(np.int32))
    # on the first pipeline the flag changes the backward pass only (its forward branch is compiled out, RenderForward.cu:908-935)
    s = scenes.tiny(seed=47, n_points=6000, size_range=(0.05, 0.6))
    s.confidence[:] = np.minimum(1.0, s.confidence * 3.0)
    v["first_pipeline_saturated_backward"] = (s, dict(saturated_alpha_accumulation=True), None)
    v["second_strict_drop_radius"] = (scenes.tiny(seed=48, size_range=(5e-3, 0.8)),
                                      dict(strict, drop_out_points_by_radius=True, drop_out_radius_threshold=2.0), None)
    v["second_combine_three_views_long_lists"] = (scenes.tiny(seed=49, n_points=20000, width=64, height=48, n_views=3),
                                                  dict(combine_lists=True), None)
    # lens distortion: all eight coefficients non-zero and different per view, a cut-off radius that culls the image corners
    s = scenes.tiny(seed=51, n_points=6000, n_views=3, num_layers=5, size_range=(5e-3, 0.5))
    s.intrinsics[:, 5:] = np.array([-0.12, 0.05, -0.01, 0.03, -0.02, 0.004, 2e-3, -3e-3], np.float32)
    s.intrinsics[1, 5:] *= -0.5
    s.intrinsics[2, 5:] *= 2.0
    v["lens_distortion"] = (s, dict(distortion=True, dist_cutoff=0.55), None)
    s = scenes.tiny(seed=52, n_points=4000, channels=8)
    s.intrinsics[:, 5:] = np.array([0.2, -0.05, 0.0, 0.0, 0.0, 0.0, -4e-3, 1e-3], np.float32)
    v["lens_distortion_second_pipeline_C8"] = (s, dict(distortion=True, render_points_in_all_lower_resolutions=False), None)
    # seeded random corners of the parameter space: K = 1 / 4, L = 2 / 5 / 6 / 7, odd image sizes, texture index, drop-out
    rr = np.random.default_rng(2024)
    for i in range(8):
        L = int(rr.choice([1, 2, 3, 5, 6, 7, 8]))
        K = int(rr.choice([1, 4, 8, 16]))
        C = int(rr.choice([3, 4, 6, 8, 16]))
        w_, h_ = int(rr.integers(33, 130)), int(rr.integers(17, 90))
        n = int(rr.integers(200, 12000))
        hi = float(rr.choice([0.05, 0.4, 1.2]))
        sc = scenes.tiny(seed=100 + i, n_points=n, width=w_, height=h_, num_layers=L, k_keep=K, n_views=int(rr.integers(1, 4)),
                         channels=C, size_range=(2e-3, hi), fx=float(rr.choice([40.0, 90.0, 160.0])))
        kw = {}
        if rr.random() < 0.3:
            kw = dict(drop_out_points_by_radius=True, drop_out_radius_threshold=float(rr.choice([1.0, 3.0])))
        idx = rr.permutation(n).astype(np.int32) if rr.random() < 0.4 else None
        v[f"rnd_{i}_L{L}_K{K}_C{C}_{w_}x{h_}"] = (sc, kw, idx)
    return v


VARIANTS = _variants()


@pytest.mark.parametrize("name", list(VARIANTS))
def test_forward_backward_parity(name, oracle_lib, cuda_lib):
    import torch
    s, kw, index = VARIANTS[name]
    okw = dict(kw)
    sa, op, frames = oracle_frames(s, train=True, index=index, **okw)
    ns, info, blend = gpu_render(s, train=True, index=index, **kw)
    for t in (ns.texture.texture_raw, ns.texture.confidence_raw, ns.texture.background_color_raw,
              ns.point_cloud_cuda.t_position, ns.point_cloud_cuda.t_point_size):
        t.requires_grad_(True)
    ns.poses.tangent_poses.requires_grad_(True)
    ns.intrinsics.intrinsics.requires_grad_(True)
    outs = blend(info)
    torch.cuda.synchronize()
    assert info.cache.last_status() == 0
    C = s.channels
    st = info.cache.stats()
    assert st["fragments"] == sum(f.F for f in frames)
    assert st["kept_fragments"] == sum(f.Kf for f in frames)
    assert st["visible_points"] == sum(f.V for f in frames)
    if name in ("sorted_cloud_block_culling", "all_culled"):  # boxes beside / behind the view are skipped as a whole
        assert st["culled_point_blocks"] > 0

    grad_flat = []
    for b, f in enumerate(frames):
        # ---- per point ----
        depth, nl, rec = info.cache.debug_points(b, s.n_points)
        odepth, onl, orec = f.points()
        assert np.array_equal(depth.view(np.uint32), odepth.view(np.uint32)), "depth differs"
        assert np.array_equal(nl, onl), "layer counts differ"
        vis = odepth > 0
        assert np.array_equal(rec.view(np.uint32)[vis], orec.view(np.uint32)[vis]), "point records differ"
        # ---- lists ----
        counts, offsets, frags = info.cache.debug_lists(b, f.P)
        ocounts, ooffsets, ofrags = f.lists()
        assert np.array_equal(counts, ocounts), "list lengths differ"
        assert np.array_equal(offsets, ooffsets), "list offsets differ"
        assert frags.size == ofrags.size
        assert np.array_equal(sort_lists(counts, offsets, frags), ofrags), "fragment lists differ"
        # ---- kept fragments (sorted top-K) and records ----
        nrec, pid, alpha = info.cache.debug_records(b, f.P)
        onrec, opid, oalpha = f.records()
        assert np.array_equal(nrec, onrec), "record counts differ"
        assert np.array_equal(pid, opid), "sorted kept indices differ"
        assert rel_err(alpha, oalpha, floor=1e-6) <= TOL_PYRAMID
        # ---- pyramid ----
        opyr = f.pyramid()
        for l, o in enumerate(outs):
            got = o[b].detach().cpu().numpy()
            assert got.shape == opyr[l].shape
            err = np.max(np.abs(got - opyr[l]) / np.maximum(np.abs(opyr[l]), 1e-3))
            assert err <= TOL_PYRAMID, f"layer {l}: {err}"
        grad_flat.append(scenes.target_gradient(s, b))

    # ---- backward: loss = sum_b <g_b, out_b> ----
    loss = 0
    for b, f in enumerate(frames):
        for l, (w, h, base) in enumerate(f.layers):
            g = torch.from_numpy(grad_flat[b][C * base:C * (base + w * h)].reshape(C, h, w)).cuda()
            loss = loss + (outs[l][b] * g).sum()
    loss.backward()
    torch.cuda.synchronize()
    ref = None
    for b, f in enumerate(frames):
        r = f.backward(grad_flat[b])
        if ref is None:
            ref = {k: v.copy() for k, v in r.items() if k not in ("pose", "intrinsics")}
            ref["pose"] = [r["pose"]]
            ref["intrinsics"] = [r["intrinsics"]]
        else:
            for k in ("texture", "confidence", "position", "point_size", "background"):
                ref[k] += r[k]
            ref["pose"].append(r["pose"])
            ref["intrinsics"].append(r["intrinsics"])
    got = dict(texture=ns.texture.texture_raw.grad, confidence=ns.texture.confidence_raw.grad.reshape(-1),
               position=ns.point_cloud_cuda.t_position.grad, point_size=ns.point_cloud_cuda.t_point_size.grad.reshape(-1),
               background=ns.texture.background_color_raw.grad)
    for k, g in got.items():
        e = rel_err(g.cpu().numpy(), ref[k])
        assert e <= TOL_GRAD, f"grad {k}: rel err {e}"
    assert np.all(ns.point_cloud_cuda.t_position.grad[:, 3].cpu().numpy() == 0)
    gpose = ns.poses.tangent_poses.grad.cpu().numpy()
    gintr = ns.intrinsics.intrinsics.grad.cpu().numpy()
    for b in range(len(frames)):
        assert rel_err(gpose[b], ref["pose"][b]) <= TOL_GRAD, "pose gradient"
        assert rel_err(gintr[b, :5], ref["intrinsics"][b][:5]) <= TOL_GRAD, "intrinsics gradient"
        if kw.get("distortion"):
            assert np.all(ref["intrinsics"][b][5:] != 0)
            assert rel_err(gintr[b, 5:], ref["intrinsics"][b][5:]) <= TOL_GRAD, "distortion coefficient gradient"
        else:
            assert np.all(gintr[b, 5:] == 0)


@pytest.mark.parametrize("flags", [{}, dict(render_points_in_all_lower_resolutions=False, combine_lists=True, saturated_alpha_accumulation=True),
                                   dict(distortion=True, dist_cutoff=0.5)], ids=["first_pipeline", "second_pipeline", "lens_distortion"])
def test_forward_inference_matches_training_output(oracle_lib, cuda_lib, flags):
    """train = false renders the same pyramid and keeps no records (RenderForward.cu:865-880 vs 957-979); with 20 views the
    inference call also runs through more than one sub-batch of views."""
    import torch
    s = scenes.tiny(seed=31, n_views=20, n_points=3000)
    if flags.get("distortion"):
        s.intrinsics[:, 5:] = np.array([-0.1, 0.03, 0.0, 0.02, 0.0, 0.0, 1e-3, -2e-3], np.float32)
    _, _, frames = oracle_frames(s, train=False, **flags)
    ns, info, blend = gpu_render(s, train=False, **flags)
    with torch.no_grad():
        outs = blend(info)
    for b, f in enumerate(frames):
        for l, o in enumerate(f.pyramid()):
            got = outs[l][b].cpu().numpy()
            assert np.max(np.abs(got - o) / np.maximum(np.abs(o), 1e-3)) <= TOL_PYRAMID


def test_config1_forward(oracle_lib, cuda_lib):
    """The CPU-runnable benchmark case in full: 200 k points, 640x480, 4 layers, K = 8, forward only."""
    import torch
    s = scenes.config1()
    _, _, frames = oracle_frames(s, train=False)
    ns, info, blend = gpu_render(s, train=False)
    with torch.no_grad():
        outs = blend(info)
    f = frames[0]
    counts, offsets, frags = info.cache.debug_lists(0, f.P)
    ocounts, ooffsets, ofrags = f.lists()
    assert np.array_equal(counts, ocounts)
    assert np.array_equal(offsets, ooffsets)
    assert np.array_equal(sort_lists(counts, offsets, frags), ofrags)
    for l, o in enumerate(f.pyramid()):
        got = outs[l][0].cpu().numpy()
        assert np.max(np.abs(got - o) / np.maximum(np.abs(o), 1e-3)) <= TOL_PYRAMID


def test_against_frozen_fixture(cuda_lib):
    """The committed fixture tests/golden/tiny_scene.npz (oracle outputs frozen by tests/golden/make_golden.py):
    the CUDA path must reproduce it without the oracle being involved at run time."""
    import importlib.util
    import os
    import torch
    here = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    gold = np.load(os.path.join(here, "tiny_scene.npz"))
    s = mg.scene()
    ns, info, blend = gpu_render(s, train=True)
    params = (ns.texture.texture_raw, ns.texture.confidence_raw, ns.texture.background_color_raw,
              ns.point_cloud_cuda.t_position, ns.point_cloud_cuda.t_point_size)
    outs = blend(info)
    C, P = s.channels, scenes.num_pyramid_pixels(s.width, s.height, s.num_layers)
    sizes = scenes.layer_sizes(s.width, s.height, s.num_layers)
    loss = 0
    for b in range(s.n_views):
        depth, nl, rec = info.cache.debug_points(b, s.n_points)
        assert np.array_equal(depth.view(np.uint32), gold[f"depth_{b}"].view(np.uint32))
        assert np.array_equal(nl, gold[f"nlayers_{b}"])
        counts, offsets, frags = info.cache.debug_lists(b, P)
        assert np.array_equal(counts, gold[f"counts_{b}"]) and np.array_equal(offsets, gold[f"offsets_{b}"])
        assert np.array_equal(sort_lists(counts, offsets, frags), gold[f"frags_{b}"])
        nrec, pid, alpha = info.cache.debug_records(b, P)
        assert np.array_equal(nrec, gold[f"nrec_{b}"]) and np.array_equal(pid, gold[f"rec_pid_{b}"])
        flat = np.concatenate([o[b].detach().cpu().numpy().reshape(-1) for o in outs])
        ref = gold[f"pyramid_{b}"]
        assert np.max(np.abs(flat - ref) / np.maximum(np.abs(ref), 1e-3)) <= TOL_PYRAMID
        g = scenes.target_gradient(s, b)
        base = 0
        for l, (w, h) in enumerate(sizes):
            loss = loss + (outs[l][b] * torch.from_numpy(g[C * base:C * (base + w * h)].reshape(C, h, w)).cuda()).sum()
            base += w * h
    loss.backward()
    for name, p_ in zip(("texture", "confidence", "background", "position", "point_size"), params):
        ref = sum(gold[f"grad_{name}_{b}"] for b in range(s.n_views))
        assert rel_err(p_.grad.cpu().numpy().reshape(ref.shape), ref) <= TOL_GRAD, name


def test_adam_matches_reference_update(oracle_lib, cuda_lib):
    """Three consecutive steps with zero-gradient holes against the scalar restatement of adam_step."""
    import torch
    from trips_b200.optim import MyAdam
    import oracle
    rng = np.random.default_rng(0)
    sizes = [(4, 1003), (1, 1003), (1003, 4), (5,)]
    ws = [rng.normal(size=sz).astype(np.float32) for sz in sizes]
    params = [torch.nn.Parameter(torch.from_numpy(w.copy()).cuda()) for w in ws]
    opt = MyAdam([dict(params=params[:2], lr=1e-3), dict(params=params[2:], lr=5e-3, relative_weight_decay=0.01,
                                                         absolute_weight_decay=0.001, weight_clipping_magnitude=2.5)])
    ref_w = [w.copy().reshape(-1) for w in ws]
    ref_m = [np.zeros_like(w) for w in ref_w]
    ref_v = [np.zeros_like(w) for w in ref_w]
    ref_s = [np.zeros(w.size, np.int64) for w in ref_w]
    for step in range(3):
        for i, p in enumerate(params):
            g = rng.normal(size=sizes[i]).astype(np.float32)
            g[rng.random(size=sizes[i]) < 0.3] = 0.0  # unseen elements
            p.grad = torch.from_numpy(g).cuda()
            kw = dict(lr=1e-3) if i < 2 else dict(lr=5e-3, rel_decay=0.01, abs_decay=0.001, clip=2.5)
            oracle.adam(ref_w[i], g.reshape(-1).copy(), ref_m[i], ref_v[i], ref_s[i], **kw)
        opt.step()
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        assert rel_err(p.detach().cpu().numpy().reshape(-1), ref_w[i], floor=1e-6) <= 1e-5
        st = opt.state[p]
        assert np.array_equal(st["param_steps"].cpu().numpy().reshape(-1), ref_s[i])
        assert rel_err(st["first_moments"].cpu().numpy().reshape(-1), ref_m[i], floor=1e-9) <= 1e-5
        assert rel_err(st["second_moments"].cpu().numpy().reshape(-1), ref_v[i], floor=1e-12) <= 1e-5


def test_error_paths(cuda_lib):
    """Argument errors come back as status codes, not aborts (the reference asserts)."""
    import torch
    from trips_b200 import TripsError
    from trips_b200.renderer import BlendPointCloudBackward
    s = scenes.tiny(n_points=100)
    ns, info, blend = gpu_render(s, train=False)
    info.images[1].w += 2
    with pytest.raises(TripsError):
        blend(info)
    info.images[1].w -= 2
    info.images[0].camera_model_type = 1  # OCAM: not implemented
    with pytest.raises(TripsError) as e:
        blend(info)
    assert e.value.status == -4
    info.images[0].camera_model_type = 0
    info.num_layers = 9
    with pytest.raises(TripsError):
        blend(info)
    info.num_layers = 4
    with torch.no_grad():
        outs = blend(info)
    with pytest.raises(TripsError) as e:  # backward after an inference forward
        BlendPointCloudBackward(None, info, [torch.zeros_like(o) for o in outs])
    assert e.value.status == -5


def test_config2_full_size_properties(cuda_lib):
    """Config 2 in full (2 M points, 4 views 1280x720, 6 layers, K = 16): size-independent properties, in addition to the
    element-wise comparison of test_gpu_fullsize.py.  (1) the counters agree with one another; (2) every
    kept list is sorted by (depth, point id) and has min(length, K) elements; (3) the forward pass is deterministic bit
    for bit although list slots are handed out by atomics; (4) the backward pass is linear in the incoming gradient;
    (5) a zero gradient gives zero gradients."""
    import torch
    from trips_b200 import scenes
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.renderer import NeuralRenderInfo, PointRendererCache, RenderParams
    from trips_b200.scenes import layer_sizes
    s = scenes.config2()
    dev = torch.device("cuda")
    ns = NeuralScene.from_synthetic(s, device=dev)
    pc, tex = ns.point_cloud_cuda, ns.texture
    cache = PointRendererCache(dev)
    views = list(range(s.n_views))
    info = NeuralRenderInfo(scene=ns, images=images_for(s, views), params=RenderParams(num_texture_channels=s.channels, k_keep=s.k_keep),
                            num_layers=s.num_layers, train=True, cache=cache)
    args = (tex.texture, tex.background_color, pc.t_position, ns.intrinsics.intrinsics, tex.confidence_value_of_point, pc.t_point_size,
            pc.t_index, ns.poses.poses_se3)
    outs = [o.clone() for o in cache.forward(info, *args)]
    assert cache.last_status() == 0
    st = cache.stats()
    B, K = len(views), s.k_keep
    P = sum(w * h for w, h in layer_sizes(s.width, s.height, s.num_layers))
    # (1), (2) on every view: list lengths, kept counts, sortedness
    total_f = total_k = 0
    for b in range(B):
        counts, offsets, _ = cache.debug_lists(b, P)
        nrec, rec_pid, rec_alpha = cache.debug_records(b, P)
        depth, nl, _ = cache.debug_points(b, s.n_points)
        total_f += int(counts.sum())
        total_k += int(np.minimum(counts, K).sum())
        assert int(nl.sum()) * 4 == int(counts.sum()), "every (point, layer) pair writes exactly four fragments"
        assert np.all(nrec <= np.minimum(counts, K))
        idx = np.arange(16)[None, :] < nrec[:, None]
        d = np.where(idx, depth[np.clip(rec_pid, 0, s.n_points - 1)], np.inf)
        assert np.all(d[:, 1:] >= d[:, :-1]), "records must be in depth order"
        ties = idx[:, 1:] & (d[:, 1:] == d[:, :-1])
        assert np.all(rec_pid[:, 1:][ties] > rec_pid[:, :-1][ties]), "equal depths are ordered by point id"
        assert np.all((rec_alpha[idx] >= 0) & (rec_alpha[idx] <= 1))
    assert st["fragments"] == total_f and st["kept_fragments"] == total_k
    # (3) determinism
    outs2 = cache.forward(info, *args)
    for a, c in zip(outs, outs2):
        assert torch.equal(a, c)
    # (4), (5) linearity of the backward pass
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    g1 = [torch.randn(o.shape, device=dev, generator=gen) for o in outs]
    names = ("texture", "background", "points", "pose", "intrinsics", "confidence", "point_size")
    as_dict = lambda t: {k: v.clone() for k, v in zip(names, t) if v is not None}  # noqa: E731
    r1 = as_dict(cache.backward(g1, *args))
    r2 = as_dict(cache.backward([2.0 * g for g in g1], *args))
    r0 = as_dict(cache.backward([torch.zeros_like(g) for g in g1], *args))
    for k, v in r1.items():
        scale = float(v.abs().max())
        assert scale > 0, k
        assert float((r2[k] - 2.0 * v).abs().max()) <= 1e-4 * 2.0 * scale, f"{k}: backward is not linear"
        assert float(r0[k].abs().max()) == 0.0, f"{k}: zero in, zero out"


@pytest.mark.parametrize("with_index", [False, True])
def test_fused_texture_preparation(oracle_lib, cuda_lib, with_index):
    """confidence = sigmoid(10 * raw) and descriptor = |raw| computed inside the rasterizer (NeuralTexture.h:40-57):
    the scene holds raw parameters; the oracle renders the activated copy.  Forward: the usual bars.  Backward: the
    gradients arrive at the raw parameters, i.e. the oracle's gradients times the activation derivatives."""
    import copy

    import torch
    s_raw = scenes.tiny(seed=77, n_points=5000)
    rng = np.random.default_rng(77)
    s_raw.confidence[:] = rng.normal(0.0, 0.25, s_raw.confidence.shape).astype(np.float32)
    s_raw.texture[:] = rng.uniform(-1.0, 1.0, s_raw.texture.shape).astype(np.float32)
    s_raw.texture[:, :7] = 0.0  # |x| at 0: torch.abs passes no gradient there
    scale = 10.0
    s_act = copy.deepcopy(s_raw)
    s_act.confidence[:] = oracle_lib.sigmoid(s_raw.confidence, scale).reshape(s_raw.confidence.shape)
    s_act.texture[:] = np.abs(s_raw.texture)
    index = rng.permutation(s_raw.n_points).astype(np.int32) if with_index else None
    _, _, frames = oracle_frames(s_act, train=True, index=index)
    ns, info, blend = gpu_render(s_raw, train=True, index=index, confidence_is_raw=True, confidence_scale=scale, texture_abs=True)
    for t in (ns.texture.texture_raw, ns.texture.confidence_raw, ns.point_cloud_cuda.t_position):
        t.requires_grad_(True)
    outs = blend(info)
    assert info.cache.last_status() == 0
    C = s_raw.channels
    loss, ref_tex, ref_conf = 0, 0, 0
    for b, f in enumerate(frames):
        nrec, pid, alpha = info.cache.debug_records(b, f.P)
        onrec, opid, oalpha = f.records()
        assert np.array_equal(nrec, onrec) and np.array_equal(pid, opid)
        opyr = f.pyramid()
        for l, o in enumerate(outs):
            got = o[b].detach().cpu().numpy()
            assert np.max(np.abs(got - opyr[l]) / np.maximum(np.abs(opyr[l]), 1e-3)) <= TOL_PYRAMID
        g = scenes.target_gradient(s_raw, b)
        for l, (w, h, base) in enumerate(f.layers):
            loss = loss + (outs[l][b] * torch.from_numpy(g[C * base:C * (base + w * h)].reshape(C, h, w)).cuda()).sum()
        r = f.backward(g)
        ref_tex, ref_conf = ref_tex + r["texture"], ref_conf + r["confidence"]
    loss.backward()
    sg = s_act.confidence.reshape(-1).astype(np.float64)
    ref_conf_raw = ref_conf.reshape(-1) * (scale * sg * (1.0 - sg))
    ref_tex_raw = ref_tex * np.sign(s_raw.texture)
    assert rel_err(ns.texture.confidence_raw.grad.reshape(-1).cpu().numpy(), ref_conf_raw) <= TOL_GRAD
    assert rel_err(ns.texture.texture_raw.grad.cpu().numpy(), ref_tex_raw) <= TOL_GRAD
    assert np.all(ns.texture.texture_raw.grad[:, :7].cpu().numpy() == 0)


def _render_pair(s, okw, gkw, dropout=None, train=True):
    """Oracle frames and GPU outputs of one scene with the given flags; dropout: [views, points] mask or None."""
    import torch
    frames = []
    for v in range(s.n_views):
        import oracle
        sa = oracle.SceneArrays.from_scene(s, dropout=None if dropout is None else dropout[v])
        p = oracle.make_params(s.num_layers, s.k_keep, train, **okw)
        frames.append(oracle.forward(sa, oracle.make_view(s.width, s.height, s.poses[v], s.intrinsics[v]), p))
    ns, info, blend = gpu_render(s, train=train, **gkw)
    if dropout is not None:
        info.cache.dropout_points = torch.from_numpy(np.ascontiguousarray(dropout, dtype=np.float32)).cuda()
    return frames, ns, info, blend


def _compare_forward(s, frames, info, outs, train=True):
    for b, f in enumerate(frames):
        depth, nl, _ = info.cache.debug_points(b, s.n_points)
        odepth, onl, _ = f.points()
        assert np.array_equal(depth.view(np.uint32), odepth.view(np.uint32)), "depth differs"
        assert np.array_equal(nl, onl), "layer counts differ"
        counts, offsets, frags = info.cache.debug_lists(b, f.P)
        ocounts, ooffsets, ofrags = f.lists()
        assert np.array_equal(counts, ocounts) and np.array_equal(offsets, ooffsets)
        assert np.array_equal(sort_lists(counts, offsets, frags), ofrags), "fragment lists differ"
        if train:
            nrec, pid, alpha = info.cache.debug_records(b, f.P)
            onrec, opid, oalpha = f.records()
            assert np.array_equal(nrec, onrec) and np.array_equal(pid, opid)
        for l, o in enumerate(f.pyramid()):
            got = outs[l][b].detach().cpu().numpy()
            assert np.max(np.abs(got - o) / np.maximum(np.abs(o), 1e-3)) <= TOL_PYRAMID


def test_viewer_only_discards_unstable_points(oracle_lib, cuda_lib):
    """viewer_only with a stability cut-off inside the range of the confidences: points below it are not drawn
    (discard_point_for_confidence, RenderForward.cu:122-130, 224-229).  Inference render, as the viewer does."""
    import torch
    s = scenes.tiny(seed=41, n_points=6000)
    cut = 0.45
    assert 0.2 < float((s.confidence < cut).mean()) < 0.8
    flags = dict(viewer_only=True, stability_cutoff_value=cut)
    frames, ns, info, blend = _render_pair(s, flags, flags, train=False)
    with torch.no_grad():
        outs = blend(info)
    assert info.cache.last_status() == 0
    _compare_forward(s, frames, info, outs, train=False)
    kept = s.confidence.reshape(-1) >= cut
    for b, f in enumerate(frames):
        depth, _, _ = info.cache.debug_points(b, s.n_points)
        assert np.all(depth[~kept] == -1.0), "a point below the cut-off was drawn"
        assert (depth[kept] > 0).any()


def test_fixed_dropout_mask(oracle_lib, cuda_lib):
    """A drop-out mask handed to both sides (RenderForward.cu:230-240: a point whose mask value is 1 is skipped in that
    view, training only): forward intermediates bit for bit, gradients within tolerance, masked points get no gradient
    from the views that dropped them."""
    import torch
    s = scenes.tiny(seed=42, n_points=5000, n_views=3)
    rng = np.random.default_rng(42)
    mask = (rng.random((s.n_views, s.n_points)) < 0.35).astype(np.float32)
    frames, ns, info, blend = _render_pair(s, {}, {}, dropout=mask)
    for t in (ns.texture.texture_raw, ns.texture.confidence_raw, ns.point_cloud_cuda.t_position, ns.point_cloud_cuda.t_point_size):
        t.requires_grad_(True)
    outs = blend(info)
    assert info.cache.last_status() == 0
    _compare_forward(s, frames, info, outs)
    for b in range(s.n_views):
        depth, _, _ = info.cache.debug_points(b, s.n_points)
        assert np.all(depth[mask[b] == 1.0] == -1.0)
    C = s.channels
    loss, ref = 0, None
    for b, f in enumerate(frames):
        g = scenes.target_gradient(s, b)
        for l, (w, h, base) in enumerate(f.layers):
            loss = loss + (outs[l][b] * torch.from_numpy(g[C * base:C * (base + w * h)].reshape(C, h, w)).cuda()).sum()
        r = f.backward(g)
        ref = r if ref is None else {k: ref[k] + r[k] for k in r}
    loss.backward()
    got = dict(texture=ns.texture.texture_raw.grad, confidence=ns.texture.confidence_raw.grad.reshape(-1),
               position=ns.point_cloud_cuda.t_position.grad, point_size=ns.point_cloud_cuda.t_point_size.grad.reshape(-1))
    for k, g_ in got.items():
        assert rel_err(g_.cpu().numpy(), ref[k]) <= TOL_GRAD, k
    always = mask.min(axis=0) == 1.0  # dropped in every view
    assert always.any()
    assert np.all(ns.point_cloud_cuda.t_position.grad.cpu().numpy()[always] == 0)


def test_normalize_grads_changes_nothing(cuda_lib):
    """normalize_grads = true divides the point / pose / intrinsics gradients by hit counts that the reference
    allocates as zeros and never increments (PointRenderer.cu:226-272; no kernel writes out_gradient_*_count), so its
    `if (c > 0)` guard (PointRenderer.cu:1193-1230) never passes: the flag is accepted and the gradients are unchanged."""
    import torch
    s = scenes.tiny(seed=43, n_points=3000)
    res = []
    for flag in (False, True):
        ns, info, blend = gpu_render(s, train=True, normalize_grads=flag)
        ns.point_cloud_cuda.t_position.requires_grad_(True)
        ns.poses.tangent_poses.requires_grad_(True)
        outs = blend(info)
        sum((o * o).sum() for o in outs).backward()
        res.append((ns.point_cloud_cuda.t_position.grad.clone(), ns.poses.tangent_poses.grad.clone()))
    # (gradients are sums of atomics in arbitrary order: compare within the gradient tolerance)
    assert rel_err(res[1][0].cpu().numpy(), res[0][0].cpu().numpy()) <= TOL_GRAD
    assert rel_err(res[1][1].cpu().numpy(), res[0][1].cpu().numpy()) <= TOL_GRAD


def test_status_bits_survive_later_calls(cuda_lib):
    """A device status bit raised by one call is still reported after later forward calls on the context; reading it
    clears it.  (The reference would have asserted in the first call, RenderBackward.cu:217-218.)"""
    import torch
    from trips_b200 import _lib
    s = scenes.tiny(seed=44, n_points=800)
    bad = np.arange(s.n_points, dtype=np.int32)
    bad[5] = s.n_points + 7  # texture column out of range
    ns, info, blend = gpu_render(s, train=False, index=bad)
    with torch.no_grad():
        blend(info)
        ns.point_cloud_cuda.t_index = torch.arange(s.n_points, dtype=torch.int32, device="cuda").reshape(-1, 1)
        blend(info)  # a clean call afterwards must not erase the bit
    assert info.cache.last_status() & _lib.DEV_BAD_TEXTURE_INDEX
    assert info.cache.last_status() == 0


def test_steady_state_sizing_and_overflow(oracle_lib, cuda_lib):
    """Training calls with unchanged shapes size the entry and fragment buffers from the previous call (x 1.25) and do
    not wait for their own counts.  (1) A repeated call renders the same bits as the first, sized call.  (2) When the
    point cloud suddenly needs far more fragments than the buffers hold, the views that do not fit are rendered as
    background, the status word says so, nothing is written out of bounds, and the next call - whose buffers were grown
    from the reported need - is exact again."""
    import torch
    from trips_b200 import _lib
    # (enough fragments to exceed the list buffer's initial 16 MB: the buffers are then sized from the counts)
    s = scenes.tiny(seed=45, n_points=200000, n_views=2, width=160, height=120, size_range=(5e-3, 0.02))
    ns, info, blend = gpu_render(s, train=True)
    with torch.no_grad():
        first = [o.clone() for o in blend(info)]          # sized call (waits for its counts)
        again = [o.clone() for o in blend(info)]          # steady state
        for a, b_ in zip(first, again):
            assert torch.equal(a, b_)
        assert info.cache.last_status() == 0
        f_small = info.cache.stats()["fragments"]
        assert f_small * 16 > 16 * 1024 * 1024
        # the same points, four pyramid layers larger each: many times the fragments, same shapes
        ns.point_cloud_cuda.t_point_size.data += 3.0
        over = [o.clone() for o in blend(info)]
        status = info.cache.last_status()
        assert status & (_lib.DEV_FRAGMENT_OVERFLOW | _lib.DEV_ENTRY_OVERFLOW), "the overflow must be reported"
        assert info.cache.stats()["fragments"] > 1.25 * f_small
        bg = ns.texture.background_color.detach()
        for o in over:  # views that did not fit show the background colour only
            flat = o.permute(0, 2, 3, 1).reshape(o.shape[0], -1, o.shape[1])
            empty = (flat == bg).all(dim=2).all(dim=1)
            assert bool(empty.any())
        exact = [o.clone() for o in blend(info)]          # buffers grown from the reported need
        assert info.cache.last_status() == 0
    s2 = scenes.tiny(seed=45, n_points=200000, n_views=2, width=160, height=120, size_range=(5e-3, 0.02))
    s2.point_size[:] = s2.point_size + np.float32(3.0)
    _, _, frames = oracle_frames(s2, train=True)
    for b, f in enumerate(frames):
        for l, o in enumerate(f.pyramid()):
            got = exact[l][b].cpu().numpy()
            assert np.max(np.abs(got - o) / np.maximum(np.abs(o), 1e-3)) <= TOL_PYRAMID
