"""The libtorch host side (trips_b200/csrc/torch_shim.{h,cpp}): NeuralRenderInfo / PointRender / BlendPointCloud /
PointRenderModule / MyAdam in C++ on top of the C ABI.  CPU: the library builds, loads and registers its classes and
operators.  GPU: the C++ operator gives the Python mirror's outputs bit for bit, autograd reaches the same gradients,
and the C++ optimizer with its state surgery matches the Python mirror bit for bit."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def shim():
    import torch
    from trips_b200 import build
    path = build.build_torch_shim()
    torch.ops.load_library(path)
    return torch


def test_shim_registers_class_and_operator(shim):
    torch = shim
    info = torch.classes.trips_b200.NeuralRenderInfo()
    info.set_params(4, 16, True, False, 0.0, False, 0.0, False, 0.0)
    info.add_image(96, 64, 0, 0, 0, [1.0, 1.0, 0.0, 0.0, 0.0], [1.0, 0.0, 0.0, 1.0])
    info.clear_images()
    assert info.last_status() == 0  # no context yet: nothing raised
    assert hasattr(torch.ops.trips_b200, "blend_point_cloud") and hasattr(torch.ops.trips_b200, "adam_step")
    info.set_texture_preparation(True, 10.0, True)
    info.set_pipeline_flags(True, False, True, False)
    info.set_distortion(True, 20.0)
    assert torch.classes.trips_b200.PointRenderModule(4) is not None
    opt = torch.classes.trips_b200.MyAdam()
    with pytest.raises(RuntimeError):
        opt.step()  # no param group yet
    with pytest.raises(RuntimeError):
        info.add_image(96, 64, 0, 0, 0, [1.0], [1.0, 0.0, 0.0, 1.0])


# (use_layer_point_size, render_points_in_all_lower_resolutions, combine_lists, saturated_alpha_accumulation): the
# reference's defaults, and a combination that selects its second forward pipeline
@pytest.mark.gpu
# the fifth entry: lens distortion
@pytest.mark.parametrize("flags", [(True, True, False, False, False), (True, False, True, True, False), (True, True, False, False, True)],
                         ids=["first_pipeline", "second_pipeline", "lens_distortion"])
def test_shim_matches_python_mirror(shim, cuda_lib, flags):
    torch = shim
    from trips_b200 import scenes
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.renderer import BlendPointCloud, NeuralRenderInfo, PointRendererCache, RenderParams
    s = scenes.tiny(n_points=5000, seed=9, width=96, height=64, num_layers=4, n_views=2)
    if flags[4]:
        s.intrinsics[:, 5:] = np.array([-0.1, 0.04, 0.0, 0.02, 0.0, 0.0, 2e-3, -1e-3], np.float32)
    dev = torch.device("cuda")

    def leaves(ns):
        pc, tex = ns.point_cloud_cuda, ns.texture
        return {"texture": tex.texture_raw, "confidence": tex.confidence_raw, "points": pc.t_position, "size": pc.t_point_size,
                "background": tex.background_color_raw}

    # Python mirror
    ns = NeuralScene.from_synthetic(s, device=dev)
    params = RenderParams(num_texture_channels=s.channels, k_keep=s.k_keep, use_layer_point_size=flags[0],
                          render_points_in_all_lower_resolutions=flags[1], combine_lists=flags[2], saturated_alpha_accumulation=flags[3],
                          distortion=flags[4], dist_cutoff=0.6)
    info = NeuralRenderInfo(scene=ns, images=images_for(s, [0, 1]), params=params, num_layers=s.num_layers, train=True,
                            cache=PointRendererCache(dev))
    outs = BlendPointCloud(info)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    gs = [torch.randn(o.shape, device=dev, generator=gen) for o in outs]
    torch.autograd.backward(outs, gs)
    ref_out = [o.detach().clone() for o in outs]
    ref_grad = {k: v.grad.detach().clone() for k, v in leaves(ns).items() if v.grad is not None}

    # C++ shim on a fresh copy of the same scene
    ns2 = NeuralScene.from_synthetic(s, device=dev)
    pc, tex = ns2.point_cloud_cuda, ns2.texture
    cinfo = torch.classes.trips_b200.NeuralRenderInfo()
    cinfo.set_scene(tex.texture, tex.background_color, pc.t_position, ns2.poses.poses_se3, None, ns2.intrinsics.intrinsics,
                    tex.confidence_value_of_point, pc.t_point_size, pc.t_index)
    for im in images_for(s, [0, 1]):
        cinfo.add_image(im.w, im.h, im.image_index, im.camera_index, im.camera_model_type, [float(x) for x in im.crop_transform],
                        [float(x) for x in im.crop_rotation])
    cinfo.set_params(s.num_layers, s.k_keep, True, False, 0.0, False, 0.0, False, 0.0)
    cinfo.set_pipeline_flags(*flags[:4])
    cinfo.set_distortion(flags[4], 0.6)
    couts = torch.ops.trips_b200.blend_point_cloud(cinfo)  # BlendPointCloud(NeuralRenderInfo*), RenderInfo.cpp:27
    assert cinfo.last_status() == 0
    assert len(couts) == len(ref_out)
    for a, b in zip(couts, ref_out):
        assert torch.equal(a, b)
    torch.autograd.backward(couts, gs)
    got = {k: v.grad for k, v in leaves(ns2).items() if v.grad is not None}
    assert set(got) == set(ref_grad) and len(got) >= 4
    for k, v in ref_grad.items():
        scale = float(v.abs().max())
        assert float((got[k] - v).abs().max()) <= 1e-4 * max(scale, 1e-30), k


@pytest.mark.gpu
def test_shim_adam_step_matches_python_myadam(shim, cuda_lib):
    torch = shim
    from trips_b200.optim import MyAdam
    from trips_b200.renderer import PointRendererCache
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    shapes = [(4, 3001), (1, 3001), (3001, 4), (3001, 1)]
    ws = [torch.randn(s, device=dev, generator=gen) for s in shapes]
    ref = [torch.nn.Parameter(w.clone()) for w in ws]
    opt = MyAdam(ref, lr=1e-3, betas=(0.9, 0.999), cache=PointRendererCache(dev))
    m = [torch.zeros_like(w) for w in ws]
    v = [torch.zeros_like(w) for w in ws]
    st = [torch.zeros(w.shape, dtype=torch.int32, device=dev) for w in ws]
    for _ in range(3):
        gs = [torch.randn(w.shape, device=dev, generator=gen) * (torch.rand(w.shape, device=dev, generator=gen) < 0.5) for w in ws]
        for p, g in zip(ref, gs):
            p.grad = g.clone()
        opt.step()
        torch.ops.trips_b200.adam_step(ws, gs, m, v, st, 1e-3, 0.9, 0.999, 1e-8)
    for w, p in zip(ws, ref):
        assert torch.equal(w, p.detach())  # the same kernel behind both host sides
    assert int(st[0].max()) == 3 and int(st[0].min()) >= 0


@pytest.mark.gpu
def test_shim_module_pose_gradient_and_fused_preparation(shim, cuda_lib):
    """PointRenderModule::forward(NeuralRenderInfo*) (RenderModule.cpp:44-110) with the pose tangents inside the info object
    and the texture preparation fused: outputs and gradients equal the Python mirror's."""
    torch = shim
    from trips_b200 import scenes
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.renderer import BlendPointCloud, NeuralRenderInfo, PointRendererCache, RenderParams
    s = scenes.tiny(n_points=3000, seed=19, n_views=2)
    s.confidence[:] = (s.confidence - 0.5) * 0.2  # raw parameters
    dev = torch.device("cuda")
    kw = dict(confidence_is_raw=True, confidence_scale=10.0, texture_abs=True)
    ns = NeuralScene.from_synthetic(s, device=dev)
    ns.poses.tangent_poses.requires_grad_(True)
    info = NeuralRenderInfo(scene=ns, images=images_for(s, [0, 1]), params=RenderParams(num_texture_channels=s.channels, k_keep=s.k_keep, **kw),
                            num_layers=s.num_layers, train=True, cache=PointRendererCache(dev))
    outs = BlendPointCloud(info)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    gs = [torch.randn(o.shape, device=dev, generator=gen) for o in outs]
    torch.autograd.backward(outs, gs)

    ns2 = NeuralScene.from_synthetic(s, device=dev)
    ns2.poses.tangent_poses.requires_grad_(True)
    pc, tex = ns2.point_cloud_cuda, ns2.texture
    cinfo = torch.classes.trips_b200.NeuralRenderInfo()
    cinfo.set_scene(tex.texture, tex.background_color, pc.t_position, ns2.poses.poses_se3, ns2.poses.tangent_poses, ns2.intrinsics.intrinsics,
                    tex.confidence_value_of_point, pc.t_point_size, pc.t_index)
    for im in images_for(s, [0, 1]):
        cinfo.add_image(im.w, im.h, im.image_index, im.camera_index, im.camera_model_type, [float(x) for x in im.crop_transform],
                        [float(x) for x in im.crop_rotation])
    cinfo.set_params(1, s.k_keep, False, False, 0.0, False, 0.0, False, 0.0)  # layers and train come from the module
    cinfo.set_texture_preparation(True, 10.0, True)
    module = torch.classes.trips_b200.PointRenderModule(s.num_layers)
    module.train(True)
    couts = module.forward(cinfo)
    assert len(couts) == s.num_layers
    for a, b in zip(couts, outs):
        assert torch.equal(a, b.detach())
    torch.autograd.backward(couts, gs)
    for a, b in ((ns2.poses.tangent_poses.grad, ns.poses.tangent_poses.grad), (tex.texture_raw.grad, ns.texture.texture_raw.grad),
                 (tex.confidence_raw.grad, ns.texture.confidence_raw.grad)):
        assert a is not None and b is not None
        assert float((a - b).abs().max()) <= 1e-4 * max(float(b.abs().max()), 1e-30)


@pytest.mark.gpu
def test_shim_myadam_class_and_state_surgery(shim, cuda_lib):
    """torch::optim::MyAdam in C++ (options per group, step, shrinkInternalState, appendToInternalState; MyAdam.h:50-85,
    MyAdam.cu:346-415) against the Python mirror: weights and state bit for bit over steps, a shrink and a growth."""
    torch = shim
    from trips_b200.optim import MyAdam
    from trips_b200.renderer import PointRendererCache
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev)
    gen.manual_seed(21)
    n = 2003
    shapes = [(4, n), (1, n), (5,)]
    init = [torch.randn(s, device=dev, generator=gen) for s in shapes]
    ref = [torch.nn.Parameter(w.clone()) for w in init]
    mine = [w.clone().requires_grad_(True) for w in init]
    groups = [dict(lr=1e-3), dict(lr=5e-3, relative_weight_decay=0.01, absolute_weight_decay=0.001, weight_clipping_magnitude=2.5),
              dict(lr=2e-3, adabound=True)]
    opt = MyAdam([dict(params=[p], **g) for p, g in zip(ref, groups)], cache=PointRendererCache(dev))
    copt = torch.classes.trips_b200.MyAdam()
    for p, g in zip(mine, groups):
        copt.add_param_group([p], g["lr"], 0.9, 0.999, 1e-8, g.get("relative_weight_decay", 0.0), g.get("absolute_weight_decay", 0.0),
                             g.get("weight_clipping_magnitude", 0.0), g.get("adabound", False))
    assert copt.state(0, 0) == []

    def one_step():
        for p, q in zip(ref, mine):
            g = torch.randn(p.shape, device=dev, generator=gen) * (torch.rand(p.shape, device=dev, generator=gen) < 0.6)
            p.grad, q.grad = g.clone(), g.clone()
        opt.step()
        copt.step()

    def same():
        for gi, (p, q) in enumerate(zip(ref, mine)):
            assert torch.equal(p.detach(), q.detach())
            st = copt.state(gi, 0)
            for a, k in zip(st, ("first_moments", "second_moments", "param_steps")):
                assert torch.equal(a, opt.state[p][k]) and a.dtype == opt.state[p][k].dtype

    for _ in range(3):
        one_step()
    same()
    # remove a third of the columns of the per-point tensors (groups 0 and 1), as NeuralScene::RemovePoints does
    keep = torch.nonzero(torch.rand(n, device=dev, generator=gen) > 0.33).reshape(-1)
    with torch.no_grad():
        for gi in (0, 1):
            opt.shrinkInternalState(gi, keep)
            copt.shrinkInternalState(gi, keep)
            ref[gi].data = ref[gi].data.index_select(1, keep).contiguous()
            mine[gi].data = mine[gi].data.index_select(1, keep).contiguous()
    one_step()
    same()
    # grow by 100 points
    new_n = keep.numel() + 100
    with torch.no_grad():
        for gi in (0, 1):
            opt.appendToInternalState(gi, new_n)
            copt.appendToInternalState(gi, new_n)
            pad = torch.full((ref[gi].shape[0], 100), 0.5, device=dev)
            ref[gi].data = torch.cat([ref[gi].data, pad], 1).contiguous()
            mine[gi].data = torch.cat([mine[gi].data, pad], 1).contiguous()
    one_step()
    same()
    copt.scale_lr(0.5)
    for g in opt.param_groups:
        g["lr"] *= 0.5
    one_step()
    same()
