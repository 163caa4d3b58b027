"""The libtorch host side (trips_b200/csrc/torch_shim.cpp): NeuralRenderInfo / PointRender / BlendPointCloud in C++ on
top of the C ABI.  CPU: the library builds, loads and registers its class and operator.  GPU: the C++ operator gives
the Python mirror's outputs bit for bit, and autograd reaches the same gradients."""
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
    with pytest.raises(RuntimeError):
        info.add_image(96, 64, 0, 0, 0, [1.0], [1.0, 0.0, 0.0, 1.0])


@pytest.mark.gpu
def test_shim_matches_python_mirror(shim, cuda_lib):
    torch = shim
    from trips_b200 import scenes
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.renderer import BlendPointCloud, NeuralRenderInfo, PointRendererCache, RenderParams
    s = scenes.tiny(n_points=5000, seed=9, width=96, height=64, num_layers=4, n_views=2)
    dev = torch.device("cuda")

    def leaves(ns):
        pc, tex = ns.point_cloud_cuda, ns.texture
        return {"texture": tex.texture_raw, "confidence": tex.confidence_raw, "points": pc.t_position, "size": pc.t_point_size,
                "background": tex.background_color_raw}

    # Python mirror
    ns = NeuralScene.from_synthetic(s, device=dev)
    info = NeuralRenderInfo(scene=ns, images=images_for(s, [0, 1]), params=RenderParams(num_texture_channels=s.channels, k_keep=s.k_keep),
                            num_layers=s.num_layers, train=True, cache=PointRendererCache(dev))
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
    cinfo.set_scene(tex.texture, tex.background_color, pc.t_position, ns2.poses.poses_se3, ns2.intrinsics.intrinsics,
                    tex.confidence_value_of_point, pc.t_point_size, pc.t_index)
    for im in images_for(s, [0, 1]):
        cinfo.add_image(im.w, im.h, im.image_index, im.camera_index, im.camera_model_type, [float(x) for x in im.crop_transform],
                        [float(x) for x in im.crop_rotation])
    cinfo.set_params(s.num_layers, s.k_keep, True, False, 0.0, False, 0.0, False, 0.0)
    couts = torch.ops.trips_b200.blend_point_cloud(cinfo, torch.empty(0, device=dev, dtype=torch.float64))
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
