"""Checkpoint files carry the reference's file and tensor names (NeuralScene.cpp:533-628, NeuralPointCloudCuda.cpp:103-108,
NeuralTexture.cpp:53-55, NeuralStructure.cpp:34-35,142) and round-trip, including the Adam state the reference cannot save."""
import numpy as np
import torch


def _scene(n, seed):
    from trips_b200 import scenes
    from trips_b200.modules import NeuralScene
    return NeuralScene.from_synthetic(scenes.tiny(n_points=n, seed=seed, n_views=2), device="cpu")


def test_checkpoint_names_and_round_trip(tmp_path):
    from trips_b200 import checkpoint
    from trips_b200.optim import MyAdam
    a = _scene(300, 1)
    pc, tex = a.point_cloud_cuda, a.texture
    opt = MyAdam([tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size], lr=1e-3, cache=None)
    g = torch.Generator().manual_seed(0)
    for p in opt.param_groups[0]["params"]:  # state as a few steps would leave it
        opt.state[p] = {"first_moments": torch.randn(p.shape, generator=g), "second_moments": torch.rand(p.shape, generator=g),
                        "param_steps": torch.randint(0, 9, p.shape, generator=g, dtype=torch.int32)}
    checkpoint.SaveCheckpoint(a, str(tmp_path), optimizers=[opt])
    assert sorted(f.name for f in tmp_path.iterdir()) == ["intrinsics.pth", "optimizer.pth", "points.pth", "poses.pth", "texture.pth"]
    # the archives are TorchScript modules whose attributes carry the reference's names
    pts = torch.jit.load(str(tmp_path / "points.pth"))
    assert {k for k, _ in pts.named_parameters()} == {"t_position", "t_point_size"}
    assert {k for k, _ in pts.named_buffers()} == {"t_index", "t_original_color"}
    txt = torch.jit.load(str(tmp_path / "texture.pth"))
    assert {k for k, _ in txt.named_parameters()} == {"texture", "background_color", "confidence_value_of_point"}
    assert {k for k, _ in torch.jit.load(str(tmp_path / "poses.pth")).named_buffers()} == {"poses_se3"}
    assert {k for k, _ in torch.jit.load(str(tmp_path / "intrinsics.pth")).named_parameters()} == {"intrinsics"}
    # a scene of another size takes over everything, optimizer state included
    b = _scene(120, 2)
    pcb, texb = b.point_cloud_cuda, b.texture
    optb = MyAdam([texb.texture_raw, texb.confidence_raw, pcb.t_position, pcb.t_point_size], lr=1e-3, cache=None)
    read = checkpoint.LoadCheckpoint(b, str(tmp_path), optimizers=[optb])
    assert len(read) == 5
    for x, y in ((pc.t_position, pcb.t_position), (pc.t_point_size, pcb.t_point_size), (pc.t_index, pcb.t_index),
                 (tex.texture_raw, texb.texture_raw), (tex.confidence_raw, texb.confidence_raw),
                 (tex.background_color_raw, texb.background_color_raw), (a.poses.poses_se3, b.poses.poses_se3),
                 (a.intrinsics.intrinsics, b.intrinsics.intrinsics)):
        assert x.dtype == y.dtype and torch.equal(x.detach(), y.detach())
    for p, q in zip(opt.param_groups[0]["params"], optb.param_groups[0]["params"]):
        for k in ("first_moments", "second_moments", "param_steps"):
            assert torch.equal(opt.state[p][k], optb.state[q][k]) and opt.state[p][k].dtype == optb.state[q][k].dtype


def test_load_checkpoint_takes_what_exists(tmp_path):
    from trips_b200 import checkpoint
    a, b = _scene(50, 3), _scene(50, 4)
    checkpoint.SaveCheckpoint(a, str(tmp_path))
    (tmp_path / "texture.pth").unlink()
    before = b.texture.texture_raw.detach().clone()
    assert "texture.pth" not in checkpoint.LoadCheckpoint(b, str(tmp_path))
    assert torch.equal(b.texture.texture_raw.detach(), before)
    assert torch.equal(b.point_cloud_cuda.t_position.detach(), a.point_cloud_cuda.t_position.detach())
