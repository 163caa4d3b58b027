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
    a.scene_name = "playground"
    checkpoint.SaveCheckpoint(a, str(tmp_path), optimizers=[opt])
    # <dir>/scene_<scene name>_<module>.pth, NeuralScene.cpp:535,597
    pre = "scene_playground_"
    assert sorted(f.name for f in tmp_path.iterdir()) == [pre + n for n in ("intrinsics.pth", "optimizer.pth", "points.pth", "poses.pth", "texture.pth")]
    # the archives are TorchScript modules whose attributes carry the reference's names
    pts = torch.jit.load(str(tmp_path / (pre + "points.pth")))
    assert {k for k, _ in pts.named_parameters()} == {"t_position", "t_point_size"}
    assert {k for k, _ in pts.named_buffers()} == {"t_index", "t_original_color"}
    txt = torch.jit.load(str(tmp_path / (pre + "texture.pth")))
    assert {k for k, _ in txt.named_parameters()} == {"texture", "background_color", "confidence_value_of_point"}
    assert {k for k, _ in torch.jit.load(str(tmp_path / (pre + "poses.pth"))).named_buffers()} == {"poses_se3"}
    assert {k for k, _ in torch.jit.load(str(tmp_path / (pre + "intrinsics.pth"))).named_parameters()} == {"intrinsics"}
    # a scene of another size takes over everything, optimizer state included
    b = _scene(120, 2)
    pcb, texb = b.point_cloud_cuda, b.texture
    optb = MyAdam([texb.texture_raw, texb.confidence_raw, pcb.t_position, pcb.t_point_size], lr=1e-3, cache=None)
    assert checkpoint.LoadCheckpoint(b, str(tmp_path), optimizers=[optb]) == []  # another scene name: nothing is found, nothing is read
    b.scene_name = "playground"
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
    a.scene_name = b.scene_name = "s"
    checkpoint.SaveCheckpoint(a, str(tmp_path))
    (tmp_path / "scene_s_texture.pth").unlink()
    before = b.texture.texture_raw.detach().clone()
    assert "texture.pth" not in checkpoint.LoadCheckpoint(b, str(tmp_path))
    assert torch.equal(b.texture.texture_raw.detach(), before)
    assert torch.equal(b.point_cloud_cuda.t_position.detach(), a.point_cloud_cuda.t_position.detach())


def test_checkpoints_load_in_libtorch_and_back(tmp_path):
    """The files written by SaveCheckpoint are read by a libtorch program with torch::load into modules that register
    the reference's names (tests/libtorch_checkpoint.cpp), every tensor arrives with its dtype, size and content, and the
    files that program writes with torch::save are read back by LoadCheckpoint: the format is the reference's in both
    directions."""
    import os
    import shutil
    import subprocess
    from torch.utils import cpp_extension as ce
    from trips_b200 import build, checkpoint
    shim = build.build_torch_shim()
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / "libtorch_checkpoint")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    cmd = [cxx, "-O1", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-I", os.path.join(here, "..", "include"),
           "-I", os.path.join(here, "..", "trips_b200", "csrc")]
    for inc in ce.include_paths("cuda"):
        cmd += ["-isystem", inc]
    cmd += [os.path.join(here, "libtorch_checkpoint.cpp"), "-o", exe, "-L", os.path.dirname(shim), "-ltrips_b200_torch", "-ltrips_b200",
            f"-Wl,-rpath,{os.path.dirname(shim)}"]
    for lp in ce.library_paths("cuda"):
        cmd += ["-L", lp, f"-Wl,-rpath,{lp}"]
    cmd += ["-lc10", "-ltorch_cpu", "-ltorch"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]

    a = _scene(257, 5)
    a.scene_name = "src"
    with torch.no_grad():
        a.poses.tangent_poses.copy_(torch.randn(a.poses.tangent_poses.shape, dtype=torch.float64))
    src, dst = tmp_path / "a", tmp_path / "b"
    dst.mkdir()
    checkpoint.SaveCheckpoint(a, str(src))
    pc, tex = a.point_cloud_cuda, a.texture
    r = subprocess.run([exe, checkpoint.checkpoint_prefix(a, str(src)), str(pc.t_position.shape[0]), str(tex.texture_raw.shape[0]),
                        str(a.poses.poses_se3.shape[0]), str(a.intrinsics.intrinsics.shape[0]), str(dst / "scene_src_")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    seen = {ln.split()[0]: ln.split()[1:] for ln in r.stdout.strip().splitlines()}
    expect = {"t_position": pc.t_position, "t_point_size": pc.t_point_size, "t_index": pc.t_index, "t_original_color": pc.t_original_color,
              "texture": tex.texture_raw, "background_color": tex.background_color_raw, "confidence_value_of_point": tex.confidence_raw,
              "tangent_poses": a.poses.tangent_poses, "poses_se3": a.poses.poses_se3, "intrinsics": a.intrinsics.intrinsics}
    names = {torch.float32: "Float", torch.float64: "Double", torch.int32: "Int"}
    for k, t in expect.items():
        dt, numel, total = seen[k]
        assert dt == names[t.dtype] and int(numel) == t.numel(), (k, seen[k])
        assert abs(float(total) - float(t.detach().double().sum())) <= 1e-9 * max(1.0, abs(float(total))), k
    # what libtorch wrote loads here
    b = _scene(11, 6)
    b.scene_name = "src"
    assert len(checkpoint.LoadCheckpoint(b, str(dst))) == 4
    for k, t in expect.items():
        got = {"t_position": b.point_cloud_cuda.t_position, "t_point_size": b.point_cloud_cuda.t_point_size, "t_index": b.point_cloud_cuda.t_index,
               "t_original_color": b.point_cloud_cuda.t_original_color, "texture": b.texture.texture_raw,
               "background_color": b.texture.background_color_raw, "confidence_value_of_point": b.texture.confidence_raw,
               "tangent_poses": b.poses.tangent_poses, "poses_se3": b.poses.poses_se3, "intrinsics": b.intrinsics.intrinsics}[k]
        assert got.dtype == t.dtype and torch.equal(got.detach().cpu(), t.detach().cpu()), k
