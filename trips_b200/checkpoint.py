"""Checkpoints with the reference's file and tensor names.

NeuralScene::SaveCheckpoint / LoadCheckpoint (src/lib/data/NeuralScene.cpp:533-628) write one libtorch archive per
module under the prefix <checkpoint_dir>/scene_<scene name>_ (NeuralScene.cpp:535,597): points.pth (t_position, t_point_size as parameters; t_index, t_original_color as buffers,
NeuralPointCloudCuda.cpp:103-108), texture.pth (texture, background_color, confidence_value_of_point: the RAW
tensors under the names of their activated versions, NeuralTexture.cpp:53-55), poses.pth (tangent_poses, poses_se3,
NeuralStructure.cpp:34-35), intrinsics.pth (intrinsics, NeuralStructure.cpp:142).  A libtorch archive is a
TorchScript module whose attributes carry those names, so it is written here by scripting a container module and read
back with torch.jit.load.  tests/test_checkpoint.py compiles a small libtorch program that torch::load()s the files
written here into modules registering the reference's names, and torch::save()s them back for this side to read.

The reference cannot save optimizer state (MyAdam::save / load abort, MyAdam.cu:417-425); optimizer.pth holds the
three state tensors of every parameter under "<parameter name>.first_moments|second_moments|param_steps".
"""
from __future__ import annotations

import os
from typing import Dict

import torch
from torch import nn

POINTS, TEXTURE, POSES, INTRINSICS, OPTIMIZER = "points.pth", "texture.pth", "poses.pth", "intrinsics.pth", "optimizer.pth"


class _Archive(nn.Module):
    """A module that only carries named tensors (what torch::save(module, path) serialises)."""

    def __init__(self, params: Dict[str, torch.Tensor], buffers: Dict[str, torch.Tensor]):
        super().__init__()
        for k, v in params.items():
            self.register_parameter(k, nn.Parameter(v.detach().clone(), requires_grad=False))
        for k, v in buffers.items():
            self.register_buffer(k, v.detach().clone())

    def forward(self):
        return 0


def _write(path: str, params: Dict[str, torch.Tensor], buffers: Dict[str, torch.Tensor]):
    torch.jit.script(_Archive(params, buffers)).save(path)


def _read(path: str, device=None) -> Dict[str, torch.Tensor]:
    m = torch.jit.load(path, map_location=device)
    out = {k: v.detach() for k, v in m.named_parameters()}
    out.update({k: v for k, v in m.named_buffers()})
    return out


def _state_names(scene) -> Dict[int, str]:
    pc, tex = scene.point_cloud_cuda, scene.texture
    return {id(pc.t_position): "t_position", id(pc.t_point_size): "t_point_size", id(tex.texture_raw): "texture",
            id(tex.confidence_raw): "confidence_value_of_point", id(tex.background_color_raw): "background_color"}


def checkpoint_prefix(scene, checkpoint_dir: str, scene_name=None) -> str:
    """<checkpoint_dir>/scene_<scene name>_ (NeuralScene.cpp:535,597); the name defaults to scene.scene_name."""
    name = scene_name if scene_name is not None else getattr(scene, "scene_name", "scene")
    return os.path.join(checkpoint_dir, f"scene_{name}_")


def SaveCheckpoint(scene, checkpoint_dir: str, optimizers=(), scene_name=None):
    """Writes <prefix>points.pth, texture.pth, poses.pth, intrinsics.pth and, with optimizers, optimizer.pth."""
    os.makedirs(checkpoint_dir, exist_ok=True)
    checkpoint_dir = checkpoint_prefix(scene, checkpoint_dir, scene_name)
    pc, tex = scene.point_cloud_cuda, scene.texture
    p = {"t_position": pc.t_position}
    b = {"t_index": pc.t_index, "t_original_color": pc.t_original_color}
    (p if isinstance(pc.t_point_size, nn.Parameter) else b)["t_point_size"] = pc.t_point_size
    _write(checkpoint_dir + POINTS, p, b)
    _write(checkpoint_dir + TEXTURE, {"texture": tex.texture_raw, "background_color": tex.background_color_raw,
                                                    "confidence_value_of_point": tex.confidence_raw}, {})
    _write(checkpoint_dir + POSES, {"tangent_poses": scene.poses.tangent_poses}, {"poses_se3": scene.poses.poses_se3})
    _write(checkpoint_dir + INTRINSICS, {"intrinsics": scene.intrinsics.intrinsics}, {})
    names = _state_names(scene)
    state = {}
    for opt in optimizers:
        for group in opt.param_groups:
            for q in group["params"]:
                st = opt.state.get(q)
                if st and id(q) in names:
                    for k in ("first_moments", "second_moments", "param_steps"):
                        state[f"{names[id(q)]}.{k}".replace(".", "__")] = st[k]
    if state:
        _write(checkpoint_dir + OPTIMIZER, {}, state)


@torch.no_grad()
def LoadCheckpoint(scene, checkpoint_dir: str, optimizers=(), scene_name=None):
    """Loads whatever of the five files exists under the scene's prefix (as the reference does); tensors are replaced, so
    the number of points may differ from the scene's current one.  Returns the list of files read (without the prefix)."""
    pc, tex = scene.point_cloud_cuda, scene.texture
    prefix = checkpoint_prefix(scene, checkpoint_dir, scene_name)
    dev = pc.t_position.device
    read = []

    def have(name):
        path = prefix + name
        if os.path.exists(path):
            read.append(name)
            return _read(path, dev)
        return None

    t = have(POINTS)
    if t:
        pc.t_position.data = t["t_position"].to(dev).contiguous()
        if "t_point_size" in t:
            pc.t_point_size.data = t["t_point_size"].to(dev).contiguous()
        pc.t_index = t["t_index"].to(dev).contiguous()
        pc.t_original_color = t["t_original_color"].to(dev).contiguous()
    t = have(TEXTURE)
    if t:
        tex.texture_raw.data = t["texture"].to(dev).contiguous()
        tex.background_color_raw.data = t["background_color"].to(dev).contiguous()
        tex.confidence_raw.data = t["confidence_value_of_point"].to(dev).contiguous()
        tex._prepared.clear()
    t = have(POSES)
    if t:
        scene.poses.tangent_poses.data = t["tangent_poses"].to(dev)
        scene.poses.poses_se3 = t["poses_se3"].to(dev).contiguous()
    t = have(INTRINSICS)
    if t:
        scene.intrinsics.intrinsics.data = t["intrinsics"].to(dev).contiguous()
    t = have(OPTIMIZER) if optimizers else None
    if t:
        by_name = {v: k for k, v in _state_names(scene).items()}
        for opt in optimizers:
            for group in opt.param_groups:
                for q in group["params"]:
                    name = next((n for n, i in by_name.items() if i == id(q)), None)
                    if name and f"{name}__first_moments" in t:
                        opt.state[q] = {k: t[f"{name}__{k}"].to(dev).contiguous() for k in ("first_moments", "second_moments", "param_steps")}
    return read
