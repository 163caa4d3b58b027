"""Parameter stores and the render module, mirroring the reference's torch modules (names, shapes, dtypes).

  NeuralPointCloudCuda   src/lib/rendering/NeuralPointCloudCuda.{h,cpp}  t_position [N,4], t_point_size [N,1],
                         t_index [N,1] int32, t_original_color [N,4]
  NeuralPointTexture     src/lib/models/NeuralTexture.{h,cpp}  texture_raw [C,N], confidence_raw [1,N],
                         background_color_raw [C]; PrepareTexture / PrepareConfidence
  PoseModule             src/lib/data/NeuralStructure.cpp:11-36   poses_se3 [n,8] f64, tangent_poses [n,6] f64
  IntrinsicsModule       src/lib/data/NeuralStructure.cpp:81-142  intrinsics [n,13] f32
  PointRenderModule      src/lib/rendering/RenderModule.{h,cpp}
The registered tensor names are the reference's checkpoint format (NeuralPointCloudCuda.cpp:103-108, NeuralTexture.cpp:53-55).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch
from torch import nn

from .renderer import BlendPointCloud, NeuralRenderInfo, PointRendererCache, ReducedImageInfo, RenderParams
from .scenes import Scene, inverse_softplus


class NeuralPointCloudCuda(nn.Module):
    def __init__(self, position: torch.Tensor, size_world: Optional[torch.Tensor] = None, point_size_raw: Optional[torch.Tensor] = None,
                 index: Optional[torch.Tensor] = None, original_color: Optional[torch.Tensor] = None, use_pointsize: bool = True):
        super().__init__()
        n = position.shape[0]
        assert position.shape == (n, 4) and position.dtype == torch.float32
        if point_size_raw is None:
            # data_point_size.push_back(inverse_softplus(data[i](0) * 0.5f)), NeuralPointCloudCuda.cpp:50
            sw = size_world.detach().cpu().numpy().astype(np.float64) * 0.5
            point_size_raw = torch.from_numpy(inverse_softplus(sw)).to(position.device)
        self.t_position = nn.Parameter(position.contiguous())
        ps = point_size_raw.reshape(n, 1).contiguous().float()
        if use_pointsize:
            self.t_point_size = nn.Parameter(ps)
        else:
            self.register_buffer("t_point_size", ps)
        if index is None:
            index = torch.arange(n, dtype=torch.int32, device=position.device)
        self.register_buffer("t_index", index.reshape(n, 1).to(torch.int32).contiguous())
        if original_color is None:
            original_color = torch.ones((n, 4), dtype=torch.float32, device=position.device)
        self.register_buffer("t_original_color", original_color.contiguous())

    def Size(self) -> int:
        return self.t_position.shape[0]

    def Indices(self):
        return self.t_index.reshape(-1).cpu().tolist()

    def RemoveSelected(self, to_keep: torch.Tensor):
        """Keep the listed points (NeuralPointCloudCuda.h:51-69)."""
        with torch.no_grad():
            self.t_position = nn.Parameter(self.t_position.data[to_keep].contiguous())
            new_ps = self.t_point_size.data[to_keep].contiguous()
            if isinstance(self.t_point_size, nn.Parameter):
                self.t_point_size = nn.Parameter(new_ps)
            else:
                self.t_point_size = new_ps
            self.t_original_color = self.t_original_color[to_keep].contiguous()
            self.t_index = self.t_index[to_keep].contiguous()


class NeuralPointTexture(nn.Module):
    def __init__(self, num_channels: int, num_points: int, random_init: bool = False, texture: Optional[torch.Tensor] = None,
                 confidence_raw: Optional[torch.Tensor] = None, device="cuda", use_abs: bool = False):
        super().__init__()
        if texture is None:
            texture = torch.rand((num_channels, num_points), device=device) if random_init else torch.ones((num_channels, num_points), device=device)
        if confidence_raw is None:
            confidence_raw = torch.ones((1, num_points), device=device)
        self.texture_raw = nn.Parameter(texture.contiguous().float())
        self.confidence_raw = nn.Parameter(confidence_raw.reshape(1, -1).contiguous().float())
        self.background_color_raw = nn.Parameter(torch.full((num_channels,), 0.25, device=device))  # NeuralTexture.cpp:18,37
        self.use_abs = use_abs
        # tensors the renderer reads (texture, confidence_value_of_point, background_color); the Prepare* calls
        # replace them with activated versions.  Kept outside nn.Module's parameter registry.
        self._prepared = {}

    @property
    def texture(self):
        return self._prepared.get("texture", self.texture_raw)

    @property
    def confidence_value_of_point(self):
        return self._prepared.get("confidence", self.confidence_raw)

    @property
    def background_color(self):
        return self._prepared.get("background", self.background_color_raw)

    def state_dict(self, *a, **k):
        sd = super().state_dict(*a, **k)
        # checkpoint names of the reference (NeuralTexture.cpp:53-55)
        ren = {"texture_raw": "texture", "confidence_raw": "confidence_value_of_point", "background_color_raw": "background_color"}
        return {ren.get(k2, k2): v for k2, v in sd.items()}

    def PrepareConfidence(self, narrowing_fac: float = 0.0):
        # confidence_value_of_point = sigmoid((10 + narrowing) * raw), NeuralTexture.h:40-43
        self._prepared["confidence"] = torch.sigmoid((10.0 + narrowing_fac) * self.confidence_raw)

    def PrepareTexture(self, abs_: Optional[bool] = None):
        use_abs = self.use_abs if abs_ is None else abs_
        if use_abs:
            self._prepared["texture"] = torch.abs(self.texture_raw)  # NeuralTexture.h:45-57
        else:
            self._prepared.pop("texture", None)

    def NumPoints(self) -> int:
        return self.texture_raw.shape[1]

    def TextureChannels(self) -> int:
        return self.texture_raw.shape[0]


class PoseModule(nn.Module):
    def __init__(self, poses_se3: torch.Tensor):
        super().__init__()
        assert poses_se3.dtype == torch.float64 and poses_se3.shape[1] == 8
        self.register_buffer("poses_se3", poses_se3.contiguous())
        self.tangent_poses = nn.Parameter(torch.zeros((poses_se3.shape[0], 6), dtype=torch.float64, device=poses_se3.device))
        self.tangent_poses.requires_grad_(False)


class IntrinsicsModule(nn.Module):
    def __init__(self, intrinsics: torch.Tensor):
        super().__init__()
        assert intrinsics.dtype == torch.float32 and intrinsics.shape[1] == 13
        self.intrinsics = nn.Parameter(intrinsics.contiguous())
        self.intrinsics.requires_grad_(False)


class NeuralScene(nn.Module):
    """The slice of src/lib/data/NeuralScene.h the renderer reads: the four modules above."""

    def __init__(self, point_cloud_cuda: NeuralPointCloudCuda, texture: NeuralPointTexture, poses: PoseModule,
                 intrinsics: IntrinsicsModule):
        super().__init__()
        self.point_cloud_cuda = point_cloud_cuda
        self.texture = texture
        self.poses = poses
        self.intrinsics = intrinsics
        self.dynamic_refinement_t = torch.zeros(1, device=point_cloud_cuda.t_position.device)  # dummy, NeuralScene.cpp
        self.scene_name = "scene"  # SceneData::scene_name: part of the checkpoint file names (NeuralScene.cpp:535,597)

    @classmethod
    def from_synthetic(cls, s: Scene, device="cuda", confidence_is_activated: bool = True) -> "NeuralScene":
        """Upload a synthetic scene.  Its confidence is already activated: it is stored as the raw parameter and
        PrepareConfidence is not applied unless the caller does so."""
        dev = torch.device(device)
        pc = NeuralPointCloudCuda(torch.from_numpy(s.position).to(dev), point_size_raw=torch.from_numpy(s.point_size).to(dev))
        tex = NeuralPointTexture(s.channels, s.n_points, texture=torch.from_numpy(s.texture).to(dev),
                                 confidence_raw=torch.from_numpy(s.confidence).to(dev), device=dev)
        with torch.no_grad():
            tex.background_color_raw.copy_(torch.from_numpy(s.background).to(dev))
        poses = PoseModule(torch.from_numpy(s.poses).to(dev))
        intr = IntrinsicsModule(torch.from_numpy(s.intrinsics).to(dev))
        ns = cls(pc, tex, poses, intr)
        ns.scene_name = s.name
        return ns

    # -- point removal / growth on the device (NeuralScene::RemovePoints / AddNewPoints, NeuralScene.cpp:1224-1431) ----
    def _point_tensors(self, optimizers=()):
        """(holder, attribute or state key, tensor, rows, point_major, fill value) of every per-point tensor."""
        pc, tex = self.point_cloud_cuda, self.texture
        out = [(pc.t_position, None, pc.t_position.data, 4, True, 0.0), (pc.t_point_size, None, pc.t_point_size.data, 1, True, 0.0),
               (pc, "t_original_color", pc.t_original_color, 4, True, 1.0),
               (tex.texture_raw, None, tex.texture_raw.data, tex.texture_raw.shape[0], False, 0.5),  # NeuralTexture.cpp:160
               (tex.confidence_raw, None, tex.confidence_raw.data, 1, False, 0.5)]
        params = {id(pc.t_position): (4, True), id(pc.t_point_size): (1, True), id(tex.texture_raw): (tex.texture_raw.shape[0], False),
                  id(tex.confidence_raw): (1, False)}
        for opt in optimizers:
            for group in opt.param_groups:
                for p in group["params"]:
                    st = opt.state.get(p)
                    if st and id(p) in params:
                        rows, pm = params[id(p)]
                        for k in ("first_moments", "second_moments", "param_steps"):
                            out.append((st, k, st[k], rows, pm, 0.0))  # MyAdam.cu:346-415: kept entries, zeros for new ones
        return out

    @torch.no_grad()
    def ResizePoints(self, cache, indices_to_remove: Optional[torch.Tensor] = None, new_size: Optional[int] = None, optimizers=()):
        """Removes the listed points (distinct indices, any order) and / or grows the scene to `new_size` points in one
        device pass over all per-point parameters and the Adam state of `optimizers` (trips_resize_points).  New points
        get 0.5 in texture and confidence, zeros elsewhere; the caller writes their positions and sizes afterwards.
        Returns the number of kept points."""
        import ctypes as C

        import numpy as np

        from . import _lib
        pc = self.point_cloud_cuda
        n_old = pc.t_position.shape[0]
        n_remove = 0 if indices_to_remove is None else int(indices_to_remove.numel())
        n_keep = n_old - n_remove
        n_new = n_keep if new_size is None else int(new_size)
        rem = None
        if n_remove:
            rem = indices_to_remove.reshape(-1).to(device=pc.t_position.device, dtype=torch.int64).contiguous()
        items = self._point_tensors(optimizers)
        table, new_tensors = [], []
        for holder, key, t, rows, pm, fill in items:
            assert t.is_contiguous() and t.element_size() in (4, 8)
            shape = (n_new, rows) if pm else (rows, n_new)
            nt = torch.empty(shape, dtype=t.dtype, device=t.device)
            bits = int(np.float32(fill).view(np.uint32)) if t.dtype.is_floating_point else int(fill)
            table.append(_lib.TripsPointTensor(t.data_ptr(), nt.data_ptr(), rows, t.element_size(), int(pm), bits))
            new_tensors.append(nt)
        arr = (_lib.TripsPointTensor * len(table))(*table)
        stream = C.c_void_p(torch.cuda.current_stream(pc.t_position.device).cuda_stream)
        _lib.check(_lib.lib().trips_resize_points(cache._h, None if rem is None else rem.data_ptr(), n_remove, n_old, n_new, arr, len(table),
                                                  stream), cache._h)
        for (holder, key, t, rows, pm, fill), nt in zip(items, new_tensors):
            nt = nt.view((n_new,) + tuple(t.shape[1:])) if pm else nt
            if key is None:
                holder.data = nt  # same Parameter object: optimizer state stays keyed to it
            elif isinstance(holder, dict):
                holder[key] = nt
            else:
                setattr(holder, key, nt)
        if pc.t_index is not None:
            pc.t_index = torch.arange(n_new, dtype=torch.int32, device=pc.t_position.device).reshape(n_new, 1)  # points and texture columns stay aligned
        for p in (pc.t_position, pc.t_point_size, self.texture.texture_raw, self.texture.confidence_raw):
            p.grad = None  # the reference resets the gradients to zeros of the new shape (NeuralScene.cpp:1440-1466)
        self.texture._prepared.clear()
        return n_keep


def images_for(s: Scene, views=None) -> List[ReducedImageInfo]:
    views = range(s.n_views) if views is None else views
    return [ReducedImageInfo(w=s.width, h=s.height, image_index=int(v), camera_index=int(v)) for v in views]


class PointRenderModule(nn.Module):
    """PointRenderModuleImpl (RenderModule.h:10-27): owns one PointRendererCache reused across calls."""

    def __init__(self, params: Optional[RenderParams] = None, num_layers: int = 1):
        super().__init__()
        self.params = params or RenderParams()
        self.num_layers = num_layers
        self.cache: Optional[PointRendererCache] = None

    def forward(self, scene: NeuralScene, images: List[ReducedImageInfo], current_epoch: int = 0, timer_system=None):
        if self.cache is None:
            self.cache = PointRendererCache(scene.point_cloud_cuda.t_position.device)
        nri = NeuralRenderInfo(scene=scene, images=images, params=self.params, num_layers=self.num_layers,
                               train=self.training, current_epoch=current_epoch, timer_system=timer_system, cache=self.cache)
        return self.forward_info(nri)

    def forward_info(self, nri: NeuralRenderInfo):
        if nri.cache is None:
            if self.cache is None:
                self.cache = PointRendererCache(nri.scene.point_cloud_cuda.t_position.device)
            nri.cache = self.cache
        return BlendPointCloud(nri), []
