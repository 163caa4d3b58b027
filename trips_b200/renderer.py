"""Host-side mirror of TRIPS's renderer operator interface on top of the C ABI.

Names, argument order and return values follow the reference so that a test or a training loop written against
src/lib/rendering/PointRenderer.h reads the same here:

  ReducedImageInfo      src/lib/data/SceneData.h:40-61
  RenderParams          src/lib/data/Settings.h:19-108 (the fields the live path reads)
  NeuralRenderInfo      src/lib/rendering/PointRenderer.h:23-34
  PointRendererCache    src/lib/rendering/PointRenderer.h:120-232 (owner of all scratch memory)
  PointRender           src/lib/rendering/PointRenderer.h:39-47, RenderInfo.cpp:44-80 (autograd boundary)
  BlendPointCloud       src/lib/rendering/RenderInfo.cpp:27-40
  BlendPointCloudForward / BlendPointCloudBackward   src/lib/rendering/PointRenderer.cu:676, 1232

PyTorch is used for device memory, streams and autograd only; every computation is done by libtrips_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from . import _lib
from .scenes import layer_sizes


@dataclass
class ReducedImageInfo:
    w: int = 0
    h: int = 0
    image_index: int = -1
    camera_index: int = -1
    camera_model_type: int = 0  # CameraModel::PINHOLE_DISTORTION
    crop_transform: Sequence[float] = (1.0, 1.0, 0.0, 0.0, 0.0)  # fx fy cx cy s
    crop_rotation: Sequence[float] = (1.0, 0.0, 0.0, 1.0)  # row-major 2x2


@dataclass
class RenderParams:
    num_texture_channels: int = 4
    use_layer_point_size: bool = True
    render_points_in_all_lower_resolutions: bool = True
    combine_lists: bool = False
    saturated_alpha_accumulation: bool = False
    check_normal: bool = False
    dropout: float = 0.0
    drop_out_points_by_radius: bool = False
    drop_out_radius_threshold: float = 0.6
    viewer_only: bool = False
    stability_cutoff_value: float = 10000.0
    normalize_grads: bool = False
    need_point_gradient: bool = True
    render_mode: int = 4  # TILED_BILINEAR_BLEND
    k_keep: int = 16  # PointRendererCache::max_pixels_per_list
    bg_uses_Tn: bool = False
    # texture preparation fused into the rasterizer (NeuralTexture.h:40-57): the tensors handed to PointRender are the raw
    # parameters, and the gradients are those of the raw parameters
    confidence_is_raw: bool = False
    confidence_scale: float = 10.0
    texture_abs: bool = False
    # lens distortion: apply the 8 coefficients of the intrinsics rows and the cut-off radius (RenderParams::dist_cutoff)
    distortion: bool = False
    dist_cutoff: float = 20.0


@dataclass
class NeuralRenderInfo:
    scene: object = None
    images: List[ReducedImageInfo] = field(default_factory=list)
    params: RenderParams = field(default_factory=RenderParams)
    num_layers: int = 1
    train: bool = False
    current_epoch: int = 0
    timer_system: object = None
    cache: "PointRendererCache" = None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class PointRendererCache:
    """Owns the library context (all scratch buffers and the records saved for backward)."""

    def __init__(self, device: Optional[torch.device] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("trips_b200 needs a CUDA device: there is no CPU fallback")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = C.c_void_p()
        _lib.check(_lib.lib().trips_context_create(C.byref(h), self.device.index or 0))
        self._h = h
        self._dropout = None
        self._keepalive = None
        # [views, points] float32, 1 = the point is dropped in that view.  None: the mask is drawn per forward pass with
        # probability RenderParams.dropout, as the reference does; set it to render with a mask of the caller's choosing.
        self.dropout_points = None

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().trips_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers ------------------------------------------------------------------------------------------------
    @staticmethod
    def _check_live_path(p: RenderParams):
        # normalize_grads is accepted and changes nothing, exactly as in the reference: NormalizeGradient divides by hit
        # counts (PointRenderer.cu:1193-1230, call sites :1348-1412) that are allocated as zeros (:226-272) and that no
        # kernel of the reference ever increments, so its `if (c > 0)` guard never passes.
        # use_layer_point_size, render_points_in_all_lower_resolutions and combine_lists select the reference's second forward
        # pipeline when they differ from their defaults (PointRenderer.cu:730-731); the library follows its rules then.
        # Normals are not part of the point cloud handed to the tiled renderer (GetPointWoNormal, RenderForward.cu:260).
        if p.check_normal:
            raise _lib.TripsError(_lib.ERR_UNSUPPORTED, "check_normal")

    def _scene_struct(self, texture, background_color, points, intrinsics, confidence, point_size, index, poses, dropout):
        n = points.shape[0]
        c, n_tex = texture.shape
        for t, dt in ((texture, torch.float32), (background_color, torch.float32), (points, torch.float32),
                      (intrinsics, torch.float32), (confidence, torch.float32), (point_size, torch.float32),
                      (poses, torch.float64)):
            if t.dtype != dt or not t.is_cuda or not t.is_contiguous():
                raise ValueError("scene tensors must be contiguous CUDA tensors of the reference dtypes")
        if points.shape[1] != 4 or intrinsics.shape[1] != 13 or poses.shape[1] != 8:
            raise ValueError("expected t_position [N,4], intrinsics [n,13], poses_se3 [n,8]")
        if index is not None and (index.dtype != torch.int32 or not index.is_contiguous()):
            raise ValueError("t_index must be contiguous int32")
        return _lib.TripsScene(n, n_tex, c, _ptr(points), _ptr(point_size), _ptr(index), _ptr(texture), _ptr(confidence),
                               _ptr(background_color), _ptr(dropout), _ptr(poses), poses.shape[0], _ptr(intrinsics),
                               intrinsics.shape[0])

    @staticmethod
    def _views(images: Sequence[ReducedImageInfo]):
        arr = (_lib.TripsView * len(images))()
        for i, im in enumerate(images):
            arr[i].w, arr[i].h = im.w, im.h
            arr[i].image_index, arr[i].camera_index = im.image_index, im.camera_index
            arr[i].camera_model_type = im.camera_model_type
            arr[i].crop_transform[:] = [float(x) for x in im.crop_transform]
            arr[i].crop_rotation[:] = [float(x) for x in im.crop_rotation]
        return arr

    @staticmethod
    def _params(info: NeuralRenderInfo):
        p = info.params
        return _lib.TripsRenderParams(info.num_layers, p.k_keep, int(info.train), int(p.drop_out_points_by_radius),
                                      p.drop_out_radius_threshold, int(p.viewer_only), p.stability_cutoff_value,
                                      int(p.bg_uses_Tn), int(p.confidence_is_raw), float(p.confidence_scale), int(p.texture_abs),
                                      int(p.use_layer_point_size), int(p.render_points_in_all_lower_resolutions), int(p.combine_lists),
                                      int(p.saturated_alpha_accumulation), int(p.distortion), float(p.dist_cutoff))

    # -- forward / backward -----------------------------------------------------------------------------------------
    def forward(self, info: NeuralRenderInfo, texture, background_color, points, intrinsics, confidence, point_size,
                index, poses) -> List[torch.Tensor]:
        self._check_live_path(info.params)
        B = len(info.images)
        w, h = info.images[0].w, info.images[0].h
        c = texture.shape[0]
        n = points.shape[0]
        dropout = None
        if info.train and self.dropout_points is not None:
            # a mask handed in by the caller (the reference keeps the mask in PointRendererCache::dropout_points)
            dropout = self.dropout_points
            if dropout.shape != (B, n) or dropout.dtype != torch.float32 or not dropout.is_cuda or not dropout.is_contiguous():
                raise ValueError("dropout_points must be a contiguous float32 CUDA tensor [views, points]")
        elif info.train and info.params.dropout > 0:
            # PointRendererCache::InitializeData, PointRenderer.cu:518-523
            dropout = torch.empty((B, n), device=points.device, dtype=torch.float32).bernoulli_(info.params.dropout)
        self._dropout = dropout
        sc = self._scene_struct(texture, background_color, points, intrinsics, confidence.reshape(-1), point_size.reshape(-1),
                                None if index is None else index.reshape(-1), poses, dropout)
        outs = [torch.empty((B, c, lh, lw), device=points.device, dtype=torch.float32)
                for (lw, lh) in layer_sizes(w, h, info.num_layers)]
        out_ptrs = (C.c_void_p * info.num_layers)(*[o.data_ptr() for o in outs])
        views = self._views(info.images)
        params = self._params(info)
        _lib.check(_lib.lib().trips_forward(self._h, C.byref(sc), views, B, C.byref(params), out_ptrs,
                                            _stream_ptr(points.device)), self._h)
        return outs

    def backward(self, grad_layers: Sequence[torch.Tensor], texture, background_color, points, intrinsics, confidence,
                 point_size, index, poses, want_pose=False, want_intrinsics=False, want_points=True, want_size=True,
                 out: Optional[dict] = None):
        """`out` may hold preallocated gradient tensors (keys texture, background, points, confidence, point_size),
        e.g. views into one flat buffer that is then all-reduced in a single call."""
        dev = points.device
        out = out or {}
        sc = self._scene_struct(texture, background_color, points, intrinsics, confidence.reshape(-1), point_size.reshape(-1),
                                None if index is None else index.reshape(-1), poses, self._dropout)
        grads_in = [g.contiguous() for g in grad_layers]
        for g in grads_in:
            if g.dtype != torch.float32:
                raise ValueError("image gradients must be float32")  # PointRenderer.cu:1236-1239
        gp = (C.c_void_p * len(grads_in))(*[g.data_ptr() for g in grads_in])
        g_tex = out.get("texture") if out.get("texture") is not None else torch.empty_like(texture)
        g_bg = out.get("background") if out.get("background") is not None else torch.empty_like(background_color)
        g_conf = out.get("confidence") if out.get("confidence") is not None else torch.empty_like(confidence)
        g_points = (out.get("points") if out.get("points") is not None else torch.empty_like(points)) if want_points else None
        g_size = (out.get("point_size") if out.get("point_size") is not None else torch.empty_like(point_size)) if want_size else None
        g_pose = torch.empty((poses.shape[0], 6), device=dev, dtype=torch.float64) if want_pose else None
        g_intr = torch.empty_like(intrinsics) if want_intrinsics else None
        gs = _lib.TripsGrads(_ptr(g_tex), _ptr(g_bg), _ptr(g_points), _ptr(g_pose), _ptr(g_intr), _ptr(g_conf), _ptr(g_size))
        _lib.check(_lib.lib().trips_backward(self._h, C.byref(sc), gp, C.byref(gs), _stream_ptr(dev)), self._h)
        return g_tex, g_bg, g_points, g_pose, g_intr, g_conf, g_size

    # -- stage timers (the reference's timer_system scopes) and the L1 benchmark loss ------------------------------------
    def enable_stage_timers(self, on: bool = True):
        _lib.check(_lib.lib().trips_enable_stage_timers(self._h, int(on)), self._h)

    def stage_times(self, reset: bool = True) -> dict:
        """{stage name: (accumulated ms, timed spans, kernels launched)} since the last reset."""
        n = _lib.NUM_STAGES
        ms = (C.c_double * n)()
        calls = (C.c_int64 * n)()
        launches = (C.c_int64 * n)()
        _lib.check(_lib.lib().trips_get_stage_times(self._h, ms, calls, launches, int(reset)), self._h)
        return {_lib.lib().trips_stage_name(i).decode(): (ms[i], calls[i], launches[i]) for i in range(n)}

    def l1_loss_backward(self, outs: Sequence[torch.Tensor], targets: Sequence[torch.Tensor], grads: Sequence[torch.Tensor],
                         loss_out: torch.Tensor):
        """grads[l] = sign(outs[l] - targets[l]) / total numel, loss_out (float64 scalar on the device) = mean |diff|."""
        n = len(outs)
        assert loss_out.dtype == torch.float64 and loss_out.is_cuda
        op = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
        tp = (C.c_void_p * n)(*[t.data_ptr() for t in targets])
        gp = (C.c_void_p * n)(*[t.data_ptr() for t in grads])
        numel = (C.c_int64 * n)(*[t.numel() for t in outs])
        _lib.check(_lib.lib().trips_l1_loss_backward(self._h, op, tp, gp, numel, n, _ptr(loss_out), _stream_ptr(outs[0].device)),
                   self._h)

    # -- inspection -----------------------------------------------------------------------------------------------
    def stats(self) -> dict:
        s = _lib.TripsStats()
        _lib.check(_lib.lib().trips_get_stats(self._h, C.byref(s), None), self._h)
        return {k: getattr(s, k) for k, _ in s._fields_}

    def last_status(self) -> int:
        return int(_lib.lib().trips_last_status(self._h, _stream_ptr(self.device)))

    def debug_points(self, view: int, n_points: int):
        import numpy as np
        depth = np.empty(n_points, np.float32)
        nl = np.empty(n_points, np.int32)
        rec = np.empty((n_points, 4), np.float32)
        _lib.check(_lib.lib().trips_debug_points(self._h, view, depth.ctypes.data, nl.ctypes.data, rec.ctypes.data,
                                                 _stream_ptr(self.device)), self._h)
        return depth, nl, rec

    def debug_lists(self, view: int, n_pixels: int):
        import numpy as np
        counts = np.empty(n_pixels, np.int32)
        offsets = np.empty(n_pixels, np.int64)
        nf = C.c_int64()
        st = _stream_ptr(self.device)
        _lib.check(_lib.lib().trips_debug_lists(self._h, view, counts.ctypes.data, offsets.ctypes.data, None, C.byref(nf), st), self._h)
        frags = np.empty(nf.value, np.uint64)
        _lib.check(_lib.lib().trips_debug_lists(self._h, view, None, None, frags.ctypes.data, C.byref(nf), st), self._h)
        return counts, offsets, frags

    def debug_records(self, view: int, n_pixels: int):
        import numpy as np
        nrec = np.empty(n_pixels, np.int32)
        pid = np.empty((n_pixels, 16), np.int32)
        alpha = np.empty((n_pixels, 16), np.float32)
        _lib.check(_lib.lib().trips_debug_records(self._h, view, nrec.ctypes.data, pid.ctypes.data, alpha.ctypes.data,
                                                  _stream_ptr(self.device)), self._h)
        return nrec, pid, alpha


def BlendPointCloudForward(ctx, info: NeuralRenderInfo):
    """Returns (color layers, mask layers); masks are not produced (output_background_mask is off by default)."""
    scene = info.scene
    if info.cache is None:
        raise ValueError("NeuralRenderInfo.cache must be set")  # SAIGA_ASSERT(info->cache)
    outs = info.cache.forward(info, scene.texture.texture, scene.texture.background_color, scene.point_cloud_cuda.t_position,
                              scene.intrinsics.intrinsics, scene.texture.confidence_value_of_point,
                              scene.point_cloud_cuda.t_point_size, scene.point_cloud_cuda.t_index, scene.poses.poses_se3)
    return outs, []


def BlendPointCloudBackward(ctx, info: NeuralRenderInfo, image_gradients):
    """Returns the 8 gradients in the order of PointRenderer.cu:1423-1426."""
    scene = info.scene
    grads = list(image_gradients)[: info.num_layers]
    pc = scene.point_cloud_cuda
    g_tex, g_bg, g_points, g_pose, g_intr, g_conf, g_size = info.cache.backward(
        grads, scene.texture.texture, scene.texture.background_color, pc.t_position, scene.intrinsics.intrinsics,
        scene.texture.confidence_value_of_point, pc.t_point_size, pc.t_index, scene.poses.poses_se3,
        want_pose=scene.poses.tangent_poses.requires_grad, want_intrinsics=scene.intrinsics.intrinsics.requires_grad,
        want_points=pc.t_position.requires_grad, want_size=pc.t_point_size.requires_grad)
    return [g_tex, g_bg, g_points, g_pose, g_intr, g_conf, None, g_size]


class PointRender(torch.autograd.Function):
    """torch::autograd::PointRender: one output tensor per pyramid layer."""

    @staticmethod
    def forward(ctx, texture, background_color, points, pose_tangents, intrinsics, confidence, dynamic_refinement,
                layer_value_of_point, info):
        ctx.render_info = info
        color, mask = BlendPointCloudForward(ctx, info)
        return tuple(color + mask)

    @staticmethod
    def backward(ctx, *grad_output):
        info = ctx.render_info
        derives = BlendPointCloudBackward(ctx, info, grad_output)
        assert len(derives) == 8
        # the trailing None is for the `info` argument, RenderInfo.cpp:76-77
        return tuple(derives) + (None,)


def BlendPointCloud(info: NeuralRenderInfo):
    """Render the scene into a batch of image pyramids (one tensor [B,C,H_l,W_l] per layer)."""
    s = info.scene
    assert s is not None and s.texture is not None
    return list(PointRender.apply(s.texture.texture, s.texture.background_color, s.point_cloud_cuda.t_position,
                                  s.poses.tangent_poses, s.intrinsics.intrinsics, s.texture.confidence_value_of_point,
                                  s.dynamic_refinement_t, s.point_cloud_cuda.t_point_size, info))
