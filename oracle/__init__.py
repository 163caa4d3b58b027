"""ctypes binding of the CPU oracle (oracle/trips_oracle.cpp).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this package; the shipped
library (trips_b200) never does.  Parity unpinned: see the header of trips_oracle.h.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtrips_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (g++ -O3 -fopenmp -ffp-contract=off)."""
    if force and os.path.exists(_LIB_PATH):
        os.remove(_LIB_PATH)
    subprocess.run(["make", "-s", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


class OrScene(C.Structure):
    _fields_ = [("n_points", C.c_int), ("n_tex", C.c_int), ("channels", C.c_int), ("position", C.c_void_p),
                ("point_size", C.c_void_p), ("index", C.c_void_p), ("texture", C.c_void_p), ("confidence", C.c_void_p),
                ("background", C.c_void_p), ("dropout", C.c_void_p)]


class OrView(C.Structure):
    _fields_ = [("w", C.c_int), ("h", C.c_int), ("pose", C.c_double * 8), ("intrinsics", C.c_float * 13),
                ("crop_transform", C.c_float * 5), ("crop_rotation", C.c_float * 4)]


class OrParams(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("k_keep", C.c_int), ("train", C.c_int), ("drop_out_points_by_radius", C.c_int),
                ("drop_out_radius_threshold", C.c_float), ("viewer_only", C.c_int), ("stability_cutoff_value", C.c_float),
                ("bg_uses_Tn", C.c_int), ("use_layer_point_size", C.c_int), ("render_points_in_all_lower_resolutions", C.c_int),
                ("combine_lists", C.c_int), ("saturated_alpha_accumulation", C.c_int), ("distortion", C.c_int),
                ("dist_cutoff", C.c_float)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.or_forward.restype = C.c_void_p
        L.or_forward.argtypes = [C.POINTER(OrScene), C.POINTER(OrView), C.POINTER(OrParams)]
        L.or_frame_free.argtypes = [C.c_void_p]
        for name in ("or_num_pixels", "or_num_fragments", "or_num_kept", "or_num_visible"):
            getattr(L, name).restype = C.c_int64
            getattr(L, name).argtypes = [C.c_void_p]
        L.or_layer_size.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int64)]
        L.or_get_points.argtypes = [C.c_void_p] + [C.c_void_p] * 3
        L.or_get_lists.argtypes = [C.c_void_p] + [C.c_void_p] * 3
        L.or_get_first_layer.argtypes = [C.c_void_p, C.c_void_p]
        L.or_get_pyramid.argtypes = [C.c_void_p, C.c_void_p]
        L.or_get_records.argtypes = [C.c_void_p] + [C.c_void_p] * 3
        L.or_backward.argtypes = [C.c_void_p, C.POINTER(OrScene), C.POINTER(OrView), C.POINTER(OrParams)] + [C.c_void_p] * 8
        L.or_adam.argtypes = [C.c_int64] + [C.c_void_p] * 5 + [C.c_float] * 9
        L.or_layer_factor.restype = C.c_float
        L.or_layer_factor.argtypes = [C.c_float, C.c_int, C.c_int, C.POINTER(C.c_float)]
        for name in ("or_softplus", "or_expf", "or_logf"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.or_project.argtypes = [C.POINTER(OrView), C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.or_max_threads.restype = C.c_int
        L.or_set_threads.restype = None
        L.or_sigmoid.restype = None
        L.or_sigmoid.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_longlong]
        L.or_set_threads.argtypes = [C.c_int]
        L.or_layer_divergence.restype = None
        L.or_layer_divergence.argtypes = [C.c_void_p, C.POINTER(OrScene), C.POINTER(OrView), C.POINTER(OrParams), C.c_void_p]
        L.or_math_sweep.restype = None
        L.or_math_sweep.argtypes = [C.c_uint32, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def make_params(num_layers, k_keep, train, drop_out_points_by_radius=False, drop_out_radius_threshold=0.6,
                viewer_only=False, stability_cutoff_value=10000.0, bg_uses_Tn=False, use_layer_point_size=True,
                render_points_in_all_lower_resolutions=True, combine_lists=False, saturated_alpha_accumulation=False,
                distortion=False, dist_cutoff=20.0) -> OrParams:
    return OrParams(num_layers, k_keep, int(train), int(drop_out_points_by_radius), drop_out_radius_threshold,
                    int(viewer_only), stability_cutoff_value, int(bg_uses_Tn), int(use_layer_point_size),
                    int(render_points_in_all_lower_resolutions), int(combine_lists), int(saturated_alpha_accumulation),
                    int(distortion), float(dist_cutoff))


def make_view(w, h, pose8, intr13, crop_transform=(1, 1, 0, 0, 0), crop_rotation=(1, 0, 0, 1)) -> OrView:
    v = OrView()
    v.w, v.h = int(w), int(h)
    v.pose[:] = [float(x) for x in pose8]
    v.intrinsics[:] = [float(x) for x in intr13]
    v.crop_transform[:] = [float(x) for x in crop_transform]
    v.crop_rotation[:] = [float(x) for x in crop_rotation]
    return v


class SceneArrays:
    """Keeps contiguous numpy arrays alive for the lifetime of the OrScene struct."""

    def __init__(self, position, point_size, texture, confidence, background, index=None, dropout=None):
        self.position = np.ascontiguousarray(position, dtype=np.float32)
        self.point_size = np.ascontiguousarray(point_size, dtype=np.float32).reshape(-1)
        self.texture = np.ascontiguousarray(texture, dtype=np.float32)
        self.confidence = np.ascontiguousarray(confidence, dtype=np.float32).reshape(-1)
        self.background = np.ascontiguousarray(background, dtype=np.float32)
        self.index = None if index is None else np.ascontiguousarray(index, dtype=np.int32).reshape(-1)
        self.dropout = None if dropout is None else np.ascontiguousarray(dropout, dtype=np.float32)
        self.n = self.position.shape[0]
        self.channels, self.n_tex = self.texture.shape
        self.struct = OrScene(self.n, self.n_tex, self.channels, _ptr(self.position), _ptr(self.point_size),
                              _ptr(self.index), _ptr(self.texture), _ptr(self.confidence), _ptr(self.background),
                              _ptr(self.dropout))

    @classmethod
    def from_scene(cls, s, **kw):
        return cls(s.position, s.point_size, s.texture, s.confidence, s.background, **kw)


class Frame:
    """All intermediates of one view rendered by the oracle."""

    def __init__(self, handle, scene: SceneArrays, view: OrView, params: OrParams):
        self._h = handle
        self.scene, self.view, self.params = scene, view, params
        L = lib()
        self.P = L.or_num_pixels(handle)
        self.F = L.or_num_fragments(handle)
        self.Kf = L.or_num_kept(handle)
        self.V = L.or_num_visible(handle)
        self.layers = []
        for l in range(params.num_layers):
            w, h, b = C.c_int(), C.c_int(), C.c_int64()
            L.or_layer_size(handle, l, C.byref(w), C.byref(h), C.byref(b))
            self.layers.append((w.value, h.value, b.value))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().or_frame_free(self._h)
            self._h = None

    def points(self):
        n = self.scene.n
        depth = np.empty(n, np.float32)
        nl = np.empty(n, np.int32)
        rec = np.empty((n, 4), np.float32)
        lib().or_get_points(self._h, _ptr(depth), _ptr(nl), _ptr(rec))
        return depth, nl, rec

    def first_layer(self):
        first = np.empty(self.scene.n, np.int32)
        lib().or_get_first_layer(self._h, _ptr(first))
        return first

    def lists(self):
        counts = np.empty(self.P, np.int32)
        offsets = np.empty(self.P, np.int64)
        frags = np.empty(self.F, np.uint64)
        lib().or_get_lists(self._h, _ptr(counts), _ptr(offsets), _ptr(frags))
        return counts, offsets, frags

    def pyramid_flat(self):
        out = np.empty(self.scene.channels * self.P, np.float32)
        lib().or_get_pyramid(self._h, _ptr(out))
        return out

    def pyramid(self):
        flat = self.pyramid_flat()
        c = self.scene.channels
        return [flat[c * b:c * (b + w * h)].reshape(c, h, w) for (w, h, b) in self.layers]

    def records(self):
        nrec = np.empty(self.P, np.int32)
        pid = np.empty((self.P, 16), np.int32)
        alpha = np.empty((self.P, 16), np.float32)
        lib().or_get_records(self._h, _ptr(nrec), _ptr(pid), _ptr(alpha))
        return nrec, pid, alpha

    def backward(self, grad_flat, want_pose=True):
        s = self.scene
        g = np.ascontiguousarray(grad_flat, dtype=np.float32)
        assert g.size == s.channels * self.P
        out = dict(texture=np.zeros((s.channels, s.n_tex), np.float64), confidence=np.zeros(s.n_tex, np.float64),
                   position=np.zeros((s.n, 4), np.float64), point_size=np.zeros(s.n, np.float64),
                   background=np.zeros(s.channels, np.float64), pose=np.zeros(6, np.float64),
                   intrinsics=np.zeros(13, np.float64))
        lib().or_backward(self._h, C.byref(s.struct), C.byref(self.view), C.byref(self.params), _ptr(g),
                          _ptr(out["texture"]), _ptr(out["confidence"]), _ptr(out["position"]), _ptr(out["point_size"]),
                          _ptr(out["background"]), _ptr(out["pose"]), _ptr(out["intrinsics"]))
        return out


def layer_divergence(frame: "Frame") -> dict:
    """How many visible points of the frame would pick other pyramid layers with the host libm (see trips_oracle.h)."""
    out = np.zeros(6, np.int64)
    lib().or_layer_divergence(frame._h, C.byref(frame.scene.struct), C.byref(frame.view), C.byref(frame.params), _ptr(out))
    return dict(zip(("visible", "ps_gt_1", "ceil_log2_differs", "floor_log2_differs", "layers_differ_with_libm_softplus",
                     "softplus_bits_differ"), (int(x) for x in out)))


def math_sweep(stride: int = 64):
    """(max ulp error of the reproducible exp, of the reproducible log) against double-precision libm."""
    a, b = C.c_double(), C.c_double()
    lib().or_math_sweep(int(stride), C.byref(a), C.byref(b))
    return a.value, b.value


def forward(scene: SceneArrays, view: OrView, params: OrParams) -> Frame:
    h = lib().or_forward(C.byref(scene.struct), C.byref(view), C.byref(params))
    if not h:
        raise ValueError("oracle: invalid parameters")
    return Frame(h, scene, view, params)


def adam(w, g, m, v, steps, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, rel_decay=0.0, abs_decay=0.0, clip=0.0,
         lower_lr=0.0, upper_lr=float(np.finfo(np.float32).max)):
    """In-place reference Adam step over flat float32 arrays; `steps` is int64."""
    for a in (w, g, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    assert steps.dtype == np.int64
    lib().or_adam(w.size, _ptr(w), _ptr(g), _ptr(m), _ptr(v), _ptr(steps), lr, beta1, beta2, eps, rel_decay, abs_decay,
                  clip, lower_lr, upper_lr)


def sigmoid(raw: np.ndarray, scale: float) -> np.ndarray:
    """sigmoid(scale * raw) as PrepareConfidence computes it (NeuralTexture.h:40-43), float32."""
    raw = np.ascontiguousarray(raw, dtype=np.float32)
    out = np.empty_like(raw)
    lib().or_sigmoid(_ptr(raw), scale, _ptr(out), raw.size)
    return out


def max_threads() -> int:
    return lib().or_max_threads()


def use_all_cores() -> int:
    """Sets the OpenMP team size to the cores this process may run on (torchrun exports OMP_NUM_THREADS=1)."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().or_set_threads(n)
    return max_threads()


def resize_points(tensors, indices_to_remove, n_new):
    """CPU restatement of point removal / growth over per-point tensors (numpy; checker for trips_resize_points).

    tensors: list of (array, point_major, fill).  Kept points keep their order (index_select with the ascending list of
    kept indices: NeuralScene.cpp:1390-1405,1425-1431; NeuralTexture.cpp:195-208; MyAdam.cu:346-373); points beyond
    the kept ones are filled with the tensor's constant (NeuralTexture.cpp:153-193; MyAdam.cu:376-415)."""
    out = []
    for a, point_major, fill in tensors:
        n_old = a.shape[0] if point_major else a.shape[-1]
        keep = np.setdiff1d(np.arange(n_old), np.asarray(indices_to_remove, dtype=np.int64))
        kept = np.take(a, keep, axis=0 if point_major else a.ndim - 1)
        pad_shape = list(kept.shape)
        pad_shape[0 if point_major else -1] = n_new - keep.size
        out.append(np.concatenate([kept, np.full(pad_shape, fill, dtype=a.dtype)], axis=0 if point_major else a.ndim - 1))
    return out
