"""ctypes view of the C ABI declared in include/trips_b200.h.

The library is loaded on first use.  If libtrips_b200.so is missing (not built) loading raises: there is no
CPU or PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TRIPS_B200_LIB selects another build of the same library (e.g. one compiled with different tuning macros)
LIB_PATH = os.environ.get("TRIPS_B200_LIB") or os.path.join(HERE, "libtrips_b200.so")

MAX_LAYERS = 8
MAX_KEEP = 16
NUM_STAGES = 12
MAX_RANKS = 16
MAX_SEGMENTS = 8
ADAM_STATIC_MAX_TENSORS = 64

OK = 0
ERR_INVALID_ARG = -1
ERR_CUDA = -2
ERR_OUT_OF_MEMORY = -3
ERR_UNSUPPORTED = -4
ERR_NO_FORWARD = -5
ERR_TOO_LARGE = -6

DEV_BAD_TEXTURE_INDEX = 1
DEV_NONZERO_DISTORTION = 2
DEV_FRAGMENT_OVERFLOW = 4
DEV_BAD_FRAGMENT = 8
DEV_BAD_POINT_INDEX = 16
DEV_ENTRY_OVERFLOW = 32


class TripsScene(C.Structure):
    _fields_ = [("n_points", C.c_int), ("n_tex", C.c_int), ("channels", C.c_int), ("position", C.c_void_p),
                ("point_size", C.c_void_p), ("index", C.c_void_p), ("texture", C.c_void_p), ("confidence", C.c_void_p),
                ("background", C.c_void_p), ("dropout", C.c_void_p), ("poses", C.c_void_p), ("n_images", C.c_int),
                ("intrinsics", C.c_void_p), ("n_cameras", C.c_int)]


class TripsView(C.Structure):
    _fields_ = [("w", C.c_int), ("h", C.c_int), ("image_index", C.c_int), ("camera_index", C.c_int),
                ("camera_model_type", C.c_int), ("crop_transform", C.c_float * 5), ("crop_rotation", C.c_float * 4)]


class TripsRenderParams(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("k_keep", C.c_int), ("train", C.c_int), ("drop_out_points_by_radius", C.c_int),
                ("drop_out_radius_threshold", C.c_float), ("viewer_only", C.c_int), ("stability_cutoff_value", C.c_float),
                ("bg_uses_Tn", C.c_int), ("confidence_is_raw", C.c_int), ("confidence_scale", C.c_float), ("texture_abs", C.c_int),
                ("use_layer_point_size", C.c_int), ("render_points_in_all_lower_resolutions", C.c_int), ("combine_lists", C.c_int),
                ("saturated_alpha_accumulation", C.c_int), ("distortion", C.c_int), ("dist_cutoff", C.c_float)]


class TripsGrads(C.Structure):
    _fields_ = [("texture", C.c_void_p), ("background", C.c_void_p), ("points", C.c_void_p), ("pose_tangent", C.c_void_p),
                ("intrinsics", C.c_void_p), ("confidence", C.c_void_p), ("point_size", C.c_void_p)]


class TripsStats(C.Structure):
    _fields_ = [("visible_points", C.c_int64), ("fragments", C.c_int64), ("kept_fragments", C.c_int64),
                ("pixels", C.c_int64), ("max_list_length", C.c_int64), ("culled_point_blocks", C.c_int64)]


class TripsAdamTensor(C.Structure):
    _fields_ = [("weights", C.c_void_p), ("gradients", C.c_void_p), ("first_moments", C.c_void_p),
                ("second_moments", C.c_void_p), ("steps", C.c_void_p), ("n", C.c_int64), ("lr", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float), ("relative_weight_decay", C.c_float),
                ("absolute_weight_decay", C.c_float), ("weight_clipping_magnitude", C.c_float),
                ("lower_lr_bound", C.c_float), ("upper_lr_bound", C.c_float)]


class TripsAdamSegment(C.Structure):
    _fields_ = [("offset", C.c_int64), ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("relative_weight_decay", C.c_float), ("absolute_weight_decay", C.c_float),
                ("weight_clipping_magnitude", C.c_float), ("lower_lr_bound", C.c_float), ("upper_lr_bound", C.c_float)]


class TripsPointTensor(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("rows", C.c_int), ("elem_bytes", C.c_int), ("point_major", C.c_int),
                ("fill_bits", C.c_uint32)]


# every symbol include/trips_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "trips_context_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "trips_context_destroy": (None, [C.c_void_p]),
    "trips_status_string": (C.c_char_p, [C.c_int]),
    "trips_last_error": (C.c_char_p, [C.c_void_p]),
    "trips_forward": (C.c_int, [C.c_void_p, C.POINTER(TripsScene), C.POINTER(TripsView), C.c_int,
                                C.POINTER(TripsRenderParams), C.POINTER(C.c_void_p), C.c_void_p]),
    "trips_backward": (C.c_int, [C.c_void_p, C.POINTER(TripsScene), C.POINTER(C.c_void_p), C.POINTER(TripsGrads), C.c_void_p]),
    "trips_last_status": (C.c_uint32, [C.c_void_p, C.c_void_p]),
    "trips_get_stats": (C.c_int, [C.c_void_p, C.POINTER(TripsStats), C.c_void_p]),
    "trips_adam_step": (C.c_int, [C.c_void_p, C.POINTER(TripsAdamTensor), C.c_int, C.c_void_p]),
    "trips_fused_reduce_adam": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                          C.POINTER(TripsAdamSegment), C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p]),
    "trips_fused_reduce_adam_multicast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(TripsAdamSegment), C.c_int,
                                                    C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "trips_resize_points": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.POINTER(TripsPointTensor), C.c_int, C.c_void_p]),
    "trips_adam_step_static": (C.c_int, [C.POINTER(TripsAdamTensor), C.c_int, C.c_void_p]),
    "trips_enable_stage_timers": (C.c_int, [C.c_void_p, C.c_int]),
    "trips_get_stage_times": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "trips_stage_name": (C.c_char_p, [C.c_int]),
    "trips_l1_loss_backward": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                         C.POINTER(C.c_int64), C.c_int, C.c_void_p, C.c_void_p]),
    "trips_debug_points": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "trips_debug_lists": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.c_void_p]),
    "trips_debug_records": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


class TripsError(RuntimeError):
    def __init__(self, status: int, detail: str = ""):
        self.status = status
        name = lib().trips_status_string(status).decode() if _lib is not None else str(status)
        super().__init__(f"trips_b200: {name} ({status}){': ' + detail if detail else ''}")


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m trips_b200.build` (there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, ctx=None):
    if status != OK:
        detail = lib().trips_last_error(ctx).decode() if ctx else ""
        raise TripsError(status, detail)
