"""CPU-only checks of the boundary and the host logic: the library loads and exports every symbol the header
declares, argument errors are status codes, and the host-side mirrors behave like the reference classes."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "trips_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trips_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(cuda_lib):
    from trips_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(cuda_lib, n), f"{n} is declared in include/trips_b200.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype in trips_b200/_lib.py"
    assert sorted(_lib.SYMBOLS) == names


def test_status_strings_and_argument_errors_without_a_gpu(cuda_lib):
    from trips_b200 import _lib
    assert cuda_lib.trips_status_string(0) == b"ok"
    assert b"unsupported" in cuda_lib.trips_status_string(_lib.ERR_UNSUPPORTED)
    assert cuda_lib.trips_context_create(None, 0) == _lib.ERR_INVALID_ARG
    assert cuda_lib.trips_forward(None, None, None, 0, None, None, None) == _lib.ERR_INVALID_ARG
    assert cuda_lib.trips_adam_step_static(None, 0, None) == _lib.ERR_INVALID_ARG
    assert cuda_lib.trips_fused_reduce_adam_multicast(None, None, None, None, None, 0, 0, 0, None, None, None, None) == _lib.ERR_INVALID_ARG
    assert cuda_lib.trips_stage_name(1) == b"bin_points"
    import torch
    if not torch.cuda.is_available():
        h = C.c_void_p()
        assert cuda_lib.trips_context_create(C.byref(h), 0) == _lib.ERR_CUDA  # no device: an error code, not a crash
        assert not h.value


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from trips_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_renderer_needs_cuda_and_rejects_unsupported_flags():
    import torch
    from trips_b200 import TripsError
    from trips_b200.renderer import PointRendererCache, RenderParams
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            PointRendererCache()
    with pytest.raises(TripsError) as e:
        PointRendererCache._check_live_path(RenderParams(check_normal=True))
    assert e.value.status == -4
    # the flags of the reference's second forward pipeline are accepted
    for kw in (dict(), dict(use_layer_point_size=False), dict(render_points_in_all_lower_resolutions=False), dict(combine_lists=True),
               dict(saturated_alpha_accumulation=True)):
        PointRendererCache._check_live_path(RenderParams(**kw))


def test_layer_sizes_are_ceil_halved():
    from trips_b200.scenes import layer_sizes, num_pyramid_pixels
    assert layer_sizes(1920, 1080, 8) == [(1920, 1080), (960, 540), (480, 270), (240, 135), (120, 68), (60, 34), (30, 17), (15, 9)]
    assert num_pyramid_pixels(1920, 1080, 8) == 2764845
    assert num_pyramid_pixels(1280, 720, 6) == 1228520
    assert num_pyramid_pixels(640, 480, 4) == 408000


def test_synthetic_scenes_have_reference_layouts():
    from trips_b200 import scenes
    s = scenes.tiny(n_points=50, n_views=3)
    assert s.position.shape == (50, 4) and s.position.dtype == np.float32
    assert s.texture.shape == (4, 50) and s.confidence.shape == (50,)
    assert s.poses.shape == (3, 8) and s.poses.dtype == np.float64 and s.intrinsics.shape == (3, 13)
    assert np.allclose(np.linalg.norm(s.poses[:, :4], axis=1), 1)  # unit quaternions
    assert np.all(s.intrinsics[:, 5:] == 0)
    # raw sizes invert the softplus parametrisation (NeuralPointCloudCuda.cpp:19-24)
    assert np.allclose(np.log1p(np.exp(s.point_size.astype(np.float64))), s.position[:, 3], rtol=1e-5)
    a, b = scenes.tiny(n_points=50, seed=3), scenes.tiny(n_points=50, seed=3)
    assert np.array_equal(a.position, b.position) and np.array_equal(a.texture, b.texture)
    # a camera looks at its target: the target projects onto the optical axis
    pose = scenes.look_at_pose((1.0, 2.0, 3.0), (0.0, 0.0, 0.0))
    q, t = pose[:4], pose[4:7]
    x, y, z, w = q
    R = np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)],
                  [2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)],
                  [2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]])
    pv = R @ np.zeros(3) + t
    assert abs(pv[0]) < 1e-9 and abs(pv[1]) < 1e-9 and abs(pv[2] - np.sqrt(14)) < 1e-9


def test_parameter_modules_keep_reference_names():
    import torch
    from trips_b200.modules import NeuralPointCloudCuda, NeuralPointTexture
    tex = NeuralPointTexture(4, 10, device="cpu")
    assert sorted(tex.state_dict()) == ["background_color", "confidence_value_of_point", "texture"]  # NeuralTexture.cpp:53-55
    assert tex.texture is tex.texture_raw
    tex.PrepareConfidence()
    assert torch.allclose(tex.confidence_value_of_point, torch.sigmoid(10 * tex.confidence_raw))
    tex.PrepareTexture(abs_=True)
    assert torch.equal(tex.texture, tex.texture_raw.abs())
    pc = NeuralPointCloudCuda(torch.rand(10, 4), size_world=torch.full((10,), 0.2))
    assert sorted(pc.state_dict()) == ["t_index", "t_original_color", "t_point_size", "t_position"]  # NeuralPointCloudCuda.cpp:103-108
    assert pc.t_index.dtype == torch.int32 and pc.t_point_size.shape == (10, 1)
    # inverse_softplus(0.5 * size), NeuralPointCloudCuda.cpp:50
    assert torch.allclose(torch.nn.functional.softplus(pc.t_point_size), torch.full((10, 1), 0.1), atol=1e-6)
    pc.RemoveSelected(torch.tensor([0, 3, 4]))
    assert pc.Size() == 3 and pc.t_index.reshape(-1).tolist() == [0, 3, 4]


def test_my_adam_state_surgery_and_validation():
    import torch
    from trips_b200.optim import MyAdam, UpdateOptimLR
    with pytest.raises(ValueError):
        MyAdam([torch.nn.Parameter(torch.zeros(3))], lr=-1.0)
    with pytest.raises(ValueError):
        MyAdam([torch.nn.Parameter(torch.zeros(3))], betas=(1.0, 0.9))
    p = torch.nn.Parameter(torch.zeros(4, 6))
    opt = MyAdam([dict(params=[p], lr=1e-2)])
    opt.state[p] = dict(param_steps=torch.arange(24, dtype=torch.int32).reshape(4, 6), first_moments=torch.rand(4, 6),
                        second_moments=torch.rand(4, 6), current_step=3)
    m = opt.state[p]["first_moments"].clone()
    opt.shrinkInternalState(0, torch.tensor([[0], [2], [5]]))  # keeps columns of the last dimension, MyAdam.cu:346-373
    assert opt.state[p]["first_moments"].shape == (4, 3) and torch.equal(opt.state[p]["first_moments"], m[:, [0, 2, 5]])
    assert opt.state[p]["param_steps"][1].tolist() == [6, 8, 11]
    opt.appendToInternalState(0, 5)  # zero-extends to 5 columns, MyAdam.cu:376-415
    assert opt.state[p]["second_moments"].shape == (4, 5) and torch.all(opt.state[p]["second_moments"][:, 3:] == 0)
    UpdateOptimLR(opt, 0.5)
    assert opt.param_groups[0]["lr"] == 5e-3
    q = torch.nn.Parameter(torch.zeros(4, 5))
    opt.rebind(p, q)
    assert q in opt.state and p not in opt.state and opt.param_groups[0]["params"][0] is q


def test_bench_helpers():
    import bench
    assert bench.stage_bytes("collect", 10, 20, 4, 2, 100, 50) == 800
    assert bench.stage_bytes("adam", 1000, 0, 4, 1, 0, 0) == 36 * 1000 * 10
    peak, kind = bench.measured_peak()
    assert peak > 1000 and kind in ("measured", "fallback")
    cs = bench.ClockSampler(0)
    cs.proc = object()
    cs.lines = ["1965, 1965, 450.1, Not Active, Not Active, Not Active, Active", "1800, 1965, 900.0, Not Active, Not Active, Not Active, Not Active"]
    cs.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=0: None})()
    out = cs.stop()
    assert out["sm_mhz"] == 1882.5 and out["reasons"] == ["sw_power_cap"] and out["sm_max_mhz"] == 1965


def test_ctypes_structs_match_the_header_layout(tmp_path):
    """Every struct of include/trips_b200.h as the C compiler lays it out (size and the offset of every field) against
    the ctypes mirror in trips_b200/_lib.py: a field added on one side only would shift everything after it silently."""
    import ctypes as C
    import subprocess

    from trips_b200 import _lib
    structs = {"TripsScene": _lib.TripsScene, "TripsView": _lib.TripsView, "TripsRenderParams": _lib.TripsRenderParams,
               "TripsGrads": _lib.TripsGrads, "TripsStats": _lib.TripsStats, "TripsAdamTensor": _lib.TripsAdamTensor,
               "TripsAdamSegment": _lib.TripsAdamSegment, "TripsPointTensor": _lib.TripsPointTensor}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "trips_b200.h"', 'int main(void) {']
    for name, st in structs.items():
        lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in st._fields_:
            lines.append(f'  printf("{name}.{field} %zu\\n", offsetof({name}, {field}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = dict(l.split() for l in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for name, st in structs.items():
        assert int(out[name]) == C.sizeof(st), name
        for field, _ in st._fields_:
            assert int(out[f"{name}.{field}"]) == getattr(st, field).offset, f"{name}.{field}"
