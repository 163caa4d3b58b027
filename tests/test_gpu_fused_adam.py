"""trips_fused_reduce_adam (gradient sum over ranks + Adam + parameter broadcast in one kernel) against the plain
fused Adam applied to the summed gradient.  Ranks are emulated on one GPU: each "rank" has its own flat gradient and
parameter buffer, and the kernel is launched once per rank on its slice, exactly as the ranks of a node would do over
peer pointers.  Slices that do not start on a 16-byte boundary exercise the scalar edges."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,cuts", [(1, None), (2, None), (3, [0, 1001, 20007, None])])
def test_fused_reduce_adam_equals_sum_then_adam(cuda_lib, world, cuts):
    import torch
    from trips_b200 import _lib
    from trips_b200.dist import slice_bounds
    rng = np.random.default_rng(world)
    sizes = [4 * 5003, 5004, 20012, 5003, 4]  # texture, confidence, points, size, background of a 5003-point cloud
    lrs = [1e-3, 2e-3, 5e-4, 1e-3, 1e-2]
    numel = sum(-(-n // 4) * 4 for n in sizes)
    offs = np.cumsum([0] + [-(-n // 4) * 4 for n in sizes])[:-1]
    flt_max = float(np.finfo(np.float32).max)
    w0 = rng.normal(size=numel).astype(np.float32)
    ctx = C.c_void_p()
    _lib.check(cuda_lib.trips_context_create(C.byref(ctx), torch.cuda.current_device()))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    params = [torch.from_numpy(w0.copy()).cuda() for _ in range(world)]
    grads = [torch.zeros(numel, device="cuda") for _ in range(world)]
    ref_w = torch.from_numpy(w0.copy()).cuda()
    ref_m, ref_v = torch.zeros(numel, device="cuda"), torch.zeros(numel, device="cuda")
    ref_s = torch.zeros(numel, dtype=torch.int32, device="cuda")
    segs = (_lib.TripsAdamSegment * len(sizes))(*[_lib.TripsAdamSegment(int(o), lr, 0.9, 0.999, 1e-8, 0.0, 0.0, 0.0, 0.0, flt_max)
                                                   for o, lr in zip(offs, lrs)])
    if cuts is None:
        bounds = [slice_bounds(numel, world, r) for r in range(world)]
    else:
        edges = [c if c is not None else numel for c in cuts]
        bounds = [(edges[r], edges[r + 1]) for r in range(world)]
    state = [(torch.zeros(max(1, hi - lo), device="cuda"), torch.zeros(max(1, hi - lo), device="cuda"),
              torch.zeros(max(1, hi - lo), dtype=torch.int32, device="cuda")) for lo, hi in bounds]
    gp = (C.c_void_p * world)(*[g.data_ptr() for g in grads])
    pp = (C.c_void_p * world)(*[p.data_ptr() for p in params])
    try:
        for step in range(3):
            total = torch.zeros(numel, device="cuda")
            for r in range(world):
                g = rng.normal(size=numel).astype(np.float32)
                g[rng.random(numel) < 0.6] = 0.0  # most elements unseen by a rank; some unseen by all
                grads[r].copy_(torch.from_numpy(g))
            for r in range(world):
                total += grads[r]  # rank order, as in the kernel
            for r, (lo, hi) in enumerate(bounds):
                m, v, s = state[r]
                _lib.check(cuda_lib.trips_fused_reduce_adam(ctx, gp, pp, world, r, segs, len(sizes), lo, hi, m.data_ptr(),
                                                            v.data_ptr(), s.data_ptr(), stream), ctx)
            table = []
            for o, n, lr in zip(offs, sizes, lrs):
                o = int(o)
                table.append(_lib.TripsAdamTensor(ref_w[o:].data_ptr(), total[o:].data_ptr(), ref_m[o:].data_ptr(), ref_v[o:].data_ptr(),
                                                  ref_s[o:].data_ptr(), -(-n // 4) * 4, lr, 0.9, 0.999, 1e-8, 0.0, 0.0, 0.0, 0.0, flt_max))
            _lib.check(cuda_lib.trips_adam_step(ctx, (_lib.TripsAdamTensor * len(table))(*table), len(table), stream), ctx)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(params[r], ref_w), f"step {step}: replica {r} differs from sum-then-Adam"
            for r, (lo, hi) in enumerate(bounds):
                if hi > lo:
                    assert torch.equal(state[r][2][:hi - lo], ref_s[lo:hi])
                    assert torch.equal(state[r][0][:hi - lo], ref_m[lo:hi])
        unseen = (ref_s == 0)
        assert unseen.any() and torch.equal(ref_w[unseen], torch.from_numpy(w0).cuda()[unseen])
    finally:
        cuda_lib.trips_context_destroy(ctx)


def test_fused_reduce_adam_rejects_bad_arguments(cuda_lib):
    import torch
    from trips_b200 import _lib
    ctx = C.c_void_p()
    _lib.check(cuda_lib.trips_context_create(C.byref(ctx), torch.cuda.current_device()))
    t = torch.zeros(64, device="cuda")
    s = torch.zeros(64, dtype=torch.int32, device="cuda")
    gp = (C.c_void_p * 1)(t.data_ptr())
    seg = (_lib.TripsAdamSegment * 1)(_lib.TripsAdamSegment(0, 1e-3, 0.9, 0.999, 1e-8, 0, 0, 0, 0, 1e38))
    bad_seg = (_lib.TripsAdamSegment * 1)(_lib.TripsAdamSegment(4, 1e-3, 0.9, 0.999, 1e-8, 0, 0, 0, 0, 1e38))
    f = cuda_lib.trips_fused_reduce_adam
    try:
        assert f(ctx, gp, gp, 0, 0, seg, 1, 0, 64, t.data_ptr(), t.data_ptr(), s.data_ptr(), None) == _lib.ERR_INVALID_ARG
        assert f(ctx, gp, gp, 1, 1, seg, 1, 0, 64, t.data_ptr(), t.data_ptr(), s.data_ptr(), None) == _lib.ERR_INVALID_ARG
        assert f(ctx, gp, gp, 1, 0, bad_seg, 1, 0, 64, t.data_ptr(), t.data_ptr(), s.data_ptr(), None) == _lib.ERR_INVALID_ARG
        assert f(ctx, gp, gp, 1, 0, seg, 1, 8, 4, t.data_ptr(), t.data_ptr(), s.data_ptr(), None) == _lib.ERR_INVALID_ARG
        assert f(ctx, gp, gp, 1, 0, seg, 1, 0, 0, None, None, None, None) == _lib.OK  # empty slice: nothing to do
    finally:
        cuda_lib.trips_context_destroy(ctx)
