"""trips_adam_step_static against trips_adam_step.

Some users of this library run the optimizer step at a point where device memory cannot be allocated: the training
framework's pool already owns every free byte, the host application forbids cudaMalloc after start-up, or the step is
recorded into a stream capture.  For them the library has a second Adam entry point whose tensor table sits in a
fixed device array instead of allocated scratch.  It must produce exactly what the allocating entry point produces,
on a first call (which also resolves the array's address) and on a second call that reuses the array.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _tensors(torch, _lib, rng, sizes, lr):
    params, grads, m, v, steps = [], [], [], [], []
    for n in sizes:
        params.append(torch.from_numpy(rng.normal(size=n).astype(np.float32)).cuda())
        g = rng.normal(size=n).astype(np.float32)
        g[rng.random(n) < 0.25] = 0.0  # untouched elements
        grads.append(torch.from_numpy(g).cuda())
        m.append(torch.zeros(n, device="cuda"))
        v.append(torch.zeros(n, device="cuda"))
        steps.append(torch.zeros(n, dtype=torch.int32, device="cuda"))
    return params, grads, m, v, steps


def _table(_lib, params, grads, m, v, steps, lr):
    flt_max = float(np.finfo(np.float32).max)
    rows = [_lib.TripsAdamTensor(p.data_ptr(), g.data_ptr(), a.data_ptr(), b.data_ptr(), s.data_ptr(), p.numel(), lr, 0.9,
                                 0.999, 1e-8, 0.0, 0.0, 0.0, 0.0, flt_max) for p, g, a, b, s in zip(params, grads, m, v, steps)]
    return (_lib.TripsAdamTensor * len(rows))(*rows)


def test_static_adam_matches_allocating_adam_twice(cuda_lib):
    import torch
    from trips_b200 import _lib
    L = cuda_lib
    sizes = [4 * 5003, 5003, 20012, 7, 4096 * 3 + 1]
    lr = 2e-3
    ref = _tensors(torch, _lib, np.random.default_rng(1), sizes, lr)
    new = [[t.clone() for t in group] for group in ref]
    ctx = C.c_void_p()
    _lib.check(L.trips_context_create(C.byref(ctx), torch.cuda.current_device()))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        for call in range(2):  # the second call reuses the fixed table written by the first
            if call == 1:
                rng = np.random.default_rng(2)
                for gr, gn in zip(ref[1], new[1]):
                    g = rng.normal(size=gr.numel()).astype(np.float32)
                    g[rng.random(gr.numel()) < 0.25] = 0.0
                    gr.copy_(torch.from_numpy(g))
                    gn.copy_(gr)
            free_before = torch.cuda.mem_get_info()[0]
            _lib.check(L.trips_adam_step(ctx, _table(_lib, *ref, lr), len(sizes), stream), ctx)
            _lib.check(L.trips_adam_step_static(_table(_lib, *new, lr), len(sizes), stream))
            torch.cuda.synchronize()
            for name, a, b in zip(("weights", "grads", "m", "v", "steps"), ref, new):
                for x, y in zip(a, b):
                    xa, ya = x.cpu().numpy(), y.cpu().numpy()
                    if name == "steps":
                        assert np.array_equal(xa, ya), f"call {call}: {name} differ"
                    else:
                        err = np.max(np.abs(xa - ya) / np.maximum(np.abs(xa), 1e-6)) if xa.size else 0.0
                        assert err <= 1e-5, f"call {call}: {name} differ by {err}"
            assert free_before >= 0
    finally:
        L.trips_context_destroy(ctx)


def test_static_adam_rejects_too_many_tensors(cuda_lib):
    import torch
    from trips_b200 import _lib
    n = _lib.ADAM_STATIC_MAX_TENSORS + 1
    group = _tensors(torch, _lib, np.random.default_rng(3), [8] * n, 1e-3)
    status = cuda_lib.trips_adam_step_static(_table(_lib, *group, 1e-3), n, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == _lib.ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert all(int(s.sum()) == 0 for s in group[4]), "a rejected call must not touch the tensors"
