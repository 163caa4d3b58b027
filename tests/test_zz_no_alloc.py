"""trips_adam_step_static against trips_adam_step.

Some users of this library run the optimizer step at a point where device memory cannot be allocated: the training
framework's pool already owns every free byte, or the host application forbids cudaMalloc after start-up.  For them
the library has a second Adam entry point whose tensor table sits in a fixed device array instead of allocated
scratch.  It must produce exactly what the allocating entry point produces (the two run the same kernel on the same
table, so the bar is bit equality), on a first call (which also resolves the array's address) and on a second call
that reuses the array; the second call must leave the amount of free device memory unchanged; and a call on a stream
that is being captured must be refused before anything is enqueued (the table is uploaded from the call's stack frame).

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
            _lib.check(L.trips_adam_step(ctx, _table(_lib, *ref, lr), len(sizes), stream), ctx)
            tab = _table(_lib, *new, lr)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]  # driver-level free memory: sees cudaMalloc by anyone in the process
            _lib.check(L.trips_adam_step_static(tab, len(sizes), stream))
            torch.cuda.synchronize()
            free_after = torch.cuda.mem_get_info()[0]
            if call == 1:  # (the first call may make the runtime load the module that holds the array)
                assert free_after == free_before, f"the static entry point changed free device memory by {free_before - free_after} bytes"
            for name, a, b in zip(("weights", "grads", "m", "v", "steps"), ref, new):
                for x, y in zip(a, b):
                    assert torch.equal(x, y), f"call {call}: {name} differ"
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


def test_static_adam_refuses_a_capturing_stream(cuda_lib):
    """The tensor table is copied from the call's own stack frame, so the call must not be recorded into a graph: on
    a capturing stream it returns TRIPS_ERR_UNSUPPORTED after a host-only check and touches nothing."""
    import torch
    from trips_b200 import _lib
    group = _tensors(torch, _lib, np.random.default_rng(4), [64, 9], 1e-3)
    before = [p.clone() for p in group[0]]
    tab = _table(_lib, *group, 1e-3)
    # first call on this device outside any capture (resolves the array's address)
    _lib.check(cuda_lib.trips_adam_step_static(tab, 2, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    after_one = [p.clone() for p in group[0]]
    assert any(not torch.equal(a, b) for a, b in zip(before, after_one))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        graph.capture_begin(capture_error_mode="thread_local")
        try:
            status = cuda_lib.trips_adam_step_static(tab, 2, C.c_void_p(torch.cuda.current_stream().cuda_stream))
        finally:
            graph.capture_end()
    torch.cuda.synchronize()
    assert status == _lib.ERR_UNSUPPORTED
    assert all(torch.equal(a, b) for a, b in zip(after_one, group[0])), "a refused call must not touch the tensors"
