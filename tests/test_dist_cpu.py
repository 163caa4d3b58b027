"""The view-parallel step with 2 ranks on CPU (gloo): every rank renders its own views with the CPU oracle, the flat
gradient buffer is summed with one all-reduce, Adam runs on every replica.  The result must equal the single-process
step over all views, and an element whose gradient is zero on every rank must stay untouched."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _scene():
    from trips_b200 import scenes
    return scenes.tiny(n_points=600, seed=41, width=48, height=32, num_layers=3, n_views=4)


def _local_grads(s, views):
    import oracle
    from trips_b200 import scenes
    from trips_b200.dist import FlatGradLayout
    layout = FlatGradLayout(s.n_points, s.n_points, s.channels)
    flat = np.zeros(layout.numel, np.float64)
    g = layout.views(flat)
    sa = oracle.SceneArrays.from_scene(s)
    p = oracle.make_params(s.num_layers, s.k_keep, True)
    for v in views:
        f = oracle.forward(sa, oracle.make_view(s.width, s.height, s.poses[v], s.intrinsics[v]), p)
        r = f.backward(scenes.target_gradient(s, v))
        g["texture"] += r["texture"]
        g["confidence"] += r["confidence"].reshape(1, -1)
        g["points"] += r["position"]
        g["point_size"] += r["point_size"].reshape(-1, 1)
        g["background"] += r["background"]
    return layout, flat.astype(np.float32)


def _adam(s, layout, flat):
    import oracle
    g = layout.views(flat)
    params = {"texture": s.texture.copy(), "confidence": s.confidence.reshape(1, -1).copy(), "points": s.position.copy(),
              "point_size": s.point_size.reshape(-1, 1).copy(), "background": s.background.copy()}
    for k, w in params.items():
        wf = w.reshape(-1)
        oracle.adam(wf, np.ascontiguousarray(g[k]).reshape(-1), np.zeros_like(wf), np.zeros_like(wf), np.zeros(wf.size, np.int64))
    return params


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    from trips_b200.dist import allreduce_sum, shard_views
    dist.init_process_group("gloo", rank=rank, world_size=world)
    s = _scene()
    layout, flat = _local_grads(s, shard_views(s.n_views, world, rank))
    t = torch.from_numpy(flat)
    allreduce_sum(t)
    params = _adam(s, layout, t.numpy())
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), flat=t.numpy(), **params)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_views_partitions_every_view_once():
    from trips_b200.dist import shard_views
    for n in (1, 7, 8, 64):
        for world in (1, 2, 3, 8):
            got = sum((shard_views(n, world, r) for r in range(world)), [])
            assert got == list(range(n))
            sizes = [len(shard_views(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_views(8, 2, 2)


def test_flat_layout_matches_reference_gradient_shapes():
    from trips_b200.dist import FlatGradLayout
    lay = FlatGradLayout(10, 12, 4)
    assert lay.numel == 4 * 12 + 12 + 40 + 10 + 4
    v = lay.views(np.arange(lay.numel, dtype=np.float32))
    assert v["texture"].shape == (4, 12) and v["points"].shape == (10, 4) and v["point_size"].shape == (10, 1)
    assert v["confidence"][0, 0] == 48 and v["background"][-1] == lay.numel - 1
    with pytest.raises(ValueError):
        lay.views(np.zeros(3, np.float32))


@pytest.mark.timeout(300)
def test_two_rank_step_equals_single_process(oracle_lib, tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    s = _scene()
    layout, flat = _local_grads(s, range(s.n_views))
    ref = _adam(s, layout, flat)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    assert np.array_equal(r0["flat"], r1["flat"])  # every replica sees the same sum
    scale = np.abs(flat).max()
    assert np.max(np.abs(r0["flat"] - flat)) <= 1e-6 * scale
    for k, w in ref.items():
        assert np.array_equal(r0[k], r1[k]), k
        np.testing.assert_allclose(r0[k], w, rtol=0, atol=2.5e-3)  # one Adam step moves a seen element by ~lr = 1e-3
        seen = np.ascontiguousarray(layout.views(flat)[k]) != 0
        start = {"texture": s.texture, "confidence": s.confidence.reshape(1, -1), "points": s.position,
                 "point_size": s.point_size.reshape(-1, 1), "background": s.background}[k]
        assert np.array_equal(r0[k][~seen], start[~seen]), f"{k}: elements unseen on every rank must not move"
        assert (r0[k][seen] != start[seen]).mean() > 0.99


def test_slice_bounds_cover_the_flat_vector_once():
    from trips_b200.dist import slice_bounds
    for numel in (0, 3, 4, 1001, 60_000_004):
        for world in (1, 2, 3, 8, 16):
            b = [slice_bounds(numel, world, r) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == numel
            for (lo, hi), (lo2, _) in zip(b, b[1:]):
                assert lo <= hi == lo2 and (lo % 4 == 0 or lo == hi)  # contiguous; non-empty slices start 16-byte aligned


def _failing_worker(rank, world, port, out_dir):
    """Rank 1 leaves before the gradient sum (between steps, nothing in flight); rank 0 must get an error, not a hang."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import datetime

    import torch
    import torch.distributed as dist
    from trips_b200.dist import allreduce_sum
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(1000)
    allreduce_sum(t)  # step 0: everybody is there
    assert float(t[0]) == world
    if rank == 1:
        os._exit(0)  # dies without saying goodbye
    outcome = "no error"
    try:
        allreduce_sum(t)  # step 1: the peer is gone
    except Exception as e:  # noqa: BLE001 - any error type is fine, a hang is not
        outcome = type(e).__name__
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)  # the process group cannot be shut down cleanly without the peer


@pytest.mark.timeout(120)
def test_lost_rank_surfaces_as_an_error_on_the_survivor(tmp_path):
    """Failure detection without touching a GPU: the collective of the surviving rank ends with an exception within
    the process-group timeout (the GPU path uses the same host-side mechanism: NCCL's timeout set at init)."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        assert not p.is_alive(), "a rank hung instead of failing"
    assert (tmp_path / "rank0.txt").read_text() != "no error"
