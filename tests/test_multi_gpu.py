"""The view-parallel step on two real GPUs: gradient sum over peer memory + Adam + parameter broadcast in one kernel
(trips_fused_reduce_adam through dist.FusedPointOptimizer) against NCCL all-reduce followed by trips_adam_step.

Two child processes, one per GPU (skipped on a box with one GPU).  Each rank renders and differentiates its own views
of a small scene with the CUDA library; the gradient buffer of the step is kept, reduced once by the fused kernel
(peer loads over NVLink, peer stores of the new weights into both replicas) and once by NCCL on a copy.  With two
ranks both sums add the same two numbers, so weights must agree bit for bit, the two replicas must be identical after
every step, and elements no rank touched must not move.  The library's kernel runs twice: over plain peer loads and
stores, and over NVSwitch multicast addresses (multimem.ld_reduce / multimem.st; skipped where the symmetric-memory
allocation has no multicast address).  NVLS is switched off for NCCL.  No rank leaves early (a failure on one rank is
written to its result file and the rank still joins the final barrier) and nothing waits without a limit.
"""
import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, multicast):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    import datetime

    import torch
    import torch.distributed as dist
    from trips_b200 import scenes
    from trips_b200.dist import FusedPointOptimizer, shard_views
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.optim import MyAdam
    from trips_b200.renderer import NeuralRenderInfo, PointRendererCache, RenderParams
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    s = scenes.tiny(n_points=40000, seed=61, width=160, height=96, num_layers=4, n_views=4)
    ns = NeuralScene.from_synthetic(s, device=dev)
    pc, tex = ns.point_cloud_cuda, ns.texture
    cache = PointRendererCache(dev)
    views = shard_views(s.n_views, world, rank)
    info = NeuralRenderInfo(scene=ns, images=images_for(s, views), params=RenderParams(num_texture_channels=s.channels, k_keep=s.k_keep),
                            num_layers=s.num_layers, train=True, cache=cache)
    params = [tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size, tex.background_color_raw]
    keys = ("texture", "confidence", "points", "point_size", "background")
    start = [p.detach().clone() for p in params]
    try:
        fused = FusedPointOptimizer(list(zip(keys, params)), cache, lr=1e-3, betas=(0.9, 0.999), multicast=multicast)
    except RuntimeError as exc:  # multicast required but not available: the same on every rank
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(f"SKIP: {exc}\n")
        dist.barrier()
        dist.destroy_process_group()
        return
    ref = [torch.nn.Parameter(p.detach().clone()) for p in params]
    ref_opt = MyAdam(ref, lr=1e-3, betas=(0.9, 0.999), cache=PointRendererCache(dev))
    gen = torch.Generator(device=dev)
    gen.manual_seed(100 + rank)
    ok, why, unseen_ok = True, "", True
    try:
        for step in range(3):
            args = (tex.texture, tex.background_color, pc.t_position, ns.intrinsics.intrinsics, tex.confidence_value_of_point, pc.t_point_size,
                    pc.t_index, ns.poses.poses_se3)
            outs = cache.forward(info, *args)
            grads_in = [torch.randn(o.shape, device=dev, generator=gen) * 1e-3 for o in outs]
            cache.backward(grads_in, *args, out=fused.grad_views)
            flat = fused.grad_flat.clone()  # the very same local gradients for both reductions
            before = [p.detach().clone() for p in params]
            fused.step()
            dist.all_reduce(flat)
            for k, p, b0 in zip(keys, params, before):  # MyAdam leaves elements alone whose summed gradient is zero (MyAdam.cu:57-61)
                o = fused.offsets[k]
                zero = flat[o:o + p.numel()].view(p.shape) == 0
                if not torch.equal(p.detach()[zero], b0[zero]):
                    unseen_ok = False
            for k, q in zip(keys, ref):
                o = fused.offsets[k]
                q.grad = flat[o:o + q.numel()].view(q.shape).clone()
            ref_opt.step()
            torch.cuda.synchronize()
            for k, p, q in zip(keys, params, ref):
                if not torch.equal(p.detach(), q.detach()):
                    ok, why = False, f"step {step}: {k} differs from all-reduce + Adam (max {float((p.detach() - q.detach()).abs().max())})"
            mine = torch.cat([p.detach().reshape(-1) for p in params]).view(torch.int32)
            both = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(both, mine)
            if not all(torch.equal(both[0], b) for b in both[1:]):
                ok, why = False, f"step {step}: the replicas differ"
    except Exception as exc:  # reported through the result file; the rank still joins the barrier below
        ok, why = False, f"{type(exc).__name__}: {exc}"
    moved = sum(int((p.detach() != s0).sum()) for p, s0 in zip(params, start))
    if cache.last_status() != 0:
        ok, why = False, "device status word raised"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(("ok " + fused.mode if ok and moved > 0 and unseen_ok else "FAIL: " + (why or f"moved={moved} unseen_ok={unseen_ok}")) + "\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("multicast", [False, True], ids=["peer_pointers", "multimem"])
def test_fused_reduce_adam_on_two_gpus(cuda_lib, tmp_path, multicast):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), multicast)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(420)
        assert not p.is_alive(), "a rank did not finish"
        assert p.exitcode == 0
    results = [(tmp_path / f"rank{r}.txt").read_text().strip() for r in range(2)]
    print("FUSED", results)
    if multicast and all("no multicast address" in res for res in results):
        pytest.skip("the symmetric-memory allocations have no multicast address on this machine")
    assert results[0] == results[1] == ("ok multimem" if multicast else "ok peer"), results
