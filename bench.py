#!/usr/bin/env python
"""Benchmark of the point-splatting training step (forward + backward + gradient all-reduce + fused Adam).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c2|c1|tiny]

One step = every rank renders its 8 views of the 6 M-point / 1920x1080 / 8-layer / K=16 scene, back-propagates
a gradient pyramid, the point gradients are summed over ranks (NCCL) and the fused Adam updates the point
parameters.  Rank 0 prints ONE JSON line.  `value` is views/s with all inputs resident in HBM; `e2e` is the same
step fed from pinned host memory (target pyramids H2D, L1 loss on the device, loss scalar D2H every step).
`--impl reference` times the CPU restatement of the reference's kernels (oracle/, OpenMP on the host cores): the
reference ships CUDA kernels only and cannot be built without its saiga submodule.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "fwd+bwd views/s (6M pts, 1920x1080, 8 layers, K=16, training step incl. grad all-reduce + fused Adam)"
RECORD_BYTES = 8  # bytes per kept fragment saved for backward (point id + alpha)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c3", "c2", "c1", "c4", "c5", "c5adv", "tiny"])
    ap.add_argument("--points", type=int, default=0, help="override the number of points (debugging)")
    ap.add_argument("--views-per-gpu", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--render-only", action="store_true",
                    help="step = inference render (train = 0) of the rank's views, no backward, no Adam: the render-only batch of "
                         "workload 5 (64 random views) is `--workload c5 --render-only --views-per-gpu 64/N`")
    ap.add_argument("--no-strong", action="store_true", help="N>1: skip the strong-scaling pass (8 views split over the ranks)")
    ap.add_argument("--cpu-views", type=int, default=12, help="views of the workload the CPU baseline renders")
    ap.add_argument("--op", default="step", choices=["step", "resize_points", "texture_prepare"],
                    help="'step' (default): the training-step benchmark; 'resize_points': removal of 10 % of the points over all "
                         "per-point tensors and the Adam state (trips_resize_points) against the numpy restatement")
    ap.add_argument("--collective", default="auto", choices=["auto", "fused", "fused-peer", "fused-multimem", "nccl"],
                    help="N>1: 'fused' = one kernel sums the gradients over peer memory, applies Adam and broadcasts; "
                         "(over peer pointers; 'fused-multimem' = through NVSwitch multicast addresses); 'nccl' = all-reduce then "
                         "Adam; 'auto' = fused over peer pointers when symmetric memory can be set up")
    return ap.parse_args()


def make_workload(name, world, rank, points, views_per_gpu):
    from trips_b200 import scenes
    if name == "c3":
        vpg = views_per_gpu or 8
        s = scenes.config3(n_points=points or 6_000_000, n_views=vpg * world)
    elif name == "c2":
        vpg = views_per_gpu or 4
        s = scenes.config2(n_points=points or 2_000_000, n_views=vpg * world)
    elif name == "c4":
        vpg = views_per_gpu or 2
        s = scenes.config4(n_points=points or 20_000_000, n_views=vpg * world)
    elif name in ("c5", "c5adv"):
        vpg = views_per_gpu or 8
        s = scenes.config5(n_points=points or 10_000_000, n_views=vpg * world, adversarial=(name == "c5adv"))
    elif name == "c1":
        vpg = 1
        s = scenes.config1(n_points=points or 200_000)
        s.train = True
    else:
        vpg = views_per_gpu or 2
        s = scenes.tiny(n_points=points or 4000, n_views=vpg * world)
    my_views = list(range(rank * vpg, rank * vpg + vpg)) if s.n_views >= (rank + 1) * vpg else list(range(vpg))
    return s, my_views, vpg


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def stage_bytes(stage, N, P, C, B, F, Kf, V=0):
    """Algorithmic bytes of one launch of a stage over B views (F, Kf, V are totals over those views)."""
    if stage == "bin_points":
        return 24 * N * B
    if stage == "count":
        return 4 * P * B
    if stage == "scan":
        return 8 * P * B
    if stage == "collect":
        return 8 * F
    if stage == "sort_blend":
        return 8 * F + (4 * C + 16) * Kf + 4 * C * P * B + RECORD_BYTES * Kf
    if stage == "blend_backward":
        return RECORD_BYTES * Kf + 4 * C * P * B + 8 * (C + 5) * Kf
    if stage == "adam":
        return 36 * (N * (C + 1 + 4 + 1))
    if stage == "unpack_grads":
        # no term in the reference's formula (its backward kernel adds straight into the outputs); what the stage must move:
        # per visible point and view one 32-byte gradient row cleared, read and its 32-byte entry head read, per point one row
        # (4 + C4 + 1 floats) cleared, read and written out in the reference's layouts
        c4 = (C + 3) // 4 * 4
        return 96 * V + (2 * 4 * (5 + c4) + 4 * (4 + 1 + C + 1)) * N
    return 0


# DRAM bytes (read + write) per unit of work, from the ncu captures summarised under profiles/: the tile kernels, the
# gradient finish / unpack kernels and Adam from one view of config 3 (rasterizer_kernels_c3_6Mpts_1view_ncu_sections.md:
# same list density and the same N as the benchmark), the binning kernels, which read every point once for all views of a
# call, from a quarter of the points with all 8 views (binning_adam_kernels_1.5Mpts_8views_ncu_sections.md).
# Traffic grows in proportion to the unit count.  Units: F fragments, Kf kept fragments, NB points x views, V entries
# (visible points over all views), N points.
DRAM_BYTES_PER_UNIT = {"count": [(5.2, "F")], "collect": [(20.2, "F")], "sort_blend": [(35.4, "F")], "blend_backward": [(41.6, "Kf")],
                       "bin_points": [(43.1, "NB")], "unpack_grads": [(23.4 + 126.5, "V"), (196.9, "N")], "adam": [(337.3, "N")]}


def stage_traffic(stage, N, B, F, Kf, V=0):
    if stage not in DRAM_BYTES_PER_UNIT:
        return None
    units = {"F": F, "Kf": Kf, "NB": N * B, "N": N, "V": V}
    return sum(per * units[unit] for per, unit in DRAM_BYTES_PER_UNIT[stage])


def fused_adam_bytes(numel, world):
    """One rank's launch: its slice of every rank's gradient, its parameters and state in, state and every replica out."""
    return (numel // world) * 4 * (world + 1 + 3 + 3 + world)


# ----------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle (restatement of the reference kernels) on the host cores
# ----------------------------------------------------------------------------------------------------------------
def cpu_views_per_second(s, views, repeats=1, with_backward=True):
    """Forward (+ backward) of `views` with the oracle; returns (views/s, seconds, fragments)."""
    import oracle
    from trips_b200 import scenes
    sa = oracle.SceneArrays.from_scene(s)
    p = oracle.make_params(s.num_layers, s.k_keep, with_backward)
    g = scenes.target_gradient(s, views[0])
    t0 = time.perf_counter()
    frags = 0
    n = 0
    for _ in range(repeats):
        for v in views:
            f = oracle.forward(sa, oracle.make_view(s.width, s.height, s.poses[v], s.intrinsics[v]), p)
            if with_backward:
                f.backward(g)
            frags += f.F
            n += 1
            del f
    dt = time.perf_counter() - t0
    return n / dt, dt, frags


def workload_config(s, B, world):
    """The keys that name the workload; both arms print the same ones."""
    return {"workload": s.name, "points": s.n_points, "views_per_gpu": B, "global_views_per_step": B * world, "width": s.width,
            "height": s.height, "layers": s.num_layers, "k_keep": s.k_keep, "channels": s.channels}


def run_reference(args, rank):
    """`--impl reference`: the CPU restatement of the reference's kernels timed on the host cores, on the GPU arm's
    configuration: one step = forward + backward of the rank-0 views of the workload and the Adam update of all point
    parameters (oracle.adam, MyAdam.cu:41-88).  Under torchrun only rank 0 works."""
    if rank != 0:
        return
    import oracle
    from trips_b200 import scenes
    oracle.build()
    cores = oracle.use_all_cores()
    s, my_views, vpg = make_workload(args.workload, 1, 0, args.points, args.views_per_gpu)
    sa = oracle.SceneArrays.from_scene(s)
    p = oracle.make_params(s.num_layers, s.k_keep, True)
    g = scenes.target_gradient(s, 0)
    # parameters in the reference's tensors; gradients are summed over the views in double and handed to Adam in float
    weights = {"texture": sa.texture.reshape(-1), "confidence": sa.confidence.reshape(-1), "position": sa.position.reshape(-1),
               "point_size": sa.point_size.reshape(-1)}
    state = {k: (np.zeros_like(w), np.zeros_like(w), np.zeros(w.size, np.int64)) for k, w in weights.items()}
    times = []
    for it in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        total = None
        for v in my_views:
            f = oracle.forward(sa, oracle.make_view(s.width, s.height, s.poses[v], s.intrinsics[v]), p)
            r = f.backward(g)
            del f
            if total is None:
                total = r
            else:
                for k in weights:
                    total[k] += r[k]
        for k, w in weights.items():
            m, v2, st = state[k]
            oracle.adam(w, np.ascontiguousarray(total[k].reshape(-1), dtype=np.float32), m, v2, st, lr=1e-3)
        dt = time.perf_counter() - t0
        if it >= args.warmup:
            times.append(dt)
    ms = 1000.0 * float(np.mean(times))
    value = len(my_views) * 1000.0 / ms
    sample = f"{len(my_views)} view(s) of {s.name} per step: forward + backward + Adam over all point parameters, {args.steps} steps"
    cfg = workload_config(s, len(my_views), 1)
    cfg["parallelism"] = f"OpenMP on {cores} host cores"
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "views/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "views/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "views/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })


# ----------------------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from trips_b200 import build as tb
    from trips_b200.dist import FlatGradLayout
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.optim import MyAdam
    from trips_b200.renderer import NeuralRenderInfo, PointRendererCache, RenderParams
    from trips_b200.scenes import layer_sizes, num_pyramid_pixels

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback for the GPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if rank == 0:
        tb.build()
    if world > 1:
        import datetime
        # a rank that never arrives ends the others' next collective with an error after this time instead of a hang
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        dist.barrier()

    s, my_views, vpg = make_workload(args.workload, world, rank, args.points, args.views_per_gpu)
    N, C, L = s.n_points, s.channels, s.num_layers
    P = num_pyramid_pixels(s.width, s.height, L)
    B = len(my_views)
    ns = NeuralScene.from_synthetic(s, device=dev)
    pc, tex = ns.point_cloud_cuda, ns.texture
    cache = PointRendererCache(dev)
    info = NeuralRenderInfo(scene=ns, images=images_for(s, my_views), params=RenderParams(num_texture_channels=C, k_keep=s.k_keep),
                            num_layers=L, train=True, cache=cache)
    # all point gradients live in one flat buffer so that one collective (or one fused kernel) sums them over ranks
    params = [tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size, tex.background_color_raw]
    keys = ("texture", "confidence", "points", "point_size", "background")
    fused, collective = None, "none"
    if world > 1 and args.collective in ("auto", "fused", "fused-peer", "fused-multimem"):
        from trips_b200.dist import FusedPointOptimizer
        ok = torch.ones(1, device=dev)
        try:
            fused = FusedPointOptimizer(list(zip(keys, params)), cache, lr=1e-3, betas=(0.9, 0.999),
                                        multicast={"fused-peer": False, "fused-multimem": True}.get(args.collective))
        except Exception as e:  # noqa: BLE001 - symmetric memory is optional plumbing; the NCCL path is always there
            if args.collective in ("fused", "fused-peer", "fused-multimem"):
                raise
            print(f"[bench] rank {rank}: symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL all-reduce", file=sys.stderr)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            fused = None
    if fused is not None:
        gout = fused.grad_views
        collective = ("fused multimem reduce + Adam + multicast store (trips_fused_reduce_adam_multicast)" if fused.mode == "multimem"
                      else "fused peer-memory reduce + Adam + broadcast (trips_fused_reduce_adam)")
        opt, flat = None, fused.grad_flat
    else:
        layout = FlatGradLayout(N, N, C)
        flat = torch.zeros(layout.numel, device=dev)
        gout = layout.views(flat)
        for p_, k in zip(params, keys):
            p_.grad = gout[k]
        opt = MyAdam(params, lr=1e-3, betas=(0.9, 0.999), cache=cache)
        collective = "nccl all_reduce + trips_adam_step" if world > 1 else "none (single GPU)"

    def reduce_and_update():
        if fused is not None:
            fused.step()
            return
        if world > 1:
            dist.all_reduce(flat)
        opt.step()
    sizes = layer_sizes(s.width, s.height, L)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    numel = C * P
    grads_in = [((torch.randint(0, 2, (B, C, h, w), device=dev, generator=gen).float() * 2 - 1) / numel) for (w, h) in sizes]
    scene_args = lambda: (tex.texture, tex.background_color, pc.t_position, ns.intrinsics.intrinsics,  # noqa: E731
                          tex.confidence_value_of_point, pc.t_point_size, pc.t_index, ns.poses.poses_se3)

    def step_resident():
        outs = cache.forward(info, *scene_args())
        cache.backward(grads_in, *scene_args(), out=gout)
        reduce_and_update()
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.render_only:
        info.train = False

        def step_resident():  # noqa: F811 - the render-only step replaces the training step
            with torch.no_grad():
                return cache.forward(info, *scene_args())

    # the clock sampler starts with the warm-up steps (the same load): nvidia-smi needs some 100 ms before its first sample
    # and the timed region of the default run is not much longer than that
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_resident()
    barrier()
    stats = cache.stats()
    assert cache.last_status() == 0, "device status word raised"

    # ---- timed region: K steps, inputs resident in HBM.  Working set per step (>2 GB) is far larger than L2. ----
    cache.enable_stage_timers(True)
    cache.stage_times(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    e0.record()
    marks[0].record()
    for i in range(args.steps):
        step_resident()
        marks[i + 1].record()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps))
    pct = lambda q: per_step[min(len(per_step) - 1, int(round(q * (len(per_step) - 1))))]  # noqa: E731
    step_stats = {"median": pct(0.5), "p10": pct(0.1), "p90": pct(0.9)}
    clocks = sampler.stop() if sampler else None
    st = cache.stage_times(reset=True)
    cache.enable_stage_timers(False)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = world * B / (ms_step / 1000.0)

    # ---- end to end: targets come from pinned host memory, loss goes back to the host, every step ----
    e2e = None
    if not args.no_e2e and args.render_only:
        # the step's inputs are the camera poses of its views (pinned host memory), its result is the image pyramid of
        # every view, copied back to pinned host memory; the host waits for the images every step
        poses_host = ns.poses.poses_se3.detach().cpu().pin_memory()
        host_out = [torch.empty((B, C, h, w)).pin_memory() for (w, h) in sizes]
        d2h = sum(x.numel() * 4 for x in host_out)

        def step_e2e_render():
            ns.poses.poses_se3.copy_(poses_host, non_blocking=True)
            outs = step_resident()
            for h_, o in zip(host_out, outs):
                h_.copy_(o, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()

        for _ in range(2):
            step_e2e_render()
        barrier()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            step_e2e_render()
        e1.record()
        barrier()
        wall = (time.perf_counter() - t0) * 1000.0
        te = torch.tensor([max(e0.elapsed_time(e1), 0.0)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e_step = float(te.item()) / args.steps
        e2e = {"value": world * B / (ms_e_step / 1000.0), "unit": "views/s", "h2d_bytes_per_step": int(poses_host.numel() * 8),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": ms_e_step, "wall_ms_per_step": wall / args.steps}
    elif not args.no_e2e:
        rng = np.random.Generator(np.random.Philox(4242 + rank))
        host_t = [torch.from_numpy(rng.random((B, C, h, w), dtype=np.float32)).pin_memory() for (w, h) in sizes]
        dev_t = [[torch.empty_like(x, device=dev) for x in host_t] for _ in range(2)]
        grads_e = [torch.empty((B, C, h, w), device=dev) for (w, h) in sizes]
        loss_dev = torch.zeros((), device=dev, dtype=torch.float64)
        loss_host = torch.zeros((), dtype=torch.float64).pin_memory()
        copy_stream = torch.cuda.Stream(dev)
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        h2d = sum(x.numel() * 4 for x in host_t)

        def upload(slot):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[slot])
                for d, h_ in zip(dev_t[slot], host_t):
                    d.copy_(h_, non_blocking=True)
                ready[slot].record(copy_stream)

        def step_e2e(i, last):
            slot = i & 1
            if not last:
                upload(slot ^ 1)  # next step's targets travel while this step computes
            cur = torch.cuda.current_stream(dev)
            cur.wait_event(ready[slot])
            outs = cache.forward(info, *scene_args())
            cache.l1_loss_backward(outs, dev_t[slot], grads_e, loss_dev)
            consumed[slot].record(cur)
            cache.backward(grads_e, *scene_args(), out=gout)
            reduce_and_update()
            loss_host.copy_(loss_dev, non_blocking=True)
            cur.synchronize()  # the caller reads the loss every step
            return float(loss_host)

        for slot in (0, 1):
            consumed[slot].record(torch.cuda.current_stream(dev))
        upload(0)
        for i in range(2):
            step_e2e(i, False)
        barrier()
        t0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            step_e2e(i, i == args.steps - 1)
        e1.record()
        barrier()
        wall = (time.perf_counter() - t0) * 1000.0
        ms_e = max(e0.elapsed_time(e1), 0.0)
        te = torch.tensor([ms_e], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e_step = float(te.item()) / args.steps
        e2e = {"value": world * B / (ms_e_step / 1000.0), "unit": "views/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": 8, "ms_per_step": ms_e_step, "wall_ms_per_step": wall / args.steps}
        # host link: the copy of the next step's targets runs beside the kernels of this step; what it takes of the host
        # memory system grows with the number of ranks copying at once (every GPU of these machines reports NUMA node 0,
        # so there is no closer node to allocate the pinned buffers on)
        e2e["host_link"] = {"h2d_gb_per_s_per_gpu": h2d / (ms_e_step * 1e6), "h2d_gb_per_s_all_gpus": world * h2d / (ms_e_step * 1e6),
                            "ms_over_device_step": ms_e_step - ms_step}

    # ---- N > 1: the same global batch of 8 views split over the ranks (8 / N per rank): strong scaling ----
    strong = None
    if world > 1 and not args.render_only and not args.no_strong and args.workload == "c3" and 8 % world == 0 and B >= 8 // world:
        sb = 8 // world
        info_s = NeuralRenderInfo(scene=ns, images=images_for(s, my_views[:sb]), params=info.params, num_layers=L, train=True, cache=cache)
        grads_s = [g[:sb].contiguous() for g in grads_in]

        def step_strong():
            cache.forward(info_s, *scene_args())
            cache.backward(grads_s, *scene_args(), out=gout)
            reduce_and_update()

        for _ in range(max(args.warmup, 3)):
            step_strong()
        barrier()
        e0.record()
        for _ in range(args.steps):
            step_strong()
        e1.record()
        barrier()
        ts = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        ms_s = float(ts.item()) / args.steps
        strong = {"scaling": "strong", "global_views_per_step": 8, "views_per_gpu": sb, "ms_per_step": ms_s, "value": 8.0 / (ms_s * 1e-3),
                  "unit": "views/s", "note": "the same 6 M-point scene, 8 views per step split over the ranks, gradient sum + Adam every step"}

    # ---- N > 1: every rank must hold the same parameters after the same number of steps ----
    replicas_equal = None
    if world > 1 and not args.render_only:
        digest = []
        for p_ in params:
            v = p_.detach().reshape(-1).view(torch.int32).to(torch.int64)
            w_ = (torch.arange(v.numel(), device=dev, dtype=torch.int64) % 65521) + 1
            digest += [v.sum(), (v * w_).sum()]
        mine = torch.stack(digest)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        replicas_equal = all(bool(torch.equal(allr[0], x)) for x in allr[1:])
    status_after = cache.last_status()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel, from the stage timers of the timed region ----
    peak, peak_kind = measured_peak()
    F, Kf = stats["fragments"], stats["kept_fragments"]
    per_stage = {}
    launches_total = 0
    for name, (ms, calls, launches) in st.items():
        launches_total += launches
        if calls:
            # a stage may be timed in several spans per step (the unpack stage: clearing the accumulators before the
            # backward kernel, finishing them after it): the figure is the stage's time per step
            per_stage[name] = {"ms_per_launch": ms / args.steps, "launches": int(launches)}
    step_stages = ("bin_points", "count", "scan", "collect", "sort_blend", "blend_backward", "unpack_grads", "adam", "fused_reduce_adam")
    if args.render_only:
        step_stages = ("bin_points", "count", "scan", "collect", "sort_blend")

    def bytes_of(k):
        if k == "fused_reduce_adam":
            return fused_adam_bytes(fused.numel, world) if fused is not None else 0
        if k == "adam" and fused is not None:
            return 0
        return stage_bytes(k, N, P, C, B, F, Kf, stats["visible_points"])

    dom = max((k for k in per_stage if k in step_stages), key=lambda k: per_stage[k]["ms_per_launch"])
    dom_bytes = bytes_of(dom)
    achieved = dom_bytes / (per_stage[dom]["ms_per_launch"] * 1e-3) / 1e9
    for k, v in per_stage.items():
        b_ = bytes_of(k)
        v["alg_gb"] = b_ / 1e9
        v["gbs"] = (b_ / (v["ms_per_launch"] * 1e-3) / 1e9) if b_ else None
    total_alg = sum(bytes_of(k) for k in step_stages)
    V = stats["visible_points"]
    dom_traffic = stage_traffic(dom, N, B, F, Kf, V)
    total_traffic = sum(stage_traffic(k, N, B, F, Kf, V) or 0 for k in per_stage if k in step_stages)
    for k, v in per_stage.items():
        t_ = stage_traffic(k, N, B, F, Kf, V)
        v["dram_gb"] = t_ / 1e9 if t_ else None
        v["traffic_over_alg"] = (t_ / bytes_of(k)) if (t_ and bytes_of(k)) else None
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": peak_kind, "traffic": dom_traffic,
                # the same kernel on measured DRAM bytes: much of its algorithmic traffic (gradient read-modify-writes) stays in L2
                "frac_dram": (dom_traffic / (per_stage[dom]["ms_per_launch"] * 1e-3) / 1e9 / peak) if dom_traffic else None,
                # the whole step against the HBM roofline: algorithmic bytes of all stages / step time, and the same on measured DRAM bytes
                "step_frac": total_alg / (ms_step * 1e-3) / 1e9 / peak,
                "step_frac_dram": (total_traffic / (ms_step * 1e-3) / 1e9 / peak) if total_traffic else None,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per unit of work (profiles/rasterizer_kernels_c3_6Mpts_1view_ncu_sections.md, binning_adam_kernels_1.5Mpts_8views_ncu_sections.md) x units of this run",
                "alg_bytes_per_launch": dom_bytes,
                "step_alg_bytes": total_alg, "step_gbs": total_alg / (ms_step * 1e-3) / 1e9, "stages": per_stage}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        oracle.use_all_cores()
        vps, secs, cfr = cpu_views_per_second(s, [my_views[i % B] for i in range(args.cpu_views)], with_backward=not args.render_only)
        what = "forward only" if args.render_only else "forward + backward"
        cpu = {"value": vps, "unit": "views/s", "cores": oracle.max_threads(), "kind": "port",
               "sample": f"{args.cpu_views} view(s) of {s.name}, {what} with the OpenMP oracle ({secs:.1f} s)"}

    out = {
        "metric": METRIC, "value": value, "unit": "views/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "ms_per_view": ms_step / B, "step_ms": step_stats, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {**workload_config(s, B, world), "parallelism": f"view-dp{world}", "collective": collective,
                   "step": "render only (train = 0)" if args.render_only else "forward + backward + gradient sum + Adam",
                   "l2_policy": "inputs (>2 GB touched per step) larger than the 126 MB L2; no explicit flush",
                   "fragments_per_step": int(F), "kept_fragments_per_step": int(Kf), "visible_points_per_step": int(stats["visible_points"]),
                   "max_list_length": int(stats["max_list_length"]), "fragments_per_s": F * world / (ms_step * 1e-3),
                   "backward_atomic_floats_per_s": (C + 5) * Kf / (per_stage["blend_backward"]["ms_per_launch"] * 1e-3) if "blend_backward" in per_stage else None},
        "e2e": e2e, "gpu_launches": int(launches_total), "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
        "device_status_after_run": int(status_after),
    }
    if strong is not None:
        out["strong"] = strong
    if replicas_equal is not None:
        out["replicas_equal"] = replicas_equal
    emit(out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_resize(args):
    """Secondary measurement: one device pass that removes 10 % of the points of the workload's scene from position,
    size, texture, confidence and their Adam state (16 tensors), against numpy on the host."""
    import torch
    import oracle
    from trips_b200 import build as tb
    from trips_b200.modules import NeuralScene
    from trips_b200.optim import MyAdam
    from trips_b200.renderer import PointRendererCache
    tb.build()
    oracle.build()
    dev = torch.device("cuda", 0)
    s, _, _ = make_workload(args.workload, 1, 0, args.points, 1)
    N, C = s.n_points, s.channels
    rng = np.random.Generator(np.random.Philox(7))
    remove = rng.permutation(N)[: N // 10]
    rem_dev = torch.from_numpy(remove).to(dev)
    times = []
    for it in range(max(args.warmup, 3) + args.steps):
        ns = NeuralScene.from_synthetic(s, device=dev)
        pc, tex = ns.point_cloud_cuda, ns.texture
        cache = PointRendererCache(dev)
        params = [tex.texture_raw, tex.confidence_raw, pc.t_position, pc.t_point_size]
        opt = MyAdam(params, lr=1e-3, cache=cache)
        for p_ in params:
            p_.grad = torch.ones_like(p_)
        opt.step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ns.ResizePoints(cache, rem_dev, optimizers=[opt])
        e1.record()
        torch.cuda.synchronize()
        if it >= max(args.warmup, 3):
            times.append(e0.elapsed_time(e1))
        assert cache.last_status() == 0
        del ns, opt, cache
    ms = float(np.median(times))
    rows = 4 * (C + 1 + 4 + 1) + 4  # parameters + three state tensors each, + original colour
    alg = 4 * rows * (N + (N - N // 10))  # every element read once, kept elements written once
    spec = []
    for shape, pm in (((N, 4), True), ((N, 1), True), ((C, N), False), ((1, N), False)):
        for _ in range(4):
            spec.append((np.zeros(shape, np.float32), pm, 0.0))
    t0 = time.perf_counter()
    oracle.resize_points(spec, remove, N - N // 10)
    cpu_s = time.perf_counter() - t0
    peak, kind = measured_peak()
    emit({"metric": "points/s through removal of 10 % of the points over all per-point tensors and Adam state", "value": N / (ms * 1e-3),
          "unit": "points/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
          "dtype": "u32", "data": "synthetic", "config": {"workload": s.name, "points": N, "removed": int(N // 10), "tensors": 17},
          "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "frac": alg / (ms * 1e-3) / 1e9 / peak,
                       "peak_kind": kind, "traffic": None, "note": "includes torch allocation of the 17 destination tensors"},
          "cpu_baseline": {"value": N / cpu_s, "unit": "points/s", "cores": 1, "kind": "port",
                           "sample": f"numpy take over 16 float32 tensors of the same shapes ({cpu_s:.2f} s)"}})


def run_texture_prepare(args):
    """Secondary measurement: forward + backward of the workload with the texture preparation (sigmoid(10 raw) on the
    confidences, |raw| on the descriptors, NeuralTexture.h:40-57) done by torch ops with autograd, as the reference
    does, against the same step with the preparation fused into the rasterizer (confidence_is_raw / texture_abs)."""
    import torch
    from trips_b200 import build as tb
    from trips_b200.modules import NeuralScene, images_for
    from trips_b200.renderer import NeuralRenderInfo, PointRendererCache, RenderParams
    from trips_b200.scenes import layer_sizes
    tb.build()
    dev = torch.device("cuda", 0)
    s, my_views, _ = make_workload(args.workload, 1, 0, args.points, args.views_per_gpu)
    C, L, B = s.channels, s.num_layers, len(my_views)
    ns = NeuralScene.from_synthetic(s, device=dev)
    pc, tex = ns.point_cloud_cuda, ns.texture
    with torch.no_grad():  # raw parameters whose activations are the workload's values
        tex.confidence_raw.copy_(torch.logit(tex.confidence_raw.clamp(1e-4, 1 - 1e-4)) / 10.0)
    cache = PointRendererCache(dev)
    grads_in = [torch.full((B, C, h, w), 1e-6, device=dev) for (w, h) in layer_sizes(s.width, s.height, L)]
    results = {}
    for fused in (False, True):
        info = NeuralRenderInfo(scene=ns, images=images_for(s, my_views),
                                params=RenderParams(num_texture_channels=C, k_keep=s.k_keep, confidence_is_raw=fused, confidence_scale=10.0,
                                                    texture_abs=fused), num_layers=L, train=True, cache=cache)

        def step():
            if fused:
                t, c = tex.texture_raw, tex.confidence_raw
            else:
                t, c = torch.abs(tex.texture_raw), torch.sigmoid(10.0 * tex.confidence_raw)
            cache.forward(info, t, tex.background_color, pc.t_position, ns.intrinsics.intrinsics, c, pc.t_point_size, pc.t_index,
                          ns.poses.poses_se3)
            g = cache.backward(grads_in, t, tex.background_color, pc.t_position, ns.intrinsics.intrinsics, c, pc.t_point_size, pc.t_index,
                               ns.poses.poses_se3)
            if not fused:  # the backward of the two torch ops, as autograd would run them
                g_tex, g_conf = g[0], g[5]
                g_tex = g_tex * torch.sign(tex.texture_raw)
                sg = torch.sigmoid(10.0 * tex.confidence_raw)
                g_conf = g_conf * (10.0 * sg * (1.0 - sg))
            return g

        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        results[fused] = e0.elapsed_time(e1) / args.steps
        assert cache.last_status() == 0
    emit({"metric": "fwd+bwd views/s with the texture preparation fused into the rasterizer", "value": B / (results[True] * 1e-3),
          "unit": "views/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": results[True],
          "higher_is_better": True, "dtype": "f32", "data": "synthetic",
          "config": {"workload": s.name, "points": s.n_points, "views_per_gpu": B, "unfused_ms_per_step": results[False],
                     "saved_ms_per_step": results[False] - results[True]}})


_JSON_FD = None


def emit(obj):
    """The one JSON line, written to the process's original stdout."""
    line = (json.dumps(obj) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, line)


def main():
    global _JSON_FD
    args = parse_args()
    # Libraries write to stdout behind our back (NCCL prints its version banner there at the WARN and VERSION debug
    # levels).  Stdout must carry the JSON line only: keep the original descriptor for it and point fd 1 at stderr.
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.op == "resize_points":
        if rank == 0:
            run_resize(args)
        return
    if args.op == "texture_prepare":
        if rank == 0:
            run_texture_prepare(args)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
