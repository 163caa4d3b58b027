"""Seeded synthetic scenes standing in for the datasets TRIPS is trained on.

The reference trains on Tanks&Temples / MipNeRF-360 captures (README.md:237-261) which are not available
offline; these generators produce point clouds, cameras and gradients with the shapes, sizes and value
distributions of the five benchmark workloads.  Everything is generated with numpy's counter-based Philox
generator so that the CPU oracle, the CUDA library and the benchmarks see identical bytes.

Layouts follow the reference's parameter store:
  position   [N,4] f32  xyz + drop-out radius      (NeuralPointCloudCuda.cpp:56-66, t_position)
  point_size [N]   f32  inverse_softplus(size)     (NeuralPointCloudCuda.cpp:19-24,50, t_point_size)
  texture    [C,N] f32, confidence [N] f32 (post-sigmoid), background [C] f32 (NeuralTexture.cpp:14-63)
  poses      [B,8] f64  world->view quaternion (x,y,z,w), translation, one pad (NeuralStructure.cpp:20-33)
  intrinsics [B,13] f32 fx fy cx cy s + 8 zero distortion coefficients (NeuralStructure.cpp:104-117)
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Scene:
    name: str
    position: np.ndarray
    point_size: np.ndarray
    texture: np.ndarray
    confidence: np.ndarray
    background: np.ndarray
    poses: np.ndarray
    intrinsics: np.ndarray
    width: int
    height: int
    num_layers: int
    k_keep: int
    train: bool
    seed: int
    extra: dict = field(default_factory=dict)

    @property
    def n_points(self) -> int:
        return self.position.shape[0]

    @property
    def n_views(self) -> int:
        return self.poses.shape[0]

    @property
    def channels(self) -> int:
        return self.texture.shape[0]


def layer_sizes(w: int, h: int, num_layers: int):
    """Pyramid sizes with ceil halving (PointRenderer.cu:385-389)."""
    out = []
    for _ in range(num_layers):
        out.append((w, h))
        w = (w + 1) // 2
        h = (h + 1) // 2
    return out


def num_pyramid_pixels(w: int, h: int, num_layers: int) -> int:
    return sum(a * b for a, b in layer_sizes(w, h, num_layers))


def inverse_softplus(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    return np.where(x > 20.0, x, np.log(np.expm1(np.minimum(x, 20.0)))).astype(np.float32)


def _rot_to_quat(R: np.ndarray) -> np.ndarray:
    """Rotation matrix -> unit quaternion (x, y, z, w)."""
    t = np.trace(R)
    if t > 0:
        s = np.sqrt(t + 1.0) * 2
        q = np.array([(R[2, 1] - R[1, 2]) / s, (R[0, 2] - R[2, 0]) / s, (R[1, 0] - R[0, 1]) / s, 0.25 * s])
    elif R[0, 0] > R[1, 1] and R[0, 0] > R[2, 2]:
        s = np.sqrt(1.0 + R[0, 0] - R[1, 1] - R[2, 2]) * 2
        q = np.array([0.25 * s, (R[0, 1] + R[1, 0]) / s, (R[0, 2] + R[2, 0]) / s, (R[2, 1] - R[1, 2]) / s])
    elif R[1, 1] > R[2, 2]:
        s = np.sqrt(1.0 + R[1, 1] - R[0, 0] - R[2, 2]) * 2
        q = np.array([(R[0, 1] + R[1, 0]) / s, 0.25 * s, (R[1, 2] + R[2, 1]) / s, (R[0, 2] - R[2, 0]) / s])
    else:
        s = np.sqrt(1.0 + R[2, 2] - R[0, 0] - R[1, 1]) * 2
        q = np.array([(R[0, 2] + R[2, 0]) / s, (R[1, 2] + R[2, 1]) / s, 0.25 * s, (R[1, 0] - R[0, 1]) / s])
    return q / np.linalg.norm(q)


def look_at_pose(eye, target, up=(0.0, -1.0, 0.0)) -> np.ndarray:
    """World->view pose (8 doubles) of a camera at `eye` looking at `target`; view axes: x right, y down, z forward."""
    eye = np.asarray(eye, dtype=np.float64)
    target = np.asarray(target, dtype=np.float64)
    fwd = target - eye
    fwd /= np.linalg.norm(fwd)
    upv = np.asarray(up, dtype=np.float64)
    right = np.cross(fwd, -upv)
    if np.linalg.norm(right) < 1e-6:
        right = np.cross(fwd, np.array([1.0, 0.0, 0.0]))
    right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    R = np.stack([right, down, fwd])  # rows = view axes in world coordinates
    t = -R @ eye
    out = np.zeros(8, dtype=np.float64)
    out[:4] = _rot_to_quat(R)
    out[4:7] = t
    return out


def _intrinsics(n: int, fx: float, w: int, h: int) -> np.ndarray:
    K = np.zeros((n, 13), dtype=np.float32)
    K[:, 0] = fx
    K[:, 1] = fx
    K[:, 2] = w / 2
    K[:, 3] = h / 2
    return K


def _log_uniform(rng, lo, hi, n):
    return np.exp(rng.uniform(np.log(lo), np.log(hi), n))


def _points_on_surfaces(rng, n, n_surfaces, box):
    """Points on random planes (square patches) and spheres inside a cube of edge `box` centred at the origin."""
    half = box / 2
    kind = rng.integers(0, 2, n_surfaces)
    centre = rng.uniform(-half * 0.8, half * 0.8, (n_surfaces, 3))
    extent = rng.uniform(0.1 * box, 0.35 * box, n_surfaces)
    normal = rng.normal(size=(n_surfaces, 3))
    normal /= np.linalg.norm(normal, axis=1, keepdims=True)
    which = rng.integers(0, n_surfaces, n)
    pts = np.empty((n, 3), dtype=np.float64)
    # plane patches
    a = np.cross(normal, np.array([0.3, 0.5, 0.8]))
    a /= np.linalg.norm(a, axis=1, keepdims=True)
    b = np.cross(normal, a)
    uv = rng.uniform(-1, 1, (n, 2))
    plane_pts = centre[which] + (uv[:, :1] * a[which] + uv[:, 1:] * b[which]) * extent[which, None]
    d = rng.normal(size=(n, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    sphere_pts = centre[which] + d * (0.5 * extent[which, None])
    is_plane = kind[which] == 0
    pts[is_plane] = plane_pts[is_plane]
    pts[~is_plane] = sphere_pts[~is_plane]
    return np.clip(pts, -half, half)


def _finish(name, rng, pts, sizes, poses, fx, w, h, L, K, train, seed, channels=4, extra=None) -> Scene:
    n = pts.shape[0]
    position = np.empty((n, 4), dtype=np.float32)
    position[:, :3] = pts
    position[:, 3] = sizes
    texture = rng.uniform(0, 1, (channels, n)).astype(np.float32)
    confidence = rng.uniform(0, 1, n).astype(np.float32)
    background = np.full(channels, 0.25, dtype=np.float32)  # NeuralTexture.cpp:18,37
    poses = np.ascontiguousarray(poses, dtype=np.float64)
    return Scene(name, position, inverse_softplus(sizes), texture, confidence, background, poses,
                 _intrinsics(poses.shape[0], fx, w, h), w, h, L, K, train, seed, extra or {})


def _ring_poses(n_views, radius, height=0.0, jitter=None, rng=None):
    poses = []
    for i in range(n_views):
        ang = 2 * np.pi * i / n_views
        eye = np.array([radius * np.cos(ang), height, radius * np.sin(ang)])
        if jitter is not None and rng is not None:
            eye = eye + rng.uniform(-jitter, jitter, 3)
        poses.append(look_at_pose(eye, (0.0, 0.0, 0.0)))
    return np.stack(poses)


def config1(n_points=200_000, seed=0) -> Scene:
    """Forward-only render: unit sphere + N(0, 0.01) noise, sizes log-U[1e-3, 1e-1], 640x480 fx=500 at distance 3."""
    rng = np.random.Generator(np.random.Philox(seed))
    d = rng.normal(size=(n_points, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    pts = d + rng.normal(scale=0.01, size=(n_points, 3))
    sizes = _log_uniform(rng, 1e-3, 1e-1, n_points)
    poses = look_at_pose((0.0, 0.0, -3.0), (0.0, 0.0, 0.0))[None]
    return _finish("c1_sphere_200k_640x480_L4_K8", rng, pts, sizes, poses, 500.0, 640, 480, 4, 8, False, seed)


def config2(n_points=2_000_000, seed=2, n_views=4) -> Scene:
    """Forward+backward: 32 planes/spheres in a 10 m box, sizes log-U[1e-3, 5e-2], 1280x720 fx=1000 on a ring r=6."""
    rng = np.random.Generator(np.random.Philox(seed))
    pts = _points_on_surfaces(rng, n_points, 32, 10.0)
    sizes = _log_uniform(rng, 1e-3, 5e-2, n_points)
    poses = _ring_poses(n_views, 6.0, height=-1.0)
    return _finish("c2_surfaces_2M_1280x720_L6_K16", rng, pts, sizes, poses, 1000.0, 1280, 720, 6, 16, True, seed)


def config3(n_points=6_000_000, seed=3, n_views=8, width=1920, height=1080, fx=1500.0) -> Scene:
    """Training step: random surfaces in a 20 m box, 8 views 1920x1080 fx=1500, 8 layers, K=16."""
    rng = np.random.Generator(np.random.Philox(seed))
    pts = _points_on_surfaces(rng, n_points, 64, 20.0)
    sizes = _log_uniform(rng, 1e-3, 5e-2, n_points)
    poses = _ring_poses(n_views, 13.0, height=-3.0)
    return _finish(f"c3_surfaces_{n_points}_{width}x{height}_L8_K16", rng, pts, sizes, poses, fx, width, height, 8, 16,
                   True, seed)


def config4(n_points=20_000_000, seed=4, n_views=4) -> Scene:
    """Large-scene stress: 70 % on a 200 m ground plane, 30 % Gaussian clusters, Pareto(1.5) sizes, 2560x1440."""
    rng = np.random.Generator(np.random.Philox(seed))
    n_ground = int(n_points * 0.7)
    n_cl = n_points - n_ground
    ground = np.zeros((n_ground, 3))
    ground[:, 0] = rng.uniform(-100, 100, n_ground)
    ground[:, 2] = rng.uniform(-100, 100, n_ground)
    ground[:, 1] = rng.normal(scale=0.02, size=n_ground)
    centres = np.stack([rng.uniform(-90, 90, 48), rng.uniform(-6, -0.5, 48), rng.uniform(-90, 90, 48)], axis=1)
    which = rng.integers(0, 48, n_cl)
    clusters = centres[which] + rng.normal(scale=1.5, size=(n_cl, 3))
    pts = np.concatenate([ground, clusters])
    sizes = np.minimum(2e-3 * (1.0 + rng.pareto(1.5, n_points)), 2.0)
    poses = []
    for i in range(n_views):
        ang = 2 * np.pi * i / n_views + 0.3
        eye = np.array([60 * np.cos(ang), -1.7, 60 * np.sin(ang)])
        poses.append(look_at_pose(eye, (0.0, -1.0, 0.0)))
    return _finish("c4_ground_clusters_20M_2560x1440_L8_K16", rng, pts, sizes, np.stack(poses), 2000.0, 2560, 1440, 8, 16,
                   True, seed)


def config5(n_points=10_000_000, seed=5, n_views=64, adversarial=False) -> Scene:
    """Render-only batch of random 1080p views over 10 M points; `adversarial` squeezes every point into 64x64 px."""
    rng = np.random.Generator(np.random.Philox(seed))
    if adversarial:
        # a small blob far away on the optical axis: everything lands in a ~64x64 pixel window
        pts = rng.uniform(-1, 1, (n_points, 3)) * np.array([0.6, 0.6, 0.6])
        sizes = _log_uniform(rng, 1e-3, 5e-2, n_points)
        poses = np.stack([look_at_pose((0.0, 0.0, -30.0), (0.0, 0.0, 0.0)) for _ in range(n_views)])
        name = f"c5_adversarial_{n_points}_64x64px"
    else:
        pts = _points_on_surfaces(rng, n_points, 64, 20.0)
        sizes = _log_uniform(rng, 1e-3, 5e-2, n_points)
        poses = []
        for _ in range(n_views):
            d = rng.normal(size=3)
            d /= np.linalg.norm(d)
            eye = d * rng.uniform(11.0, 16.0)
            poses.append(look_at_pose(eye, rng.uniform(-3, 3, 3)))
        poses = np.stack(poses)
        name = f"c5_random_views_{n_points}_1920x1080_L8_K16"
    return _finish(name, rng, pts, sizes, poses, 1500.0, 1920, 1080, 8, 16, False, seed)


def tiny(n_points=4000, seed=7, width=96, height=64, num_layers=4, k_keep=16, n_views=2, train=True, fx=90.0,
         size_range=(5e-3, 0.4), channels=4) -> Scene:
    """A small scene with a wide spread of projected sizes; lists longer than K occur.  Used by parity tests."""
    rng = np.random.Generator(np.random.Philox(seed))
    pts = rng.uniform(-1.5, 1.5, (n_points, 3))
    sizes = _log_uniform(rng, size_range[0], size_range[1], n_points)
    poses = _ring_poses(n_views, 4.0, height=-0.5)
    return _finish(f"tiny_{n_points}_{width}x{height}_L{num_layers}_K{k_keep}", rng, pts, sizes, poses, fx, width, height,
                   num_layers, k_keep, train, seed, channels=channels)


def target_gradient(scene: Scene, view: int, seed_offset=1000):
    """Gradient of an L1 loss against a U(0,1) target pyramid is sign(out - target) / numel; before the forward
    output is known the benchmarks use a random +-1/numel pattern of the same shape and distribution."""
    rng = np.random.Generator(np.random.Philox(scene.seed + seed_offset + view))
    P = num_pyramid_pixels(scene.width, scene.height, scene.num_layers)
    numel = scene.channels * P
    g = rng.integers(0, 2, numel).astype(np.float32) * 2 - 1
    return g / np.float32(numel)
