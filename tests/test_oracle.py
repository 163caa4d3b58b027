"""Known-answer tests that pin the CPU oracle (the reference ships no tests or fixtures for this path).

Every expected value is derived by hand from the formulas of the reference: projection and culling
(PointRendererHelper.h:232-253, RenderForward.cu:212-218,302-308), layer selection (RenderForward.cu:342-363), the
layer factor (PointBlending.h:81-149), the blend (RenderForward.cu:882-1021), the backward pass
(RenderBackward.cu:262-439) and Adam (MyAdam.cu:41-88)."""
import math

import numpy as np
import pytest

import oracle
from trips_b200 import scenes

IDENT = [0, 0, 0, 1, 0, 0, 0, 0]


def intr(fx, w, h, cx=None, cy=None):
    k = np.zeros(13, np.float32)
    k[0] = k[1] = fx
    k[2] = w / 2 if cx is None else cx
    k[3] = h / 2 if cy is None else cy
    return k


def render(points, raw_sizes, tex, conf, w=64, h=48, fx=100.0, L=1, K=16, train=True, pose=IDENT, bg=None, **kw):
    points = np.asarray(points, np.float32).reshape(-1, 3)
    n = points.shape[0]
    pos = np.zeros((n, 4), np.float32)
    pos[:, :3] = points
    tex = np.asarray(tex, np.float32).reshape(-1, n)
    c = tex.shape[0]
    bg = np.full(c, 0.25, np.float32) if bg is None else np.asarray(bg, np.float32)
    sa = oracle.SceneArrays(pos, np.asarray(raw_sizes, np.float32), tex, np.asarray(conf, np.float32), bg)
    view = oracle.make_view(w, h, pose, intr(fx, w, h))
    return oracle.forward(sa, view, oracle.make_params(L, K, train, **kw)), sa


def test_reproducible_exp_log_are_accurate(oracle_lib):
    L = oracle_lib.lib()
    xs = np.concatenate([np.linspace(-80, 80, 4001), np.linspace(-1, 1, 2001)]).astype(np.float32)
    got = np.array([L.or_expf(float(x)) for x in xs], np.float32)
    ref = np.exp(xs.astype(np.float64))
    assert np.max(np.abs(got - ref) / ref) < 3e-7
    ys = np.concatenate([np.logspace(-30, 30, 4001), np.linspace(0.5, 2, 3001)]).astype(np.float32)
    got = np.array([L.or_logf(float(y)) for y in ys], np.float32)
    ref = np.log(ys.astype(np.float64))
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-3)) < 3e-7
    # softplus: identity above the threshold of 20 (RenderForward.cu:157), log(1+e^x) below
    assert L.or_softplus(25.0) == 25.0
    assert abs(L.or_softplus(0.0) - math.log(2)) < 1e-7
    assert abs(L.or_softplus(-3.0) - math.log1p(math.exp(-3))) < 1e-7


def test_projection_known_answers(oracle_lib):
    L = oracle_lib.lib()
    view = oracle.make_view(640, 480, IDENT, intr(500, 640, 480))
    u, v, z = (oracle.C.c_float(), oracle.C.c_float(), oracle.C.c_float())
    p = np.array([0, 0, 3], np.float32)
    L.or_project(oracle.C.byref(view), p.ctypes.data, oracle.C.byref(u), oracle.C.byref(v), oracle.C.byref(z))
    assert (u.value, v.value, z.value) == (320.0, 240.0, 3.0)  # optical axis -> principal point
    p = np.array([3, -1.5, 3], np.float32)
    L.or_project(oracle.C.byref(view), p.ctypes.data, oracle.C.byref(u), oracle.C.byref(v), oracle.C.byref(z))
    assert (u.value, v.value) == (320.0 + 500.0, 240.0 - 250.0)  # x/z = 1 -> cx + fx
    # a pose that translates by +2 along z and rotates 90 degrees about z: (x, y) -> (-y, x)
    s = math.sqrt(0.5)
    view = oracle.make_view(640, 480, [0, 0, s, s, 0, 0, 2, 0], intr(500, 640, 480))
    p = np.array([0.5, 0, 0], np.float32)
    L.or_project(oracle.C.byref(view), p.ctypes.data, oracle.C.byref(u), oracle.C.byref(v), oracle.C.byref(z))
    assert abs(z.value - 2.0) < 1e-6 and abs(u.value - 320.0) < 1e-3 and abs(v.value - (240.0 + 125.0)) < 1e-3


def test_culling_rules(oracle_lib):
    # z <= 0 culled; ip in [0, W-1) x [0, H-1); the last row / column and negative coordinates are culled
    w, h, fx = 64, 48, 100.0
    pts = [(0, 0, 1), (0, 0, -1), (0, 0, 0), (0.31, 0, 1), (0.305, 0, 1), (-0.3201, 0, 1), (-0.32, 0, 1), (0, 0.2301, 1), (0, 0.2299, 1)]
    f, _ = render(pts, [-5] * len(pts), np.ones((4, len(pts))), [0.5] * len(pts), w=w, h=h, fx=fx)
    depth, nl, rec = f.points()
    # u = 100 x + 32: 0.31 -> 63 (= W-1, culled), 0.305 -> 62.5 (kept), -0.3201 -> -0.01 (culled), -0.32 -> 0 (kept)
    # v = 100 y + 24: 0.2301 -> 47.01 (>= H-1 = 47, culled), 0.2299 -> 46.99 (kept)
    assert list(depth > 0) == [True, False, False, False, True, False, True, False, True]
    assert f.V == 4
    assert np.all(nl[depth > 0] == 1) and np.all(nl[depth <= 0] == 0)
    assert np.all(depth[depth <= 0] == -1.0)


def test_layer_selection_sweep(oracle_lib):
    # raw size above 20 is passed through by softplus, so size_px = fx * raw / z exactly; fx = 1, raw = 24
    L = 8
    cases = [(24.0, 1), (48.0, 1), (12.0, 2), (8.0, 3), (6.0, 3), (3.0, 4), (1.5, 5), (0.75, 6), (0.375, 7), (0.1, 8), (0.01, 8)]
    for z, expect_layers in cases:
        # 512x512 image so that no coarse layer clips the footprint of the central point
        f, _ = render([(0, 0, z)], [24.0], np.ones((4, 1)), [0.5], w=512, h=512, fx=1.0, L=L)
        depth, nl, rec = f.points()
        assert rec[0, 2] == np.float32(24.0) / np.float32(z)
        assert nl[0] == expect_layers, (z, nl[0])
    # the footprint must stay inside [0, W_l - 1) x [0, H_l - 1): a point near the border stops early
    f, _ = render([(29.0, 0, 1.0)], [24.0], np.ones((4, 1)), [0.5], w=64, h=64, fx=1.0, L=6)  # u = 61, size 24 px -> hi = 5
    # layer sizes 64 32 16 8 4 2: u_l = 61, 30.5, 15.25 -> floor 15 >= W_2 - 1 = 15: stop after layers 0 and 1
    assert f.points()[1][0] == 2
    counts, offsets, frags = f.lists()
    assert counts.sum() == 8 and f.F == 8  # 2 layers x 2x2 footprint


def test_layer_factor_known_answers(oracle_lib):
    L = oracle_lib.lib()
    g = oracle.C.c_float()
    lf = lambda ps, layer, n: (L.or_layer_factor(ps, layer, n, oracle.C.byref(g)), g.value)
    f, d = lf(1.0, 0, 8)
    assert abs(f - 1.0) < 1e-6 and abs(d - 0.27591) < 1e-6  # small point: 0.75 e^(ps-1) + 0.25, slope 0.27591 ps
    f, d = lf(0.5, 0, 8)
    assert abs(f - (0.75 * math.exp(-0.5) + 0.25)) < 1e-6 and abs(d - 0.27591 * 0.5) < 1e-7
    assert lf(4.0, 2, 8) == (1.0, 1.0)  # exactly on a layer
    assert lf(4.0, 0, 8) == (1.0, 0.0)  # finer layers below lo: full weight, no gradient
    f, d = lf(3.0, 2, 8)  # lo = 1, hi = 2, t = (3-2)/2
    assert (f, d) == (0.5, 0.5)
    f, d = lf(3.5, 1, 8)
    assert (f, d) == (0.25, -0.5)
    assert lf(1000.0, 3, 4) == (1.0, 1.0)  # larger than the coarsest layer: clamped
    assert lf(1000.0, 2, 4) == (1.0, 0.0)


def test_blend_closed_forms(oracle_lib):
    bg = np.array([0.25, 0.5, 0.75, 1.0], np.float32)
    tex = np.array([[0.2], [0.4], [0.6], [0.8]], np.float32)
    # one point at u = 10.25, v = 20.5, size 0.5 px: layer factor f = 0.75 e^-0.5 + 0.25
    fx, z = 100.0, 2.0
    x, y = (10.25 - 32) * z / fx, (20.5 - 24) * z / fx
    raw = float(scenes.inverse_softplus(np.array([0.5 * z / fx]))[0])
    fr, _ = render([(x, y, z)], [raw], tex, [0.8], fx=fx, bg=bg)
    ps = fr.points()[2][0, 2]
    f = np.float32(0.75) * np.float32(math.exp(ps - 1)) + np.float32(0.25)
    out = fr.pyramid()[0]
    for (px, py, b) in ((10, 20, 0.75 * 0.5), (11, 20, 0.25 * 0.5), (10, 21, 0.75 * 0.5), (11, 21, 0.25 * 0.5)):
        a = b * 0.8 * f
        # a single fragment: colour a * tex, background weighted with the transmittance BEFORE it, i.e. 1
        np.testing.assert_allclose(out[:, py, px], a * tex[:, 0] + bg, rtol=2e-5)
    assert np.all(out[:, 5, 5] == bg)  # empty list: pure background
    nrec, pid, alpha = fr.records()
    assert nrec.sum() == 4 and fr.Kf == 4

    # two points on the same pixel centre (integer u, v -> bilinear weight 1 there, 0 on the other three pixels)
    xs = [(12 - 32) * zz / fx for zz in (2.0, 3.0)]
    ys = [(7 - 24) * zz / fx for zz in (2.0, 3.0)]
    raws = [float(scenes.inverse_softplus(np.array([1.0 * zz / fx]))[0]) for zz in (2.0, 3.0)]  # 1 px -> factor 1
    tex2 = np.array([[0.2, 0.9], [0.4, 0.7], [0.6, 0.5], [0.8, 0.3]], np.float32)
    fr, _ = render([(xs[1], ys[1], 3.0), (xs[0], ys[0], 2.0)], [raws[1], raws[0]], tex2[:, ::-1], [0.5, 0.25], fx=fx, bg=bg)
    out = fr.pyramid()[0][:, 7, 12]
    ps = fr.points()[2][:, 2]
    a_near = 0.25 * (0.75 * math.exp(ps[1] - 1) + 0.25)  # point 1 is nearer (z = 2)
    a_far = 0.5 * (0.75 * math.exp(ps[0] - 1) + 0.25)
    expect = a_near * tex2[:, 0] + (1 - a_near) * a_far * tex2[:, 1] + bg * (1 - a_near)  # background sees T_{n-1}
    np.testing.assert_allclose(out, expect, rtol=3e-5)
    nrec, pid, alpha = fr.records()
    p = 7 * 64 + 12
    assert list(pid[p, :2]) == [1, 0] and nrec[p] == 2  # nearest first

    # an opaque nearest fragment: the second one is behind T = 0 < 0.001, no record for it, no background
    fr, _ = render([(xs[0], ys[0], 2.0), (xs[1], ys[1], 3.0)], [raws[0], raws[1]], tex2, [1.0, 0.5], fx=fx, bg=bg)
    ps = fr.points()[2][:, 2]
    a0 = 0.75 * math.exp(ps[0] - 1) + 0.25
    assert abs(a0 - 1.0) < 1e-6
    out = fr.pyramid()[0][:, 7, 12]
    nrec, pid, alpha = fr.records()
    if alpha[p, 0] == 1.0:
        np.testing.assert_allclose(out, tex2[:, 0], rtol=1e-6)
        assert nrec[p] == 1 and pid[p, 1] == -1


# ---- the reference's second forward pipeline (non-default flags; RenderForward.cu:1401-3674) ----
def test_strict_two_layer_write(oracle_lib):
    # fx = 1, raw = 24 (softplus passes it through): size_px = 24 / z.  512 x 512 image, central point.
    L = 8
    for z, first, layers in ((24.0, 0, 1), (8.0, 1, 2), (6.0, 2, 1), (4.8, 2, 2), (0.1, 7, 1)):
        # size 1 -> {0}; 3 -> {1, 2}; 4 -> {2}; 5 -> {2, 3}; 240 -> {7} (both ends clamp to the coarsest layer)
        f, _ = render([(0, 0, z)], [24.0], np.ones((4, 1)), [0.5], w=512, h=512, fx=1.0, L=L,
                      render_points_in_all_lower_resolutions=False)
        assert (f.first_layer()[0], f.points()[1][0]) == (first, layers), z
        counts, _, _ = f.lists()
        per_layer = [int(counts[b:b + w * h].sum()) for (w, h, b) in f.layers]
        assert per_layer == [4 if first <= l < first + layers else 0 for l in range(L)]
    # the default pipeline writes the same point to every layer up to the upper one
    f, _ = render([(0, 0, 4.8)], [24.0], np.ones((4, 1)), [0.5], w=512, h=512, fx=1.0, L=L)
    assert (f.first_layer()[0], f.points()[1][0]) == (0, 4)
    # a footprint that leaves the lower layer drops the point from both layers; one that leaves only the upper keeps the lower
    f, _ = render([(29.0, 0, 1.0)], [3.0], np.ones((4, 1)), [0.5], w=64, h=64, fx=1.0, L=6,
                  render_points_in_all_lower_resolutions=False)  # u = 61, size 3: layers 1, 2; u_1 = 30.5 ok, u_2 = 15.25 -> 15 >= 15
    assert (f.first_layer()[0], f.points()[1][0]) == (1, 1)
    # without use_layer_point_size every layer is written and the alpha carries no layer factor
    f, _ = render([(0.25, 0.5, 1.0)], [24.0], np.ones((4, 1)), [0.5], w=512, h=512, fx=1.0, L=4, use_layer_point_size=False)
    assert (f.first_layer()[0], f.points()[1][0]) == (0, 4)
    nrec, pid, alpha = f.records()
    w1, h1, b1 = f.layers[1]
    p = b1 + 128 * w1 + 128  # u = 256.25 / 2 = 128.125, v = 256.5 / 2 = 128.25
    assert nrec[p] == 1 and alpha[p, 0] == np.float32(0.875 * 0.75 * 0.5)


def test_second_pipeline_bilinear_weight_at_integer_coordinates(oracle_lib):
    # u = 12 exactly: the first pipeline gives pixel 12 the weight (1 - 0) and pixel 13 the weight 0; the second evaluates
    # the corner weights from the sub-pixel position and picks the corner by comparison, which gives 0 to both
    fx, z = 100.0, 2.0
    x, y = (12 - 32) * z / fx, (7.5 - 24) * z / fx
    raw = float(scenes.inverse_softplus(np.array([1.0 * z / fx]))[0])
    f1, _ = render([(x, y, z)], [raw], np.ones((4, 1)), [0.8], fx=fx)
    f2, _ = render([(x, y, z)], [raw], np.ones((4, 1)), [0.8], fx=fx, combine_lists=True)
    assert f1.points()[2][0, 0] == 12.0
    a1, a2 = f1.records()[2], f2.records()[2]
    p = 7 * 64 + 12
    assert a1[p, 0] > 0.39 and a1[p + 1, 0] == 0.0
    assert a2[p, 0] == 0.0 and a2[p + 1, 0] == 0.0


def test_combine_lists_known_answer(oracle_lib):
    # Point A (size 0.5 px, layer 0 only) and point B (size 3 px: layers 0, 1, 2) on a 64 x 64 image, 3 layers.  The pixel
    # (10, 20) of layer 0 then holds A and B from its own list and B again from the lists of (5, 10) on layer 1 and
    # (2, 5) on layer 2; all three copies of B carry the alpha of layer 0.
    fx = 100.0
    za, zb = 2.0, 3.0
    A = ((10.25 - 32) * za / fx, (20.5 - 32) * za / fx, za)
    B = ((10.5 - 32) * zb / fx, (20.25 - 32) * zb / fx, zb)
    raws = [float(scenes.inverse_softplus(np.array([0.5 * za / fx]))[0]), float(scenes.inverse_softplus(np.array([3.0 * zb / fx]))[0])]
    tex = np.array([[0.2, 0.9], [0.4, 0.7], [0.6, 0.5], [0.8, 0.3]], np.float32)
    bg = np.array([0.25, 0.5, 0.75, 1.0], np.float32)
    f, _ = render([A, B], raws, tex, [0.8, 0.6], w=64, h=64, fx=fx, L=3, bg=bg, combine_lists=True)
    nrec, pid, alpha = f.records()
    p = 20 * 64 + 10
    assert nrec[p] == 4 and list(pid[p, :4]) == [0, 1, 1, 1]
    ps = f.points()[2][:, 2]
    aA = np.float32(0.75 * 0.5 * 0.8) * (np.float32(0.75) * np.float32(math.exp(ps[0] - 1)) + np.float32(0.25))
    aB = np.float32(0.5 * 0.75 * 0.6)  # layer 0 is below the layers of a 3 px point: factor 1
    np.testing.assert_allclose(alpha[p, :4], [aA, aB, aB, aB], rtol=1e-6)
    T = [1.0, 1 - aA, (1 - aA) * (1 - aB), (1 - aA) * (1 - aB) ** 2]
    expect = T[0] * aA * tex[:, 0] + sum(T[k] * aB * tex[:, 1] for k in (1, 2, 3)) + bg * T[3]
    np.testing.assert_allclose(f.pyramid()[0][:, 20, 10], expect, rtol=3e-5)
    # the coarsest layer has nothing above it: its pixel holds B once
    w2, h2, b2 = f.layers[2]
    q = b2 + 5 * w2 + 2
    assert nrec[q] == 1 and pid[q, 0] == 1
    # a coarse-layer fragment that is more than a pixel away on the fine layer is kept in the list with alpha 0
    q0 = 21 * 64 + 8  # (8, 21) on layer 0 -> (4, 10) on layer 1, where B's footprint (5.25, 10.125) -> pixels 5..6 is absent; (2, 5) on layer 2 holds B
    assert nrec[q0] == 1 and pid[q0, 0] == 1 and alpha[q0, 0] == 0.0
    np.testing.assert_allclose(f.pyramid()[0][:, 21, 8], bg, rtol=1e-6)


def test_saturated_accumulation_known_answer(oracle_lib):
    # three fragments with alphas 0.5, 0.4, 0.3 on one pixel centre (integer coordinates are avoided: the second pipeline
    # gives them the weight 0): u = 12.5, v = 7.5 -> four pixels with bilinear weight 0.25 each; size 1 px -> factor 1
    fx = 100.0
    zs = (2.0, 3.0, 4.0)
    pts = [((12.5 - 32) * z / fx, (7.5 - 24) * z / fx, z) for z in zs]
    raws = [float(scenes.inverse_softplus(np.array([1.0 * z / fx]))[0]) for z in zs]
    tex = np.array([[0.2, 0.9, 0.1], [0.4, 0.7, 0.2], [0.6, 0.5, 0.3], [0.8, 0.3, 0.4]], np.float32)
    bg = np.array([0.25, 0.5, 0.75, 1.0], np.float32)
    conf = [1.0, 1.0, 1.0]
    # bilinear 0.25 would make all alphas 0.25: scale with the texture-free knob we have, the confidence
    conf = [2.0, 1.6, 1.2]  # alphas 0.5, 0.4, 0.3
    f, _ = render(pts, raws, tex, conf, fx=fx, bg=bg, combine_lists=True, saturated_alpha_accumulation=True)
    nrec, pid, alpha = f.records()
    p = 7 * 64 + 12
    ps = f.points()[2][:, 2]
    a = [np.float32(0.25 * c) * (np.float32(0.75) * np.float32(math.exp(s - 1)) + np.float32(0.25)) for c, s in zip(conf, ps)]
    np.testing.assert_allclose(alpha[p, :3], a, rtol=1e-6)
    assert nrec[p] == 3
    # weights: 1 (first), 1 (0.5 + 0.4 < 1), then the crossing fragment: 1 / (alpha + 1e-9); background sees the last weight
    w = [1.0, 1.0, 1.0 / (float(a[2]) + 1e-9)]
    expect = sum(w[k] * a[k] * tex[:, k] for k in range(3)) + bg * w[2]
    np.testing.assert_allclose(f.pyramid()[0][:, 7, 12], expect, rtol=3e-5)
    # backward as written (RenderBackward.cu:227-259): texture gradients weighted by alpha, alpha, and the remainder;
    # the crossing fragment's own alpha gradient is dropped and the sum of its colours is taken from the ones before it
    g = np.zeros(4 * f.P, np.float32)
    gin = np.array([0.3, -0.2, 0.5, 0.1], np.float32)
    for c in range(4):
        g[c * 64 * 48 + p] = gin[c]
    out = f.backward(g)
    rest = 1.0 - float(a[0]) - float(a[1])
    np.testing.assert_allclose(out["texture"][:, 0], float(a[0]) * gin, rtol=1e-5)
    np.testing.assert_allclose(out["texture"][:, 1], float(a[1]) * gin, rtol=1e-5)
    np.testing.assert_allclose(out["texture"][:, 2], rest * gin, rtol=1e-4)
    assert np.all(out["background"] == 0.0)  # nothing is left for the background
    s2 = float(tex[:, 2].sum())
    lf = [float(x) / (0.25 * c) for x, c in zip(a, conf)]
    # (that colour sum is not weighted by the incoming gradient: the three other pixels of the footprint, whose incoming
    # gradient is zero, subtract it as well)
    expect_conf = [0.25 * lf[0] * (float(tex[:, 0] @ gin) - 4 * s2), 0.25 * lf[1] * (float(tex[:, 1] @ gin) - 4 * s2), 0.0]
    np.testing.assert_allclose(out["confidence"], expect_conf, rtol=1e-4, atol=1e-7)
    # on the first pipeline the forward pass ignores the flag (its branch is compiled out, RenderForward.cu:908-935)
    f1, _ = render(pts, raws, tex, conf, fx=fx, bg=bg, saturated_alpha_accumulation=True)
    f0, _ = render(pts, raws, tex, conf, fx=fx, bg=bg)
    assert np.array_equal(f1.pyramid_flat(), f0.pyramid_flat())


def test_top_k_keeps_the_nearest_with_index_ties(oracle_lib):
    # 40 points on one pixel centre, several at identical depth: kept = 16 smallest (depth, id)
    rng = np.random.default_rng(0)
    n, fx = 40, 100.0
    z = rng.choice([2.0, 2.5, 3.0, 3.5], n).astype(np.float32)
    pts = [((9 - 32) * zz / fx, (9 - 24) * zz / fx, zz) for zz in z]
    # integer pixel positions only when the float arithmetic is exact; use the list of pixel 9,9 whatever lands there
    fr, _ = render(pts, [-6.0] * n, rng.random((4, n)), rng.random(n), fx=fx)
    counts, offsets, frags = fr.lists()
    depth, nl, rec = fr.points()
    nrec, pid, alpha = fr.records()
    for p in np.nonzero(counts > 16)[0]:
        lst = frags[offsets[p]:offsets[p] + counts[p]]
        assert np.all(lst[:-1] < lst[1:])  # stored sorted by the 64-bit key
        ids = (lst & 0xffffffff).astype(np.int64)
        order = sorted(range(len(ids)), key=lambda k: (depth[ids[k]].view(np.uint32), ids[k]))
        assert [ids[k] for k in order] == list(ids)
        assert list(pid[p, :16]) == list(ids[:16]) or nrec[p] < 16
    assert (counts > 16).any()


def test_adam_matches_scalar_loop(oracle_lib):
    rng = np.random.default_rng(1)
    n = 257
    w = rng.normal(size=n).astype(np.float32)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    s = np.zeros(n, np.int64)
    w2, m2, v2, s2 = w.astype(np.float64), m.astype(np.float64), v.astype(np.float64), s.copy()
    for it in range(3):
        g = rng.normal(size=n).astype(np.float32)
        g[rng.random(n) < 0.3] = 0
        oracle.adam(w, g.copy(), m, v, s, lr=1e-2, rel_decay=0.1, abs_decay=0.01, clip=1.5)
        for i in range(n):
            if g[i] == 0:
                continue  # unseen element: nothing changes, not even the moments (MyAdam.cu:57-61)
            m2[i] = 0.9 * m2[i] + 0.1 * g[i]
            v2[i] = 0.999 * v2[i] + 0.001 * g[i] * g[i]
            s2[i] += 1
            lr = 1e-2 * math.sqrt(1 - 0.999 ** s2[i]) / (1 - 0.9 ** s2[i])
            eff = lr / (math.sqrt(v2[i]) + 1e-8)
            nw = (1 - 0.1 * lr) * w2[i] - math.copysign(0.01 * lr, w2[i]) - eff * m2[i]
            w2[i] = min(max(nw, -1.5), 1.5)
    assert np.array_equal(s, s2)
    np.testing.assert_allclose(w, w2, rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(m, m2, rtol=1e-5, atol=1e-7)


def _loss(frame, g):
    return float(np.dot(frame.pyramid_flat().astype(np.float64), g.astype(np.float64)))


def test_backward_against_finite_differences(oracle_lib):
    """Descriptors and background enter linearly (exact differences); confidence and position are checked with the
    consistent background weight (bg_uses_Tn) on a one-layer render, where the reference's approximations
    (background weighted with the transmittance before the last kept fragment; position gradients of coarse layers not
    scaled by 2^-l; the small-point factor's derivative 0.27591 ps) do not apply."""
    s = scenes.tiny(n_points=300, width=32, height=24, num_layers=1, n_views=1, seed=5, fx=40.0, size_range=(0.01, 0.05))
    s.confidence[:] = np.clip(s.confidence * 0.6 + 0.1, 0, 1)
    g = np.random.default_rng(3).normal(size=s.channels * 32 * 24).astype(np.float32)

    def run(scene, **kw):
        sa = oracle.SceneArrays.from_scene(scene)
        v = oracle.make_view(scene.width, scene.height, scene.poses[0], scene.intrinsics[0])
        return oracle.forward(sa, v, oracle.make_params(1, 16, True, bg_uses_Tn=True, **kw))

    f0 = run(s)
    grads = f0.backward(g)
    base = _loss(f0, g)
    rng = np.random.default_rng(4)
    depth = f0.points()[0]
    vis = np.nonzero(depth > 0)[0]
    # texture: linear
    for i in rng.choice(vis, 6, replace=False):
        for c in range(2):
            s2 = scenes.tiny(n_points=300, width=32, height=24, num_layers=1, n_views=1, seed=5, fx=40.0, size_range=(0.01, 0.05))
            s2.confidence[:] = s.confidence
            s2.texture[c, i] += 0.5
            fd = (_loss(run(s2), g) - base) / 0.5
            assert abs(fd - grads["texture"][c, i]) <= 2e-3 * max(1.0, abs(fd)), (i, c)
    # background: linear
    s2 = scenes.tiny(n_points=300, width=32, height=24, num_layers=1, n_views=1, seed=5, fx=40.0, size_range=(0.01, 0.05))
    s2.confidence[:] = s.confidence
    s2.background[1] += 0.5
    fd = (_loss(run(s2), g) - base) / 0.5
    assert abs(fd - grads["background"][1]) <= 2e-3 * max(1.0, abs(fd))
    # confidence: smooth (polynomial), central differences
    errs = []
    for i in rng.choice(vis, 8, replace=False):
        lo, hi = [scenes.tiny(n_points=300, width=32, height=24, num_layers=1, n_views=1, seed=5, fx=40.0, size_range=(0.01, 0.05)) for _ in range(2)]
        lo.confidence[:] = s.confidence
        hi.confidence[:] = s.confidence
        lo.confidence[i] -= 0.01
        hi.confidence[i] += 0.01
        fd = (_loss(run(hi), g) - _loss(run(lo), g)) / 0.02
        errs.append(abs(fd - grads["confidence"][i]) / max(abs(fd), 1e-3))
    assert np.median(errs) < 2e-2, errs
    # position: the bilinear weights are piecewise linear in (u, v); central differences away from pixel borders
    errs = []
    for i in rng.choice(vis, 8, replace=False):
        for ax in range(2):
            lo, hi = [scenes.tiny(n_points=300, width=32, height=24, num_layers=1, n_views=1, seed=5, fx=40.0, size_range=(0.01, 0.05)) for _ in range(2)]
            lo.confidence[:] = s.confidence
            hi.confidence[:] = s.confidence
            lo.position[i, ax] -= 2e-4
            hi.position[i, ax] += 2e-4
            fd = (_loss(run(hi), g) - _loss(run(lo), g)) / 4e-4
            errs.append(abs(fd - grads["position"][i, ax]) / max(abs(fd), abs(grads["position"][i, ax]), 1e-2))
    assert np.median(errs) < 5e-2, errs


# ---- lens distortion (the 8-coefficient model of saiga's distortNormalizedPoint, restated) ----
def _one_point(x, y, z, intr_extra, fx=100.0, w=64, h=48, **kw):
    pos = np.array([[x, y, z, 0.0]], np.float32)
    sa = oracle.SceneArrays(pos, np.array([-6.0], np.float32), np.ones((4, 1), np.float32), np.array([0.5], np.float32),
                            np.full(4, 0.25, np.float32))
    k = intr(fx, w, h)
    k[5:] = intr_extra
    f = oracle.forward(sa, oracle.make_view(w, h, IDENT, k), oracle.make_params(1, 16, True, **kw))
    return f


def test_distortion_known_answers(oracle_lib):
    fx, z = 100.0, 2.0
    x, y = 0.2, -0.1  # normalised coordinates (x / z, y / z) = (0.1, -0.05)
    nx, ny = 0.1, -0.05
    r2 = nx * nx + ny * ny
    # coefficients are ignored unless the distortion flag is set
    f = _one_point(x, y, z, [0.5, 0, 0, 0, 0, 0, 0, 0])
    assert abs(f.points()[2][0, 0] - (32 + fx * nx)) < 1e-4
    # k1 only: radial factor 1 + k1 r^2
    f = _one_point(x, y, z, [0.5, 0, 0, 0, 0, 0, 0, 0], distortion=True)
    u, v = f.points()[2][0, :2]
    assert abs(u - (32 + fx * nx * (1 + 0.5 * r2))) < 1e-4 and abs(v - (24 + fx * ny * (1 + 0.5 * r2))) < 1e-4
    # the rational form: (1 + k1 r2 + k2 r4 + k3 r6) / (1 + k4 r2 + k5 r4 + k6 r6)
    ks = [0.3, -0.2, 0.1, 0.05, -0.03, 0.02]
    f = _one_point(x, y, z, ks + [0, 0], distortion=True)
    rad = (1 + ks[0] * r2 + ks[1] * r2 ** 2 + ks[2] * r2 ** 3) / (1 + ks[3] * r2 + ks[4] * r2 ** 2 + ks[5] * r2 ** 3)
    u, v = f.points()[2][0, :2]
    assert abs(u - (32 + fx * nx * rad)) < 1e-4 and abs(v - (24 + fx * ny * rad)) < 1e-4
    # tangential terms: x' = x + 2 p1 x y + p2 (r2 + 2 x^2), y' = y + p1 (r2 + 2 y^2) + 2 p2 x y
    p1, p2 = 0.01, -0.02
    f = _one_point(x, y, z, [0, 0, 0, 0, 0, 0, p1, p2], distortion=True)
    u, v = f.points()[2][0, :2]
    assert abs(u - (32 + fx * (nx + 2 * p1 * nx * ny + p2 * (r2 + 2 * nx * nx)))) < 1e-4
    assert abs(v - (24 + fx * (ny + p1 * (r2 + 2 * ny * ny) + 2 * p2 * nx * ny))) < 1e-4
    # outside the cut-off radius the point is culled, inside it is drawn
    assert _one_point(x, y, z, [0] * 8, distortion=True, dist_cutoff=0.1).V == 0  # r = 0.1118 > 0.1
    assert _one_point(x, y, z, [0] * 8, distortion=True, dist_cutoff=0.12).V == 1


def test_distortion_backward_against_finite_differences(oracle_lib):
    """Gradients with respect to the eight distortion coefficients, the pinhole coefficients and the positions through a
    distorted projection (one layer, consistent background weight, as in the test above)."""
    s = scenes.tiny(n_points=300, width=32, height=24, num_layers=1, n_views=1, seed=6, fx=40.0, size_range=(0.01, 0.05))
    s.confidence[:] = np.clip(s.confidence * 0.6 + 0.1, 0, 1)
    coeff = np.array([-0.12, 0.05, -0.01, 0.03, -0.02, 0.004, 2e-3, -3e-3], np.float32)
    g = np.random.default_rng(3).normal(size=s.channels * 32 * 24).astype(np.float32)

    def run(intr13, position=None):
        sa = oracle.SceneArrays.from_scene(s) if position is None else oracle.SceneArrays(position, s.point_size, s.texture, s.confidence, s.background)
        v = oracle.make_view(s.width, s.height, s.poses[0], intr13)
        return oracle.forward(sa, v, oracle.make_params(1, 16, True, bg_uses_Tn=True, distortion=True))

    k0 = s.intrinsics[0].copy()
    k0[5:] = coeff
    f0 = run(k0)
    grads = f0.backward(g)
    assert grads["intrinsics"].shape == (13,) and np.all(grads["intrinsics"][5:] != 0)
    # the loss is piecewise smooth in every camera coefficient (a sum over all points): central differences
    steps = [1e-2, 1e-2, 1e-3, 1e-3, 1e-4] + [2e-3] * 6 + [2e-4] * 2
    for k in range(13):
        lo, hi = k0.copy(), k0.copy()
        lo[k] -= steps[k]
        hi[k] += steps[k]
        fd = (_loss(run(hi), g) - _loss(run(lo), g)) / (2 * steps[k])
        ref = grads["intrinsics"][k]
        assert abs(fd - ref) <= 0.08 * max(abs(fd), abs(ref)) + 1e-3 * np.abs(grads["intrinsics"]).max(), (k, fd, ref)
    # positions through J_p_dis
    rng = np.random.default_rng(4)
    vis = np.nonzero(f0.points()[0] > 0)[0]
    errs = []
    for i in rng.choice(vis, 8, replace=False):
        for ax in range(2):
            lo, hi = s.position.copy(), s.position.copy()
            lo[i, ax] -= 2e-4
            hi[i, ax] += 2e-4
            fd = (_loss(run(k0, hi), g) - _loss(run(k0, lo), g)) / 4e-4
            errs.append(abs(fd - grads["position"][i, ax]) / max(abs(fd), abs(grads["position"][i, ax]), 1e-2))
    assert np.median(errs) < 5e-2, errs
    # and the distortion changes the picture at all
    k1 = s.intrinsics[0].copy()
    assert not np.array_equal(run(k1).pyramid_flat(), f0.pyramid_flat())


GOLDEN = __import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "tiny_scene.npz")


def test_oracle_reproduces_frozen_outputs(oracle_lib):
    """Outputs of a tiny seeded scene frozen in tests/golden/tiny_scene.npz (made by tests/golden/make_golden.py):
    guards the oracle against silent changes.  Integer results must match exactly, floats to the last bit."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(GOLDEN), "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    gold = np.load(GOLDEN)
    now = mg.compute()
    assert set(gold.files) == set(now.keys())
    for k in gold.files:
        a, b = gold[k], now[k]
        assert a.shape == b.shape and a.dtype == b.dtype, k
        if a.dtype.kind == "f" and k.startswith("grad_"):
            np.testing.assert_allclose(b, a, rtol=1e-12, atol=0, err_msg=k)  # double accumulators, OpenMP order
        else:
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), k


def test_reproducible_exp_log_against_libm_sweep(oracle_lib):
    """tm_expf / tm_logf (shared by the oracle and the CUDA library, and therefore not checked by comparing the two)
    against double-precision libm over every 16th float of their domains: within 2 units of the last place."""
    e_exp, e_log = oracle_lib.math_sweep(16)
    assert e_exp <= 2.0, e_exp
    assert e_log <= 2.0, e_log
