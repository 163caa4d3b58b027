// CPU oracle for the TRIPS trilinear point-splatting hot path.  TEST INFRASTRUCTURE ONLY -- see trips_oracle.h.
// PARITY UNPINNED: no reference fixture exists for this path; pinned by known-answer and finite-difference tests.
//
// Build: g++ -O3 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/Makefile).  -ffp-contract=off is required:
// together with nvcc -fmad=false it makes every fp32 expression below round exactly like the CUDA kernels.
#include "trips_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../trips_b200/csrc/trips_math.h"  // reproducible exp / log shared with the kernels

namespace
{
constexpr int kMaxLayers   = 8;   // RenderConstants.h:38
constexpr int kMaxKeep     = 16;  // PointRenderer.h:178
constexpr float kAlphaCut  = 0.001f;  // ALPHA_DEST_CUTOFF, RenderForward.cu:907

struct Pose
{
    float qx, qy, qz, qw, tx, ty, tz;
    float R[9];  // row-major rotation matrix of the quaternion
};

// DeviceRenderParams::Pose casts the stored SE3d to float (RenderConstants.h:85-88).
Pose make_pose(const double* p)
{
    Pose o;
    o.qx = (float)p[0];
    o.qy = (float)p[1];
    o.qz = (float)p[2];
    o.qw = (float)p[3];
    o.tx = (float)p[4];
    o.ty = (float)p[5];
    o.tz = (float)p[6];
    // Eigen::Quaternion::toRotationMatrix
    float tx = 2.f * o.qx, ty = 2.f * o.qy, tz = 2.f * o.qz;
    float twx = tx * o.qw, twy = ty * o.qw, twz = tz * o.qw;
    float txx = tx * o.qx, txy = ty * o.qx, txz = tz * o.qx;
    float tyy = ty * o.qy, tyz = tz * o.qy, tzz = tz * o.qz;
    o.R[0] = 1.f - (tyy + tzz);
    o.R[1] = txy - twz;
    o.R[2] = txz + twy;
    o.R[3] = txy + twz;
    o.R[4] = 1.f - (txx + tzz);
    o.R[5] = tyz - twx;
    o.R[6] = txz - twy;
    o.R[7] = tyz + twx;
    o.R[8] = 1.f - (txx + tyy);
    return o;
}

// Sophus SE3f * point = quaternion rotation (Eigen _transformVector) + translation.
inline void transform_point(const Pose& V, const float* p, float* out)
{
    float ux = V.qy * p[2] - V.qz * p[1];
    float uy = V.qz * p[0] - V.qx * p[2];
    float uz = V.qx * p[1] - V.qy * p[0];
    ux += ux;
    uy += uy;
    uz += uz;
    float cx = V.qy * uz - V.qz * uy;
    float cy = V.qz * ux - V.qx * uz;
    float cz = V.qx * uy - V.qy * ux;
    out[0]   = ((p[0] + V.qw * ux) + cx) + V.tx;
    out[1]   = ((p[1] + V.qw * uy) + cy) + V.ty;
    out[2]   = ((p[2] + V.qw * uz) + cz) + V.tz;
}

struct Cam
{
    Pose V;
    float fx, fy, cx, cy, s;         // K
    float cfx, cfy, ccx, ccy, cs;    // crop transform
    float r00, r01, r10, r11;        // crop rotation
    float cenx, ceny;                // (w/2, h/2) with integer division, RenderForward.cu:303
    int w, h;
    float k1, k2, k3, k4, k5, k6, p1, p2;  // distortion coefficients
    bool dist = false;                     // apply them (and the cut-off radius)
    float cut2 = 0.f;                      // dist_cutoff^2
};

// saiga's distortNormalizedPoint restated (see OrParams.distortion): rational radial factor + tangential terms.
// J (optional): d(xd, yd) / d(x, y) row-major; Jk (optional): d(xd, yd) / d(k1 k2 k3 k4 k5 k6 p1 p2), two rows of 8.
inline void distort(const Cam& c, float x, float y, float& xd, float& yd, float* J, float* Jk)
{
    const float x2 = x * x, y2 = y * y;
    const float r2 = x2 + y2, xy2 = 2.f * x * y;
    const float r4 = r2 * r2, r6 = r4 * r2;
    const float A  = ((1.f + c.k1 * r2) + c.k2 * r4) + c.k3 * r6;
    const float B  = ((1.f + c.k4 * r2) + c.k5 * r4) + c.k6 * r6;
    const float iB = 1.f / B;
    const float radial = A * iB;
    const float tx = c.p1 * xy2 + c.p2 * (r2 + 2.f * x2);
    const float ty = c.p1 * (r2 + 2.f * y2) + c.p2 * xy2;
    xd = x * radial + tx;
    yd = y * radial + ty;
    if (J)
    {
        const float dA = (c.k1 + 2.f * c.k2 * r2) + 3.f * c.k3 * r4;
        const float dB = (c.k4 + 2.f * c.k5 * r2) + 3.f * c.k6 * r4;
        const float dr = (dA * B - A * dB) * iB * iB;  // d radial / d r2
        J[0] = radial + x * dr * (2.f * x) + (2.f * c.p1 * y + 6.f * c.p2 * x);
        J[1] = x * dr * (2.f * y) + (2.f * c.p1 * x + 2.f * c.p2 * y);
        J[2] = y * dr * (2.f * x) + (2.f * c.p1 * x + 2.f * c.p2 * y);
        J[3] = radial + y * dr * (2.f * y) + (6.f * c.p1 * y + 2.f * c.p2 * x);
    }
    if (Jk)
    {
        const float AiB2 = A * iB * iB;
        Jk[0] = x * r2 * iB, Jk[1] = x * r4 * iB, Jk[2] = x * r6 * iB;
        Jk[3] = -x * AiB2 * r2, Jk[4] = -x * AiB2 * r4, Jk[5] = -x * AiB2 * r6;
        Jk[6] = xy2, Jk[7] = r2 + 2.f * x2;
        Jk[8] = y * r2 * iB, Jk[9] = y * r4 * iB, Jk[10] = y * r6 * iB;
        Jk[11] = -y * AiB2 * r2, Jk[12] = -y * AiB2 * r4, Jk[13] = -y * AiB2 * r6;
        Jk[14] = r2 + 2.f * y2, Jk[15] = xy2;
    }
}

Cam make_cam(const OrView* v, const OrParams* pr = nullptr)
{
    Cam c;
    c.V   = make_pose(v->pose);
    c.fx  = v->intrinsics[0];
    c.fy  = v->intrinsics[1];
    c.cx  = v->intrinsics[2];
    c.cy  = v->intrinsics[3];
    c.s   = v->intrinsics[4];
    c.cfx = v->crop_transform[0];
    c.cfy = v->crop_transform[1];
    c.ccx = v->crop_transform[2];
    c.ccy = v->crop_transform[3];
    c.cs  = v->crop_transform[4];
    c.r00 = v->crop_rotation[0];
    c.r01 = v->crop_rotation[1];
    c.r10 = v->crop_rotation[2];
    c.r11 = v->crop_rotation[3];
    c.w   = v->w;
    c.h   = v->h;
    c.cenx = (float)(v->w / 2);
    c.ceny = (float)(v->h / 2);
    c.k1 = v->intrinsics[5], c.k2 = v->intrinsics[6], c.k3 = v->intrinsics[7], c.k4 = v->intrinsics[8];
    c.k5 = v->intrinsics[9], c.k6 = v->intrinsics[10], c.p1 = v->intrinsics[11], c.p2 = v->intrinsics[12];
    c.dist = pr && pr->distortion;
    c.cut2 = pr ? pr->dist_cutoff * pr->dist_cutoff : 0.f;
    return c;
}

// ProjectPointPinholeWoNormal (PointRendererHelper.h:232-253) with zero distortion, followed by the crop
// transform and crop rotation of CountAndCollectTiled (RenderForward.cu:302-303, 69-76).
inline void project(const Cam& c, const float* p, float& u, float& v, float& z)
{
    float pv[3];
    transform_point(c.V, p, pv);
    z        = std::fmax(pv[2], 0.f);
    float iz = 1.f / pv[2];
    float nx = pv[0] * iz;
    float ny = pv[1] * iz;
    if (c.dist)
    {
        // outside the cut-off radius the routine returns (100000, 100000) and the caller sets z = 0
        if (nx * nx + ny * ny > c.cut2) z = 0.f;
        float xd, yd;
        distort(c, nx, ny, xd, yd, nullptr, nullptr);
        nx = xd, ny = yd;
    }
    // K.normalizedToImage
    float ix = (c.fx * nx + c.s * ny) + c.cx;
    float iy = c.fy * ny + c.cy;
    // crop_transform.normalizedToImage
    float jx = (c.cfx * ix + c.cs * iy) + c.ccx;
    float jy = c.cfy * iy + c.ccy;
    // rotateCropAroundCenter
    float dx = jx - c.cenx;
    float dy = jy - c.ceny;
    float rx = c.r00 * dx + c.r01 * dy;
    float ry = c.r10 * dx + c.r11 * dy;
    u        = rx + c.cenx;
    v        = ry + c.ceny;
}

// compute_point_size_fac (PointBlending.h:81-149).  floor/ceil of log2 are taken exactly from the float's bits.
inline float layer_factor(float ps, int layer, int L, float* grad)
{
    int lo = 0, hi = 0;
    if (ps > 1.f)
    {
        lo = std::min(std::max(0, tm_floor_log2(ps)), L - 1);
        hi = std::min(std::max(0, tm_ceil_log2(ps)), L - 1);
    }
    if (layer < lo)
    {
        if (grad) *grad = 0.f;
        return 1.f;
    }
    float f = 1.f;
    if (hi == 0)
    {
        f = 0.75f * tm_expf(ps - 1.f) + 0.25f;
        if (grad) *grad = 0.27591f * ps;
    }
    else if (lo == hi)
    {
        if (grad) *grad = 1.f;
    }
    else
    {
        float l_l = (float)(1 << lo);
        float l_h = (float)(1 << hi);
        f         = (ps - l_l) / (l_h - l_l);
        if (layer == lo) f = 1.f - f;
        if (grad)
        {
            float J = 1.f / (l_h - l_l);
            if (layer == lo) J = -J;
            *grad = J;
        }
    }
    return f;
}
}  // namespace

struct OrFrame
{
    int N = 0, C = 0, L = 0, K = 0, train = 0;
    int W[kMaxLayers], H[kMaxLayers];
    int64_t base[kMaxLayers + 1];
    int64_t P = 0, F = 0, Kf = 0, V = 0;
    std::vector<float> depth;
    std::vector<int32_t> nlayers;  // layers the point is written to ...
    std::vector<int32_t> first;    // ... starting with this one
    std::vector<float> rec;  // [N,4]
    std::vector<int32_t> counts;
    std::vector<int64_t> offsets;
    std::vector<uint64_t> frags;
    std::vector<float> pyramid;
    std::vector<int32_t> nrec;
    std::vector<int32_t> rec_pid;
    std::vector<float> rec_alpha;
};

extern "C" {

int or_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// PrepareConfidence (NeuralTexture.h:40-43): out = sigmoid(scale * raw), with the library's reproducible exponential
void or_sigmoid(const float* raw, float scale, float* out, long long n)
{
    for (long long i = 0; i < n; ++i) out[i] = tm_sigmoid(scale * raw[i]);
}

void or_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

float or_layer_factor(float ps, int layer, int num_layers, float* grad) { return layer_factor(ps, layer, num_layers, grad); }
float or_softplus(float x) { return tm_softplus(x); }
float or_expf(float x) { return tm_expf(x); }
float or_logf(float x) { return tm_logf(x); }
void or_project(const OrView* view, const float* p3, float* u, float* v, float* z)
{
    Cam c = make_cam(view);  // (no parameters: zero distortion)
    project(c, p3, *u, *v, *z);
}

OrFrame* or_forward(const OrScene* sc, const OrView* view, const OrParams* pr)
{
    OrFrame* f = new OrFrame();
    const int N = sc->n_points, C = sc->channels, L = pr->num_layers, K = pr->k_keep;
    if (L < 1 || L > kMaxLayers || K < 1 || K > kMaxKeep)
    {
        delete f;
        return nullptr;
    }
    f->N = N;
    f->C = C;
    f->L = L;
    f->K = K;
    f->train = pr->train;
    // layer sizes: ceil halving (PointRenderer.cu:385-389)
    {
        int w = view->w, h = view->h;
        int64_t b = 0;
        for (int l = 0; l < L; ++l)
        {
            f->W[l]    = w;
            f->H[l]    = h;
            f->base[l] = b;
            b += (int64_t)w * h;
            h = (int)std::ceil((float)h / 2.f);
            w = (int)std::ceil((float)w / 2.f);
        }
        f->base[L] = b;
        f->P       = b;
    }
    const Cam cam = make_cam(view, pr);
    f->depth.assign(N, -1.f);
    f->nlayers.assign(N, 0);
    f->first.assign(N, 0);
    // The reference has two forward pipelines (PointRenderer.cu:730-731).  The second one (CountTiled,
    // CollectTiled2[Pointsize], FastSortAndBlendWPrep2WarpSharedWork: RenderForward.cu:1401-3674) runs when one of
    // these three flags differs from its default; it differs from the first in the layers a point is written to, in
    // the radius test (float instead of int), in the way the bilinear weight is evaluated, in combine_lists and in the
    // saturated accumulation.
    const bool second = !(pr->use_layer_point_size && pr->render_points_in_all_lower_resolutions && !pr->combine_lists);
    const bool strict = pr->use_layer_point_size && !pr->render_points_in_all_lower_resolutions;
    f->rec.assign((size_t)N * 4, 0.f);
    f->counts.assign(f->P, 0);

    const float fxc = cam.fx * cam.cfx;
    int32_t* counts = f->counts.data();

    // ---- A1: project, cull, select layers, count (CountAndCollectTiled, RenderForward.cu:168-366) ----
    int64_t visible = 0;
#pragma omp parallel for schedule(static) reduction(+ : visible)
    for (int i = 0; i < N; ++i)
    {
        int tex = sc->index ? sc->index[i] : i;
        if (pr->viewer_only)
        {
            if (sc->confidence[tex] < pr->stability_cutoff_value) continue;  // discard_point_for_confidence, RenderForward.cu:122-130
        }
        // the drop-out mask applies in training whether or not viewer_only is set (second test at RenderForward.cu:236-240)
        if (pr->train && sc->dropout && sc->dropout[i] == 1.f) continue;
        float s = tm_softplus(sc->point_size[i]);
        float u, v, z;
        project(cam, sc->position + (size_t)i * 4, u, v, z);
        float radius_px = fxc * sc->position[(size_t)i * 4 + 3] / z;
        float ps        = fxc * s / z;
        auto dropped    = [&](float rad) {
            // first pipeline: the test takes an int (RenderForward.cu:212-218); second: the float (RenderForward.cu:1527-1531)
            return pr->drop_out_points_by_radius && (second ? rad : (float)(int)rad) < pr->drop_out_radius_threshold;
        };
        if (z <= 0.f || u < 0.f || u >= (float)(f->W[0] - 1) || v < 0.f || v >= (float)(f->H[0] - 1)) continue;
        if (dropped(radius_px)) continue;
        f->depth[i]               = z;
        f->rec[(size_t)i * 4 + 0] = u;
        f->rec[(size_t)i * 4 + 1] = v;
        f->rec[(size_t)i * 4 + 2] = ps;
        f->rec[(size_t)i * 4 + 3] = tm_bits_to_float((uint32_t)tex);
        int lo = 0, hi = 0;
        if (!pr->use_layer_point_size)
            hi = L - 1;  // every layer (RenderForward.cu:1611-1631)
        else if (ps > 1.f)
        {
            lo = std::min(tm_floor_log2(ps), L - 1);
            hi = std::min(tm_ceil_log2(ps), L - 1);
        }
        // layers first .. last, stopping where the 2x2 footprint leaves the layer; the strict write starts at the layer
        // below log2(size) and has at most two layers (RenderForward.cu:1555-1583, 2291-2393)
        const int first = strict ? lo : 0;
        const float sc0 = 1.f / (float)(1 << first);  // powf(0.5f, lo): exact
        int layer = first;
        float x = u * sc0, y = v * sc0, rad = radius_px * sc0;
        for (; layer < hi + 1; ++layer, x *= 0.5f, y *= 0.5f, rad *= 0.5f)
        {
            int px = (int)std::floor(x), py = (int)std::floor(y);
            if (px < 0 || px >= f->W[layer] - 1 || py < 0 || py >= f->H[layer] - 1 || dropped(rad)) break;
            for (int k = 0; k < 4; ++k)
            {
                int64_t pix = f->base[layer] + (int64_t)(py + k / 2) * f->W[layer] + (px + k % 2);
#pragma omp atomic
                counts[pix]++;
            }
        }
        f->first[i]   = first;
        f->nlayers[i] = layer - first;
        visible++;
    }
    f->V = visible;

    // ---- A2: exclusive scan over the whole pyramid (RenderForward.cu:1155-1232) ----
    f->offsets.resize(f->P);
    {
        int64_t run = 0;
        for (int64_t p = 0; p < f->P; ++p)
        {
            f->offsets[p] = run;
            run += counts[p];
        }
        f->F = run;
    }
    f->frags.resize(f->F);
    // ---- collect (SplattingPass, RenderForward.cu:368-436) ----
    {
        std::vector<int32_t> cursor(f->P, 0);
        int32_t* cur = cursor.data();
#pragma omp parallel for schedule(static)
        for (int i = 0; i < N; ++i)
        {
            float z = f->depth[i];
            if (!(z > 0.f)) continue;
            uint64_t key = ((uint64_t)tm_float_to_bits(z) << 32) | (uint32_t)i;
            const float sc0 = 1.f / (float)(1 << f->first[i]);
            float x = f->rec[(size_t)i * 4 + 0] * sc0, y = f->rec[(size_t)i * 4 + 1] * sc0;
            for (int layer = f->first[i]; layer < f->first[i] + f->nlayers[i]; ++layer, x *= 0.5f, y *= 0.5f)
            {
                int px = (int)std::floor(x), py = (int)std::floor(y);
                for (int k = 0; k < 4; ++k)
                {
                    int64_t pix = f->base[layer] + (int64_t)(py + k / 2) * f->W[layer] + (px + k % 2);
                    int32_t slot;
#pragma omp atomic capture
                    slot = cur[pix]++;
                    f->frags[f->offsets[pix] + slot] = key;
                }
            }
        }
    }
    // list order is unspecified in the reference (slot = atomicAdd result); the oracle stores every list
    // sorted by the 64-bit key (depth bits, then point id).
#pragma omp parallel for schedule(dynamic, 4096)
    for (int64_t p = 0; p < f->P; ++p)
    {
        if (counts[p] > 1) std::sort(f->frags.begin() + f->offsets[p], f->frags.begin() + f->offsets[p] + counts[p]);
    }

    // ---- A3: top-K + front-to-back blend (FastSortFusedNew, RenderForward.cu:474-1059) ----
    f->pyramid.assign((size_t)C * f->P, 0.f);
    f->nrec.assign(f->P, 0);
    if (pr->train)
    {
        f->rec_pid.assign((size_t)f->P * kMaxKeep, -1);
        f->rec_alpha.assign((size_t)f->P * kMaxKeep, -1.f);
    }
    int64_t kept = 0;
#pragma omp parallel for schedule(dynamic, 1024) reduction(+ : kept)
    for (int64_t p = 0; p < f->P; ++p)
    {
        int layer = 0;
        while (p >= f->base[layer + 1]) ++layer;
        int64_t t = p - f->base[layer];
        int gx = (int)(t % f->W[layer]), gy = (int)(t / f->W[layer]);
        // the nearest K fragments of the pixel's list; with combine_lists also of the lists of the pixels above it on the
        // coarser layers (RenderForward.cu:3232-3242; a point written to several layers then appears several times)
        uint64_t keys[kMaxKeep];
        int n = std::min(counts[p], K);
        kept += n;  // the statistic counts the pixel's own list, also with combine_lists
        for (int j = 0; j < n; ++j) keys[j] = f->frags[f->offsets[p] + j];
        if (pr->combine_lists)
        {
            std::vector<uint64_t> cand(f->frags.begin() + f->offsets[p], f->frags.begin() + f->offsets[p] + counts[p]);
            int x = gx / 2, y = gy / 2;
            for (int l2 = layer + 1; l2 < L; ++l2, x /= 2, y /= 2)
            {
                int64_t q = f->base[l2] + (int64_t)y * f->W[l2] + x;
                cand.insert(cand.end(), f->frags.begin() + f->offsets[q], f->frags.begin() + f->offsets[q] + counts[q]);
            }
            std::sort(cand.begin(), cand.end());
            n = (int)std::min<size_t>(cand.size(), (size_t)K);
            for (int j = 0; j < n; ++j) keys[j] = cand[j];
        }
        float alpha[kMaxKeep], T[kMaxKeep];
        float contrib[kMaxKeep][16];
        int tex[kMaxKeep], pid[kMaxKeep];
        const float fac = 1.f / (float)(1 << layer);
        for (int j = 0; j < n; ++j)
        {
            uint64_t key = keys[j];
            int i        = (int)(uint32_t)(key & 0xffffffffu);
            pid[j]       = i;
            float u = f->rec[(size_t)i * 4 + 0], v = f->rec[(size_t)i * 4 + 1], ps = f->rec[(size_t)i * 4 + 2];
            tex[j]   = (int)tm_float_to_bits(f->rec[(size_t)i * 4 + 3]);
            float ux = u * fac, uy = v * fac;
            float b;
            if (second)
            {
                // compute_blending_fac + blend_fac_index (RenderForward.cu:3493-3496, PointBlending.h:216-263): the weight of
                // the corner the pixel is, from the sub-pixel position.  A coordinate that is exactly an integer gets the
                // weight 0 on both of its pixels here; the first pipeline's closed form gives 1 and 0.
                float sx = ux - std::floor(ux), sy = uy - std::floor(uy);
                int q    = ((float)gx < ux ? 0 : 1) + ((float)gy < uy ? 0 : 2);
                b        = ((q & 1) ? sx : (1.f - sx)) * ((q & 2) ? sy : (1.f - sy));
            }
            else
                b = (1.f - std::fabs(ux - (float)gx)) * (1.f - std::fabs(uy - (float)gy));
            if (std::fabs(ux - (float)gx) > 1.f || std::fabs(uy - (float)gy) > 1.f) b = 0.f;
            float a = b * sc->confidence[tex[j]];
            if (pr->use_layer_point_size) a *= layer_factor(ps, layer, L, nullptr);
            alpha[j] = a;
        }
        float run = 1.f;
        if (second && pr->saturated_alpha_accumulation)
        {
            // RenderForward.cu:3524-3548 as written: the weight of a fragment is 1 while the alphas before it and its own sum
            // to less than 1, and saturate(1) / (alpha + 1e-9) (in double) for the fragment that crosses 1: its own lane's
            // alpha_dest is still the initial 1 when it is read there.  Below the cut-off: 0.
            for (int j = 0; j < n; ++j)
            {
                if (j > 0) run = run - alpha[j - 1];
                if (j == 0)
                    T[j] = 1.f;
                else if (run >= kAlphaCut)
                    T[j] = (run - alpha[j] > 0.f) ? 1.f : (float)(1.0 / ((double)alpha[j] + 1e-9));
                else
                    T[j] = 0.f;
            }
        }
        else
        {
            // transmittance chain: T_j = T_{j-1} * (1 - alpha_{j-1}); reported as 0 below the cut-off
            for (int j = 0; j < n; ++j)
            {
                if (j > 0) run = run * (1.f - alpha[j - 1]);
                T[j] = (j == 0 || run >= kAlphaCut) ? run : 0.f;
            }
        }
        for (int j = 0; j < kMaxKeep; ++j)
            for (int c = 0; c < C; ++c) contrib[j][c] = (j < n) ? T[j] * alpha[j] * sc->texture[(size_t)c * sc->n_tex + tex[j]] : 0.f;
        // butterfly sum over 16 lanes (xor shuffle with offsets 1,2,4,8, RenderForward.cu:983-994)
        for (int off = 1; off < kMaxKeep; off *= 2)
            for (int j = 0; j < kMaxKeep; j += 2 * off)
                for (int c = 0; c < C; ++c) contrib[j][c] = contrib[j][c] + contrib[j + off][c];
        float wb;
        if (n == 0)
            wb = 1.f;  // the reference reads a neighbouring lane here; defined as pure background
        else if (pr->bg_uses_Tn && !second)  // (an option of the first pipeline only)
        {
            float tn = run * (1.f - alpha[n - 1]);
            wb       = (T[n - 1] >= kAlphaCut && tn >= kAlphaCut) ? tn : 0.f;
        }
        else
            wb = T[n - 1];
        for (int c = 0; c < C; ++c)
        {
            float o = contrib[0][c];
            if (wb >= kAlphaCut) o += sc->background[c] * (wb * 1.f);
            f->pyramid[(size_t)C * f->base[layer] + ((size_t)c * f->H[layer] + gy) * f->W[layer] + gx] = o;
        }
        if (pr->train)
        {
            // Records exist for the leading fragments whose transmittance is above the cut-off; the backward
            // pass stops at the first absent record (RenderBackward.cu:205-210), so later ones are never read.
            int m = 0;
            while (m < n && T[m] >= kAlphaCut)
            {
                f->rec_pid[(size_t)p * kMaxKeep + m]   = pid[m];
                f->rec_alpha[(size_t)p * kMaxKeep + m] = alpha[m];
                ++m;
            }
            f->nrec[p] = m;
        }
    }
    f->Kf = kept;
    return f;
}

void or_frame_free(OrFrame* f) { delete f; }
int64_t or_num_pixels(const OrFrame* f) { return f->P; }
int64_t or_num_fragments(const OrFrame* f) { return f->F; }
int64_t or_num_kept(const OrFrame* f) { return f->Kf; }
int64_t or_num_visible(const OrFrame* f) { return f->V; }
void or_layer_size(const OrFrame* f, int layer, int* w, int* h, int64_t* base)
{
    if (w) *w = f->W[layer];
    if (h) *h = f->H[layer];
    if (base) *base = f->base[layer];
}

void or_get_points(const OrFrame* f, float* depth, int32_t* nlayers, float* rec)
{
    if (depth) memcpy(depth, f->depth.data(), sizeof(float) * f->N);
    if (nlayers) memcpy(nlayers, f->nlayers.data(), sizeof(int32_t) * f->N);
    if (rec) memcpy(rec, f->rec.data(), sizeof(float) * 4 * f->N);
}
void or_get_first_layer(const OrFrame* f, int32_t* first) { memcpy(first, f->first.data(), sizeof(int32_t) * f->N); }
void or_get_lists(const OrFrame* f, int32_t* counts, int64_t* offsets, uint64_t* frags)
{
    if (counts) memcpy(counts, f->counts.data(), sizeof(int32_t) * f->P);
    if (offsets) memcpy(offsets, f->offsets.data(), sizeof(int64_t) * f->P);
    if (frags) memcpy(frags, f->frags.data(), sizeof(uint64_t) * f->F);
}
void or_get_pyramid(const OrFrame* f, float* out) { memcpy(out, f->pyramid.data(), sizeof(float) * f->pyramid.size()); }
void or_get_records(const OrFrame* f, int32_t* nrec, int32_t* rec_pid, float* rec_alpha)
{
    if (nrec) memcpy(nrec, f->nrec.data(), sizeof(int32_t) * f->P);
    if (rec_pid && !f->rec_pid.empty()) memcpy(rec_pid, f->rec_pid.data(), sizeof(int32_t) * f->rec_pid.size());
    if (rec_alpha && !f->rec_alpha.empty()) memcpy(rec_alpha, f->rec_alpha.data(), sizeof(float) * f->rec_alpha.size());
}

// ---- A4: backward (BlendBackwardsBilinearTiled, RenderBackward.cu:90-618) ----
// Ticket -> pixel uses the ceil-halved layer sizes of the forward pass (the reference halves with floor here,
// RenderBackward.cu:112-130, which skips rows of odd-sized layers; that is treated as a defect, not followed).
void or_backward(const OrFrame* f, const OrScene* sc, const OrView* view, const OrParams* pr, const float* grad_pyramid,
                 double* g_texture, double* g_confidence, double* g_position, double* g_point_size,
                 double* g_background, double* g_pose, double* g_intrinsics)
{
    const int C = f->C, L = f->L, K = f->K;
    const Cam cam   = make_cam(view, pr);
    const float fxc = cam.fx * cam.cfx;
    std::vector<double> bg_acc(C, 0.0);
    double pose_acc[6] = {0, 0, 0, 0, 0, 0};
    double k_acc[13]   = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};  // fx fy cx cy s, then the 8 distortion coefficients
#pragma omp parallel
    {
        std::vector<double> bg_local(C, 0.0);
        double pose_local[6] = {0, 0, 0, 0, 0, 0};
        double k_local[13]   = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#pragma omp for schedule(dynamic, 1024)
        for (int64_t p = 0; p < f->P; ++p)
        {
            int layer = 0;
            while (p >= f->base[layer + 1]) ++layer;
            int64_t t = p - f->base[layer];
            int gx = (int)(t % f->W[layer]), gy = (int)(t / f->W[layer]);
            float g_in[16];
            for (int c = 0; c < C; ++c)
                g_in[c] = grad_pyramid[(size_t)C * f->base[layer] + ((size_t)c * f->H[layer] + gy) * f->W[layer] + gx];
            const int32_t* rpid  = &f->rec_pid[(size_t)p * kMaxKeep];
            const float* ralpha  = &f->rec_alpha[(size_t)p * kMaxKeep];
            float conf_grad[kMaxKeep];
            int texs[kMaxKeep];
            for (int j = 0; j < kMaxKeep; ++j) conf_grad[j] = 0.f;
            int idx          = 0;
            float alpha_dest = 1.f;
            do
            {
                bool fg         = true;
                float alpha_val = (idx >= K) ? -1.f : ralpha[idx];
                if (alpha_val == -1.f)
                {
                    fg        = false;
                    alpha_val = 1.f;
                }
                int tex = 0;
                if (fg)
                {
                    int pid   = rpid[idx];
                    tex       = sc->index ? sc->index[pid] : pid;
                    texs[idx] = tex;
                }
                float colors[16];
                for (int c = 0; c < C; ++c) colors[c] = fg ? sc->texture[(size_t)c * sc->n_tex + tex] : sc->background[c];
                float g_alpha = 0.f;
                if (pr->saturated_alpha_accumulation)
                {
                    // RenderBackward.cu:227-259 as written
                    const float sat = std::fmin(std::fmax(alpha_dest, 0.f), 1.f);
                    float alpha_TA  = ((alpha_dest - alpha_val) > 0.f) ? alpha_val : sat;
                    for (int c = 0; c < C; ++c)
                    {
                        float g = alpha_TA * g_in[c];
                        if (fg)
                        {
#pragma omp atomic
                            g_texture[(size_t)c * sc->n_tex + tex] += (double)g;
                        }
                        else
                            bg_local[c] += (double)g;
                        g_alpha += colors[c] * g_in[c];
                    }
                    if (fg) conf_grad[idx] += g_alpha;
                    if ((alpha_dest - alpha_val) < 0.f && alpha_dest > 0.f)
                    {
                        // the fragment that fills the pixel: its own gradient is dropped and the sum of its colours (not
                        // weighted by the incoming gradient) is taken from every fragment before it.  (The reference
                        // writes conf_gradients[idx] also for the background step after 16 records, one past the array.)
                        if (idx < kMaxKeep) conf_grad[idx] = 0.f;
                        for (int j = 0; j < idx; ++j)
                        {
                            float g_iter = 0.f;
                            for (int c = 0; c < C; ++c) g_iter += colors[c];
                            conf_grad[j] -= g_iter;
                        }
                    }
                    alpha_dest = std::fmin(std::fmax(alpha_dest - alpha_val, 0.f), 1.f);
                    if (!fg) break;
                    ++idx;
                    continue;
                }
                for (int c = 0; c < C; ++c)
                {
                    float g = alpha_dest * alpha_val * g_in[c];
                    if (fg)
                    {
#pragma omp atomic
                        g_texture[(size_t)c * sc->n_tex + tex] += (double)g;
                    }
                    else
                        bg_local[c] += (double)g;
                    g_alpha += colors[c] * g_in[c];
                }
                g_alpha *= alpha_dest;
                if (fg) conf_grad[idx] += g_alpha;
                for (int j = 0; j < idx; ++j)
                {
                    float a_j    = ralpha[j];
                    float g_iter = 0.f;
                    for (int c = 0; c < C; ++c)
                    {
                        const float epsilon = 1e-9f;
                        float dem           = 1.f / (1.f - a_j + epsilon);
                        float g_a           = (g_in[c] * colors[c] * alpha_dest * alpha_val * dem);
                        g_iter -= g_a;
                    }
                    conf_grad[j] += g_iter;
                }
                alpha_dest = (1.f - alpha_val) * alpha_dest;
                if (!fg) break;
                ++idx;
            } while (idx < K + 1 && alpha_dest >= kAlphaCut);

            for (int i = 0; i < idx; ++i)
            {
                int pid = rpid[i];
                int tex = texs[i];
                // the forward pass stored uv = ip * 2^-layer, the corner index and ps (RenderForward.cu:957-979);
                // they are recomputed here from the per-point record with the same arithmetic.
                const float fac = 1.f / (float)(1 << layer);
                float ux = f->rec[(size_t)pid * 4 + 0] * fac, uy = f->rec[(size_t)pid * 4 + 1] * fac;
                float ps = f->rec[(size_t)pid * 4 + 2];
                int q    = ((float)gx < ux ? 0 : 1) + ((float)gy < uy ? 0 : 2);  // blend_fac_index
                float ga = conf_grad[i];
                // compute_blending_fac (PointBlending.h:216-257)
                float sx = ux - std::floor(ux), sy = uy - std::floor(uy);
                float bf[4]   = {(1.f - sx) * (1.f - sy), sx * (1.f - sy), (1.f - sx) * sy, sx * sy};
                float J[4][2] = {{sy - 1.f, sx - 1.f}, {1.f - sy, -sx}, {-sy, 1.f - sx}, {sy, sx}};
                if (std::fabs(ux - (float)gx) > 1.f || std::fabs(uy - (float)gy) > 1.f)
                    for (int k = 0; k < 4; ++k) bf[k] *= 0.f;
                float conf = sc->confidence[tex];
                float lf_grad = 0.f;
                // (the reference applies the factor whenever the size gradient is requested, RenderBackward.cu:366-372; without
                // use_layer_point_size its forward pass stored no size to evaluate it with: no factor and no size gradient)
                float lf      = pr->use_layer_point_size ? layer_factor(ps, layer, L, &lf_grad) : 1.f;
                float g_conf  = bf[q] * lf * ga;
#pragma omp atomic
                g_confidence[tex] += (double)g_conf;
                float gbs   = conf * lf * ga;
                float grad0 = J[q][0] * gbs, grad1 = J[q][1] * gbs;  // dR_dp = J_uv^T * e_q * gbs

                // ProjectPointPinholeBackward (PointRendererHelper.h:434-494)
                const float* pos = sc->position + (size_t)pid * 4;
                float pv[3];
                transform_point(cam.V, pos, pv);
                float z = pv[2];
                if (z <= 0.f) continue;
                float g_layer_proj = fxc / z;
                float iz = 1.f / z;
                float nx = pv[0] * iz, ny = pv[1] * iz;
                // crop rotation^T, crop transform^T, K^T
                float gr0 = cam.r00 * grad0 + cam.r10 * grad1;
                float gr1 = cam.r01 * grad0 + cam.r11 * grad1;
                float gk0 = cam.cfx * gr0;               // J_p_K2^T = [[cfx,0],[cs,cfy]]
                float gk1 = cam.cs * gr0 + cam.cfy * gr1;
                float gn0 = cam.fx * gk0;                // J_p_K1^T = [[fx,0],[s,fy]]
                float gn1 = cam.s * gk0 + cam.fy * gk1;
                if (cam.dist)
                {
                    // distortNormalizedPoint between DivideByZ and K (PointRendererHelper.h:468-470): the pinhole
                    // coefficients see the distorted coordinates, the chain continues through J_p_dis^T, and the
                    // eight coefficients receive J_dis_dis^T (PointRendererHelper.h:485-491)
                    float xd, yd, Jd[4], Jk[16];
                    distort(cam, nx, ny, xd, yd, Jd, Jk);
                    for (int k = 0; k < 8; ++k) k_local[5 + k] += (double)(Jk[k] * gn0 + Jk[8 + k] * gn1);
                    const float g0 = Jd[0] * gn0 + Jd[2] * gn1;
                    const float g1 = Jd[1] * gn0 + Jd[3] * gn1;
                    gn0 = g0, gn1 = g1;
                    nx = xd, ny = yd;  // for the pinhole coefficients below
                }
                // DivideByZ^T
                float gv0 = iz * gn0;
                float gv1 = iz * gn1;
                float gv2 = (-pv[0] * iz * iz) * gn0 + (-pv[1] * iz * iz) * gn1;
                // J_point^T = R^T
                const float* R = cam.V.R;
                float gp0 = R[0] * gv0 + R[3] * gv1 + R[6] * gv2;
                float gp1 = R[1] * gv0 + R[4] * gv1 + R[7] * gv2;
                float gp2 = R[2] * gv0 + R[5] * gv1 + R[8] * gv2;
                if (g_point_size)
                {
                    float J_sp = tm_softplus_grad(sc->point_size[pid]);
                    float glp  = J_sp * g_layer_proj * lf_grad * ga;
                    float gl   = bf[q] * conf * glp;
#pragma omp atomic
                    g_point_size[pid] += (double)gl;
                }
                if (g_position)
                {
#pragma omp atomic
                    g_position[(size_t)pid * 4 + 0] += (double)gp0;
#pragma omp atomic
                    g_position[(size_t)pid * 4 + 1] += (double)gp1;
#pragma omp atomic
                    g_position[(size_t)pid * 4 + 2] += (double)gp2;
                }
                // pose tangent: J_pose = [I | -skew(pv)]  ->  g = (gv, pv x gv)
                pose_local[0] += gv0;
                pose_local[1] += gv1;
                pose_local[2] += gv2;
                pose_local[3] += (double)(pv[1] * gv2 - pv[2] * gv1);
                pose_local[4] += (double)(pv[2] * gv0 - pv[0] * gv2);
                pose_local[5] += (double)(pv[0] * gv1 - pv[1] * gv0);
                // K: d(ix,iy)/d(fx,fy,cx,cy,s) = [[nx,0,1,0,ny],[0,ny,0,1,0]]
                k_local[0] += (double)(nx * gk0);
                k_local[1] += (double)(ny * gk1);
                k_local[2] += (double)gk0;
                k_local[3] += (double)gk1;
                k_local[4] += (double)(ny * gk0);
            }
        }
#pragma omp critical
        {
            for (int c = 0; c < C; ++c) bg_acc[c] += bg_local[c];
            for (int k = 0; k < 6; ++k) pose_acc[k] += pose_local[k];
            for (int k = 0; k < 13; ++k) k_acc[k] += k_local[k];
        }
    }
    if (g_background)
        for (int c = 0; c < C; ++c) g_background[c] += bg_acc[c];
    if (g_pose)
        for (int k = 0; k < 6; ++k) g_pose[k] += pose_acc[k];
    if (g_intrinsics)
        for (int k = 0; k < 13; ++k) g_intrinsics[k] += k_acc[k];
}

// ---- A5: Adam (adam_step, MyAdam.cu:41-88) ----
void or_adam(int64_t n, float* w, const float* g, float* m, float* v, int64_t* steps, float lr, float beta1, float beta2,
             float eps, float rel_decay, float abs_decay, float clip, float lower_lr, float upper_lr)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i)
    {
        float gradient = g[i] / 1.f;
        float weight   = w[i];
        if (gradient == 0.f) continue;
        float gsq = gradient * gradient;
        float fm = m[i] = beta1 * m[i] + (1.f - beta1) * gradient;
        float sm = v[i] = beta2 * v[i] + (1.f - beta2) * gsq;
        steps[i]        = steps[i] + 1;
        uint32_t step   = (uint32_t)steps[i];
        float lr_t      = lr * (std::sqrt(1.f - std::pow(beta2, (float)step)) / (1.f - std::pow(beta1, (float)step)));
        float eff       = std::fmin(std::fmax(lr_t / (std::sqrt(sm) + eps), lower_lr), upper_lr);
        float decayed   = (1.f - rel_decay * lr_t) * weight - std::copysign(abs_decay * lr_t, weight);
        float nw        = decayed - eff * fm;
        if (clip != 0.f) nw = nw < -clip ? -clip : (clip < nw ? clip : nw);
        w[i] = nw;
    }
}

// ---- diagnostics for the parity report (no counterpart in the reference) ----
// How often the exact-bits ceil(log2(ps)) used by both this oracle and the CUDA library differs from the reference's
// expression ceil(log2f(ps)) (RenderForward.cu:345) evaluated with the host libm, and how often the number of pyramid
// layers of a point would change if softplus were evaluated with libm's expf / logf instead of the reproducible
// routines.  out[0] = visible points, out[1] = visible points with ps > 1, out[2] = points whose ceil(log2) differs,
// out[3] = points whose floor(log2) differs, out[4] = points whose layer count (before the footprint test) differs
// with a libm softplus, out[5] = points where tm_softplus and the libm softplus differ in any bit.
void or_layer_divergence(const OrFrame* f, const OrScene* sc, const OrView* view, const OrParams* pr, int64_t* out)
{
    const Cam cam   = make_cam(view, pr);
    const float fxc = cam.fx * cam.cfx;
    const int L     = pr->num_layers;
    int64_t vis = 0, big = 0, dceil = 0, dfloor = 0, dlayers = 0, dsoft = 0;
#pragma omp parallel for schedule(static) reduction(+ : vis, big, dceil, dfloor, dlayers, dsoft)
    for (int i = 0; i < f->N; ++i)
    {
        const float z = f->depth[i];
        if (!(z > 0.f)) continue;
        ++vis;
        const float ps = f->rec[(size_t)i * 4 + 2];
        const float x  = sc->point_size[i];
        const float sp_libm = x > 20.f ? x : std::log(1.f + std::exp(x));  // float overloads of libm
        if (tm_float_to_bits(sp_libm) != tm_float_to_bits(tm_softplus(x))) ++dsoft;
        const float ps_libm = fxc * sp_libm / z;
        int hi = 0, hi_libm = 0;
        if (ps > 1.f)
        {
            ++big;
            const int c_bits = tm_ceil_log2(ps), c_libm = (int)std::ceil(std::log2(ps));
            const int f_bits = tm_floor_log2(ps), f_libm = (int)std::floor(std::log2(ps));
            if (c_bits != c_libm) ++dceil;
            if (f_bits != f_libm) ++dfloor;
            hi = std::min(c_bits, L - 1);
        }
        if (ps_libm > 1.f) hi_libm = std::min((int)std::ceil(std::log2(ps_libm)), L - 1);
        if (hi != hi_libm) ++dlayers;
    }
    out[0] = vis;
    out[1] = big;
    out[2] = dceil;
    out[3] = dfloor;
    out[4] = dlayers;
    out[5] = dsoft;
}

// Largest error, in units of the last place of the double-precision libm result rounded to float, of tm_expf over
// [-87, 88] and of tm_logf over the positive normal floats, visiting every `stride`-th float.  This is the check of
// the reproducible routines (shared with the CUDA library) against an independent implementation.
void or_math_sweep(uint32_t stride, double* max_ulp_exp, double* max_ulp_log)
{
    if (stride == 0) stride = 1;
    auto ulp_of = [](float r) {
        uint32_t b = tm_float_to_bits(std::fabs(r));
        float up   = tm_bits_to_float(b + 1);
        return (double)up - (double)std::fabs(r);
    };
    double me = 0.0, ml = 0.0;
    const uint32_t pos_hi = tm_float_to_bits(88.0f), neg_hi = tm_float_to_bits(-87.0f);
#pragma omp parallel for schedule(static) reduction(max : me)
    for (int64_t k = 0; k <= (int64_t)(pos_hi / stride); ++k)
    {
        const float x = tm_bits_to_float((uint32_t)k * stride);
        const double ref = std::exp((double)x);
        me = std::max(me, std::fabs((double)tm_expf(x) - ref) / ulp_of((float)ref));
    }
#pragma omp parallel for schedule(static) reduction(max : me)
    for (int64_t k = 0; k <= (int64_t)((neg_hi - 0x80000000u) / stride); ++k)
    {
        const float x = tm_bits_to_float(0x80000000u + (uint32_t)k * stride);
        const double ref = std::exp((double)x);
        me = std::max(me, std::fabs((double)tm_expf(x) - ref) / ulp_of((float)ref));
    }
#pragma omp parallel for schedule(static) reduction(max : ml)
    for (int64_t k = 0; k <= (int64_t)((0x7f7fffffu - 0x00800000u) / stride); ++k)
    {
        const float y = tm_bits_to_float(0x00800000u + (uint32_t)k * stride);
        const double ref = std::log((double)y);
        const float rf   = (float)ref;
        const double u   = rf == 0.f ? 1.4e-45 : ulp_of(rf);
        ml = std::max(ml, std::fabs((double)tm_logf(y) - ref) / std::max(u, 1e-45));
    }
    *max_ulp_exp = me;
    *max_ulp_log = ml;
}

}  // extern "C"
