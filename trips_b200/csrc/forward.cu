// Forward rasterizer: project + count, scan, collect, per-pixel top-K sort and front-to-back blend.
//
// Stage map to the reference (src/lib/rendering/RenderForward.cu):
//   bin_count / bin_scan / bin_scatter kernels <- CountAndCollectTiled (:168-366)
//   scan_*_kernel         <- cub::DeviceScan + host glue (:1155-1232), here one device-side scan per view, no host sync
//   collect_kernel        <- SplattingPass               (:368-436)
//   sort_blend_kernel     <- FastSortFusedNew            (:474-1059)
// All views of a call are processed by one launch per stage (grid.y / ticket space spans the batch).
#include "common.cuh"

namespace trips
{
// ------------------------------------------------------------------------------------------------------------
// per-view camera constants
// ------------------------------------------------------------------------------------------------------------
__global__ void setup_cams_kernel(const TripsView* __restrict__ views, int B, const double* __restrict__ poses, int n_images,
                                  const float* __restrict__ intrinsics, int n_cameras, int distortion, float dist_cutoff,
                                  CamConst* __restrict__ cams, DevStats* stats)
{
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const TripsView v = views[b];
    CamConst c;
    const double* p = poses + (size_t)min(max(v.image_index, 0), n_images - 1) * 8;
    // DeviceRenderParams::Pose: SE3d cast to float (RenderConstants.h:85-88)
    c.qx = (float)p[0];
    c.qy = (float)p[1];
    c.qz = (float)p[2];
    c.qw = (float)p[3];
    c.tx = (float)p[4];
    c.ty = (float)p[5];
    c.tz = (float)p[6];
    // Eigen::Quaternion::toRotationMatrix
    float tx = 2.f * c.qx, ty = 2.f * c.qy, tz = 2.f * c.qz;
    float twx = tx * c.qw, twy = ty * c.qw, twz = tz * c.qw;
    float txx = tx * c.qx, txy = ty * c.qx, txz = tz * c.qx;
    float tyy = ty * c.qy, tyz = tz * c.qy, tzz = tz * c.qz;
    c.R[0] = 1.f - (tyy + tzz);
    c.R[1] = txy - twz;
    c.R[2] = txz + twy;
    c.R[3] = txy + twz;
    c.R[4] = 1.f - (txx + tzz);
    c.R[5] = tyz - twx;
    c.R[6] = txz - twy;
    c.R[7] = tyz + twx;
    c.R[8] = 1.f - (txx + tyy);
    const float* k = intrinsics + (size_t)min(max(v.camera_index, 0), n_cameras - 1) * 13;
    c.fx = k[0];
    c.fy = k[1];
    c.cx = k[2];
    c.cy = k[3];
    c.s  = k[4];
    bool dist = false;
    for (int i = 5; i < 13; ++i) dist |= (k[i] != 0.f);
    if (dist && !distortion) atomicOr(&stats->status, TRIPS_DEV_NONZERO_DISTORTION);  // a plain pinhole was asked for: ignored
    c.k1 = k[5], c.k2 = k[6], c.k3 = k[7], c.k4 = k[8], c.k5 = k[9], c.k6 = k[10], c.p1 = k[11], c.p2 = k[12];
    c.cut2 = dist_cutoff * dist_cutoff;
    c.dist = distortion ? 1 : 0;
    c.cfx  = v.crop_transform[0];
    c.cfy  = v.crop_transform[1];
    c.ccx  = v.crop_transform[2];
    c.ccy  = v.crop_transform[3];
    c.cs   = v.crop_transform[4];
    c.r00  = v.crop_rotation[0];
    c.r01  = v.crop_rotation[1];
    c.r10  = v.crop_rotation[2];
    c.r11  = v.crop_rotation[3];
    c.cenx = (float)(v.w / 2);  // integer division as in RenderForward.cu:303
    c.ceny = (float)(v.h / 2);
    c.image_index  = v.image_index;
    c.camera_index = v.camera_index;
    cams[b]        = c;
}

cudaError_t launch_setup_cams(const TripsView* d_views, int B, const double* poses, int n_images, const float* intrinsics,
                              int n_cameras, int distortion, float dist_cutoff, CamConst* cams, DevStats* stats, cudaStream_t st)
{
    setup_cams_kernel<<<(B + 63) / 64, 64, 0, st>>>(d_views, B, poses, n_images, intrinsics, n_cameras, distortion, dist_cutoff, cams, stats);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// project + cull + layer select, and sort the visible points of every view by (32x32 screen bin, 8x4 tile of the bin)
//
// Kernels: bounding boxes of blocks of consecutive points and their visibility per view; (1) count the visible points
// per (view, bin, tile) with one global counter each; (2) exclusive scan of the counters; (3) project again, take a slot
// in the point's group and write its entry there (head and tail, 32 bytes each).  Replaces the projection part of
// CountAndCollectTiled (RenderForward.cu:168-366); the list lengths are counted afterwards from the entries
// (window_kernel<false>).  Both passes read every point ONCE per call and loop over the views with the point in
// registers (the camera constants of up to kViewGroup views sit in shared memory): position, size and, in the scatter
// pass, confidence, descriptor row and rank cost N reads per call instead of N x B, and softplus(size) is evaluated
// once per point.  Projecting twice avoids writing and re-reading a per-point record for all N x B point-views.
// ------------------------------------------------------------------------------------------------------------
struct Projected
{
    float u, v, z, ps, rad;
    bool ok;
};

// Visibility test of one point in one view (RenderForward.cu:224-340).  `sp` caches softplus(raw) across the views of
// the point: negative = not computed yet (softplus is never negative); only visible points pay for it.
__device__ __forceinline__ Projected project_visible(const CamConst& cam, const Geom& g, const TripsRenderParams& pr, const float4& p,
                                                     float raw, float& sp)
{
    Projected r;
    const float fxc = cam.fx * cam.cfx;
    project_point(cam, p.x, p.y, p.z, r.u, r.v, r.z);
    r.rad = fxc * p.w / r.z;
    r.ps  = 0.f;
    bool ok = !(r.z <= 0.f || r.u < 0.f || r.u >= (float)(g.W[0] - 1) || r.v < 0.f || r.v >= (float)(g.H[0] - 1));
    // the first pipeline's test takes an int (RenderForward.cu:212-218), the second's the float (RenderForward.cu:1527-1531)
    if (ok && pr.drop_out_points_by_radius && (second_pipeline(pr) ? r.rad : (float)(int)r.rad) < pr.drop_out_radius_threshold) ok = false;
    if (ok)
    {
        if (sp < 0.f) sp = tm_softplus(raw);
        r.ps = fxc * sp / r.z;
    }
    r.ok = ok;
    return r;
}

constexpr int kBinThreads     = 256;
constexpr int kBinBlocksPerSM = 8;
constexpr int kScatterMinBlocks = 3;   // measured on config 3: 1.46 ms unbounded (95 registers), 1.34 ms at 3 resident blocks (85), 1.36 ms at 4 (64)
constexpr int kBinChunk       = 8192;  // points per bounding box
constexpr int kBinTicket      = 1024;
constexpr int kSweep          = 4;      // views whose entry slots a thread requests before it waits for any of them  // points per work ticket of the binning kernels; a ticket lies inside one box
constexpr int kViewGroup      = 16;    // views whose camera constants are in shared memory at a time (one launch per group)
static_assert(kBinChunk % kBinTicket == 0, "a ticket must not straddle two bounding boxes");

// Bounding boxes of blocks of consecutive points and the conservative frustum test on them: the reference computes
// such boxes per 10 240 points (NeuralPointCloudCuda.cpp:339-384) but never uses them.  Point clouds stored in a
// spatially coherent order (scans, reconstructions) have compact blocks, and a block whose box lies outside a view
// is skipped by both binning passes; for a cloud in random order every box spans the scene and nothing is skipped.
// Boxes are recomputed by every forward pass (points move): one read of the positions.
__global__ __launch_bounds__(256) void block_box_kernel(const float4* __restrict__ pos, int N, float* __restrict__ boxes)
{
    const int first = blockIdx.x * kBinChunk, last = min(N, first + kBinChunk);
    float lo[3] = {3.0e38f, 3.0e38f, 3.0e38f}, hi[3] = {-3.0e38f, -3.0e38f, -3.0e38f};
    bool bad = false;
    for (int i = first + threadIdx.x; i < last; i += 256)
    {
        const float4 p = pos[i];
        const float v[3] = {p.x, p.y, p.z};
#pragma unroll
        for (int k = 0; k < 3; ++k)
        {
            bad |= !(fabsf(v[k]) < 3.0e38f);  // NaN or infinite: the block is never skipped
            lo[k] = fminf(lo[k], v[k]);
            hi[k] = fmaxf(hi[k], v[k]);
        }
    }
    __shared__ float s_lo[8][3], s_hi[8][3];
    __shared__ int s_bad;
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    if (bad) s_bad = 1;
#pragma unroll
    for (int k = 0; k < 3; ++k)
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            lo[k] = fminf(lo[k], __shfl_xor_sync(kFull, lo[k], o));
            hi[k] = fmaxf(hi[k], __shfl_xor_sync(kFull, hi[k], o));
        }
        if ((threadIdx.x & 31) == 0) s_lo[threadIdx.x >> 5][k] = lo[k], s_hi[threadIdx.x >> 5][k] = hi[k];
    }
    __syncthreads();
    if (threadIdx.x < 3)
    {
        float a = s_lo[0][threadIdx.x], b = s_hi[0][threadIdx.x];
        for (int w = 1; w < 8; ++w) a = fminf(a, s_lo[w][threadIdx.x]), b = fmaxf(b, s_hi[w][threadIdx.x]);
        if (s_bad) a = -3.4e38f, b = 3.4e38f;
        boxes[(size_t)blockIdx.x * 6 + threadIdx.x]     = a;
        boxes[(size_t)blockIdx.x * 6 + 3 + threadIdx.x] = b;
    }
}

// True when no point inside the box can pass the visibility test of project_visible for this view.  The image position
// is an affine map of (x/z, y/z); multiplied by z > 0 every image border becomes a plane through the camera centre,
// i.e. a linear function of the view-space position, and a box lies outside a plane when its 8 corners do.  The borders
// are moved out by a margin of 2 pixels (+ 1e-3 of the depth), far more than the rounding difference between this
// test and the per-point arithmetic.
__device__ __forceinline__ bool box_outside_view(const CamConst& c, const Geom& g, const float* __restrict__ box)
{
    if (!(box[3] < 3.0e38f)) return false;
    // u(nx, ny) = cu + au nx + bu ny, v likewise: evaluate the projection chain at three normalised positions
    float u0, v0, u1, v1, u2, v2;
    {
        auto img = [&](float nx, float ny, float& u, float& v) {
            const float ix = (c.fx * nx + c.s * ny) + c.cx, iy = c.fy * ny + c.cy;
            const float jx = (c.cfx * ix + c.cs * iy) + c.ccx, jy = c.cfy * iy + c.ccy;
            const float dx = jx - c.cenx, dy = jy - c.ceny;
            u = (c.r00 * dx + c.r01 * dy) + c.cenx;
            v = (c.r10 * dx + c.r11 * dy) + c.ceny;
        };
        img(0.f, 0.f, u0, v0);
        img(1.f, 0.f, u1, v1);
        img(0.f, 1.f, u2, v2);
    }
    const float au = u1 - u0, bu = u2 - u0, av = v1 - v0, bv = v2 - v0;
    const float m = 2.f, wmax = (float)(g.W[0] - 1) + m, hmax = (float)(g.H[0] - 1) + m;
    bool all_behind = true, all_left = true, all_right = true, all_up = true, all_down = true;
#pragma unroll
    for (int k = 0; k < 8; ++k)
    {
        float x, y, z;
        transform_point(c, box[(k & 1) ? 3 : 0], box[(k & 2) ? 4 : 1], box[(k & 4) ? 5 : 2], x, y, z);
        const float U = au * x + bu * y + u0 * z, V = av * x + bv * y + v0 * z;
        const float slack = 1e-3f * fabsf(z) + 1e-6f * (fabsf(x) + fabsf(y));
        all_behind &= z < -slack;
        all_left &= (U + m * z) < -slack * (fabsf(au) + fabsf(bu) + fabsf(u0) + m);
        all_right &= (wmax * z - U) < -slack * (fabsf(au) + fabsf(bu) + fabsf(u0) + wmax);
        all_up &= (V + m * z) < -slack * (fabsf(av) + fabsf(bv) + fabsf(v0) + m);
        all_down &= (hmax * z - V) < -slack * (fabsf(av) + fabsf(bv) + fabsf(v0) + hmax);
    }
    return all_behind || all_left || all_right || all_up || all_down;
}

// skip[b * n_blocks + k] = 1 when block k of the point cloud cannot hold a point visible in view b.  A kernel of its
// own: inside the binning kernels the test would cost their loops 30 registers.
__global__ __launch_bounds__(128) void block_visibility_kernel(const CamConst* __restrict__ cams, const __grid_constant__ Geom g, int B,
                                                               int n_blocks, const float* __restrict__ boxes, uint8_t* __restrict__ skip,
                                                               DevStats* stats)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * n_blocks) return;
    const int b = i / n_blocks, k = i - b * n_blocks;
    const CamConst cam = cams[b];
    const bool out = box_outside_view(cam, g, boxes + (size_t)k * 6);
    skip[i] = out ? 1 : 0;
    if (out) atomicAdd(&stats->culled_blocks, 1u);
}

// Work distribution of the binning kernels: tickets of kBinTicket consecutive points from one counter, so that every SM
// is busy until the last ticket whatever the number of resident blocks is (a static split left a partial last wave).
// Returns false when the cloud is exhausted; `skip` gets one bit per view of the group whose bounding-box test rules the
// ticket's points out.
__device__ __forceinline__ bool next_point_ticket(unsigned* ticket, int N, unsigned* s_ticket, const uint8_t* __restrict__ block_skip, int v0,
                                                  int nv, int& first, int& last, unsigned& skip)
{
    __syncthreads();
    if (threadIdx.x == 0) *s_ticket = atomicAdd(ticket, 1u);
    __syncthreads();
    const unsigned t = *s_ticket;
    if (t >= ((unsigned)N + kBinTicket - 1) / kBinTicket) return false;
    first = (int)(t * kBinTicket);
    last  = min(N, first + kBinTicket);
    skip  = 0;
    if (block_skip)
    {
        const int n_box = (N + kBinChunk - 1) / kBinChunk, box = first / kBinChunk;
        for (int v = 0; v < nv; ++v) skip |= (unsigned)block_skip[(size_t)(v0 + v) * n_box + box] << v;  // uniform loads
    }
    return true;
}

// Sort key of a visible point: its 32x32 screen bin, then its 8x4 pixel tile inside the bin.  Entries of a tile are
// contiguous, so the fragments a tile kernel works on refer to a short range of entries and gradient rows: the 32
// gathers (or atomics) of a warp instruction touch a handful of 128-byte lines instead of 32 different ones.
constexpr int kSubShift = 5;  // 32 tiles (4 x 8) per bin
__device__ __forceinline__ int bin_key(const Geom& g, float u, float v)
{
    const int px = __float2int_rd(u), py = __float2int_rd(v);
    const int bin = (py >> kBinShift) * g.bins_x + (px >> kBinShift);
    return (bin << kSubShift) | (((py >> 2) & 7) << 2) | ((px >> 3) & 3);
}

// discard_point_for_confidence (RenderForward.cu:122-130): viewer only, points below the stability cut-off are not drawn
template <bool ACT>
__device__ __forceinline__ bool discarded_for_confidence(const ScenePtrs& sc, const TripsRenderParams& pr, int tex)
{
    if (!pr.viewer_only || (unsigned)tex >= (unsigned)sc.n_tex) return false;
    float c = __ldg(sc.confidence + tex);
    if (ACT && pr.confidence_is_raw) c = tm_sigmoid(pr.confidence_scale * c);
    return c < pr.stability_cutoff_value;
}

// ACT: the scene tensors may be raw parameters (fused texture preparation); compiled separately so that the common case
// carries none of its code.  One launch handles the views [v0, v0 + nv).
template <bool ACT>
__global__ __launch_bounds__(kBinThreads) void bin_count_kernel(ScenePtrs sc, const CamConst* __restrict__ cams, const __grid_constant__ Geom g,
                                                                TripsRenderParams pr, FwdBuffers fb, int v0, int nv, unsigned* ticket)
{
    __shared__ CamConst s_cam[kViewGroup];
    __shared__ unsigned s_ticket;
    for (int k = threadIdx.x; k < nv * (int)(sizeof(CamConst) / 4); k += kBinThreads) ((int*)s_cam)[k] = ((const int*)(cams + v0))[k];
    const bool use_dropout = pr.train && sc.dropout;  // the mask applies with and without viewer_only (RenderForward.cu:224-240)
    int first, last;
    unsigned skip;
    while (next_point_ticket(ticket, sc.N, &s_ticket, fb.block_skip, v0, nv, first, last, skip))
    {
        for (int i = first + threadIdx.x; i < last; i += kBinThreads)
        {
            const int tex = sc.index ? __ldg(sc.index + i) : i;
            if (discarded_for_confidence<ACT>(sc, pr, tex)) continue;
            const float4 p  = __ldg(sc.position + i);
            const float raw = __ldg(sc.point_size + i);
            float sp        = -1.f;
            for (int v = 0; v < nv; ++v)
            {
                if ((skip >> v) & 1u) continue;  // uniform
                if (use_dropout && __ldg(sc.dropout + (size_t)(v0 + v) * sc.N + i) == 1.f) continue;
                const Projected r = project_visible(s_cam[v], g, pr, p, raw, sp);
                if (r.ok) atomicAdd(fb.bin_count + ((size_t)(v0 + v) * g.n_bins << kSubShift) + bin_key(g, r.u, r.v), 1u);
            }
        }
    }
}

// one block per view: rows [n_blocks, n_bins] of per-block counts -> first entry (within the view) of every
// (block, bin) pair, ordered by bin first and block second; view_total[b] = visible points of the view
__global__ __launch_bounds__(1024) void bin_scan_kernel(const uint32_t* __restrict__ rows_in, uint32_t* __restrict__ rows_out,
                                                        uint32_t* __restrict__ bin_first, int n_bins, int n_blocks,
                                                        uint32_t* __restrict__ view_total, int first_shift, DevStats* stats)
{
    __shared__ uint32_t sm[32];
    __shared__ uint32_t carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b    = blockIdx.x;
    const uint32_t* r = rows_in + (size_t)b * n_blocks * n_bins;
    uint32_t* w       = rows_out + (size_t)b * n_blocks * n_bins;
    uint32_t* o       = bin_first + (size_t)b * (n_bins >> first_shift);  // first entry of every group of 2^first_shift keys
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int s = 0; s < n_bins; s += 1024)
    {
        const int i = s + threadIdx.x;
        uint32_t v  = 0;  // visible points of bin i (sum over blocks)
        if (i < n_bins)
            for (int k = 0; k < n_blocks; ++k) v += r[(size_t)k * n_bins + i];
        if (v >= kHotKey) atomicMax(&stats->max_key, v);  // crowded group: the next call uses the aggregating binning kernels
        uint32_t inc = v;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1)
        {
            uint32_t t = __shfl_up_sync(kFull, inc, k);
            if (lane >= k) inc += t;
        }
        if (lane == 31) sm[warp] = inc;
        __syncthreads();
        uint32_t wsum = sm[lane];
        uint32_t winc = wsum;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1)
        {
            uint32_t t = __shfl_up_sync(kFull, winc, k);
            if (lane >= k) winc += t;
        }
        const uint32_t tot   = __shfl_sync(kFull, winc, 31);
        const uint32_t woff  = __shfl_sync(kFull, winc - wsum, warp);
        const uint32_t carry = carry_s;
        if (i < n_bins)
        {
            uint32_t run = carry + woff + inc - v;  // first entry of bin i
            if ((i & ((1 << first_shift) - 1)) == 0) o[i >> first_shift] = run;
            for (int k = 0; k < n_blocks; ++k)
            {
                w[(size_t)k * n_bins + i] = run;
                run += r[(size_t)k * n_bins + i];
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + tot;
        __syncthreads();
    }
    if (threadIdx.x == 0) view_total[b] = carry_s;
}

// First entry of every view in the entry arrays.  A view whose entries do not fit the arrays (entry_cap entries: the
// arrays are sized from the previous call's count, not for the worst case) gets none: it renders as background, the
// status word says so and stats->visible still carries the number that was needed, so that the host grows the arrays.
__global__ void entry_base_kernel(const uint32_t* __restrict__ view_total, int B, unsigned long long entry_cap,
                                  unsigned long long* __restrict__ entry_base, DevStats* stats)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    unsigned long long base = 0, need = 0;
    for (int b = 0; b < B; ++b)
    {
        entry_base[b] = base;
        need += view_total[b];
        if (base + view_total[b] <= entry_cap)
            base += view_total[b];
        else
            atomicOr(&stats->status, TRIPS_DEV_ENTRY_OVERFLOW);
    }
    entry_base[B]  = base;
    stats->visible = need;
}

// One 32-byte store (sm_100 has 256-bit global stores) for the two float4 halves of a 32-byte-aligned record: half the
// store instructions of the entry scatter, each covering a whole sector.
__device__ __forceinline__ void store_entry_head(float4* dst, const float4& a, const float4& b)
{
    // Entries of one screen tile are written by many point blocks at different times.  Keeping the written lines in L2 for as
    // long as it will hold them lets neighbouring 32-byte sectors meet in one line before it goes to DRAM (measured: the
    // scatter pass 3 % faster than with the default policy, evict_first no different from the default).
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("st.global.L2::cache_hint.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8}, %9;" ::"l"(dst), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w), "f"(b.x), "f"(b.y),
                 "f"(b.z), "f"(b.w), "l"(policy)
                 : "memory");
}

// What an entry carries of its point besides the projection: fetched once per point, when it turns out visible in a view.
template <int C>
struct PointRow
{
    static constexpr int C4 = (C + 3) & ~3;
    bool fetched = false, tex_ok = false;
    int tex      = 0;
    float conf   = 0.f;
    uint32_t rk  = 0u;
    float row[C4];
};

template <int C, bool ACT>
__device__ __forceinline__ void fetch_point_row(const ScenePtrs& sc, const TripsRenderParams& pr, const FwdBuffers& fb, int i, PointRow<C>& d)
{
    if (d.fetched) return;
    d.fetched = true;
    if (d.tex_ok)
    {
        d.conf = __ldg(sc.confidence + d.tex);
        if (ACT && pr.confidence_is_raw) d.conf = tm_sigmoid(pr.confidence_scale * d.conf);  // PrepareConfidence, NeuralTexture.h:40-43
    }
    else
        atomicOr(&fb.stats->status, TRIPS_DEV_BAD_TEXTURE_INDEX);  // the point is drawn with alpha 0
#pragma unroll
    for (int c = 0; c < PointRow<C>::C4; ++c) d.row[c] = (c < C && d.tex_ok) ? __ldg(sc.texture + (size_t)c * sc.n_tex + d.tex) : 0.f;
    if (ACT && pr.texture_abs)  // PrepareTexture, NeuralTexture.h:45-57
    {
#pragma unroll
        for (int c = 0; c < PointRow<C>::C4; ++c) d.row[c] = fabsf(d.row[c]);
    }
    d.rk = fb.point_rank ? __ldg(fb.point_rank + i) : 0u;
}

// Writes entry `at` (index into the entry arrays) of point i as projected by `r`.
template <int C>
__device__ __forceinline__ void write_entry(const FwdBuffers& fb, const Geom& g, const TripsRenderParams& pr, unsigned long long at, int i,
                                            const float4& p, float raw, const Projected& r, const PointRow<C>& d)
{
    constexpr int TS = tail_stride(C);
    constexpr int C4 = PointRow<C>::C4;
    // layers first..hi, stopping where the 2x2 footprint leaves the layer (RenderForward.cu:342-363).  first = 0 except for
    // the strict write of the second pipeline, which starts at the layer below log2(size) (RenderForward.cu:2291-2393);
    // without use_layer_point_size every layer is written (RenderForward.cu:1611-1631).  The entry stores the NUMBER of
    // layers; the first layer of a strict entry is recomputed from its size where needed (strict_first_layer).
    int hi = 0, first = 0;
    if (!pr.use_layer_point_size)
        hi = g.L - 1;
    else if (r.ps > 1.f)
    {
        hi = min(tm_ceil_log2(r.ps), g.L - 1);
        if (!pr.render_points_in_all_lower_resolutions) first = min(tm_floor_log2(r.ps), g.L - 1);
    }
    const bool second = second_pipeline(pr);
    const float sc0   = __int_as_float((127 - first) << 23);  // 2^-first
    int layer = first;
    float x = r.u * sc0, y = r.v * sc0, rad = r.rad * sc0;
    for (; layer < hi + 1; ++layer, x *= 0.5f, y *= 0.5f, rad *= 0.5f)
    {
        const int px = __float2int_rd(x), py = __float2int_rd(y);
        if (px < 0 || px >= g.W[layer] - 1 || py < 0 || py >= g.H[layer] - 1) break;
        if (pr.drop_out_points_by_radius && (second ? rad : (float)(int)rad) < pr.drop_out_radius_threshold) break;
    }
    store_entry_head(fb.ent_head + at * 2, make_float4(r.u, r.v, r.ps, d.conf),
                     make_float4(__int_as_float(i), r.z, raw, __uint_as_float((uint32_t)(layer - first) | (d.rk << kRankShift))));
    float4* e = reinterpret_cast<float4*>(fb.ent_tail + at * TS);
    if constexpr (C4 == 4)
        store_entry_head(e, make_float4(p.x, p.y, p.z, __int_as_float(d.tex_ok ? d.tex : -1)), make_float4(d.row[0], d.row[1], d.row[2], d.row[3]));
    else
    {
        e[0] = make_float4(p.x, p.y, p.z, __int_as_float(d.tex_ok ? d.tex : -1));
#pragma unroll
        for (int c = 0; c < C4; c += 4) e[1 + c / 4] = make_float4(d.row[c], d.row[c + 1], d.row[c + 2], d.row[c + 3]);
    }
}

template <int C, bool ACT>
__global__ __launch_bounds__(kBinThreads, kScatterMinBlocks) void bin_scatter_kernel(ScenePtrs sc, const CamConst* __restrict__ cams, const __grid_constant__ Geom g,
                                                                  TripsRenderParams pr, FwdBuffers fb, int v0, int nv, unsigned* ticket)
{
    __shared__ CamConst s_cam[kViewGroup];
    __shared__ unsigned long long s_ebase[kViewGroup + 1];
    __shared__ unsigned s_ticket;
    for (int k = threadIdx.x; k < nv * (int)(sizeof(CamConst) / 4); k += kBinThreads) ((int*)s_cam)[k] = ((const int*)(cams + v0))[k];
    if (threadIdx.x <= nv) s_ebase[threadIdx.x] = fb.entry_base[v0 + threadIdx.x];
    __syncthreads();
    unsigned no_room = 0;  // views without entries: nothing visible, or the view did not fit the entry arrays
    for (int v = 0; v < nv; ++v) no_room |= (s_ebase[v + 1] == s_ebase[v] ? 1u : 0u) << v;
    const bool use_dropout = pr.train && sc.dropout;
    int first, last;
    unsigned skip;
    while (next_point_ticket(ticket, sc.N, &s_ticket, fb.block_skip, v0, nv, first, last, skip))
    {
        skip |= no_room;
        for (int i = first + threadIdx.x; i < last; i += kBinThreads)
        {
            PointRow<C> d;
            d.tex    = sc.index ? __ldg(sc.index + i) : i;
            d.tex_ok = (unsigned)d.tex < (unsigned)sc.n_tex;
            if (discarded_for_confidence<ACT>(sc, pr, d.tex)) continue;
            const float4 p  = __ldg(sc.position + i);
            const float raw = __ldg(sc.point_size + i);
            float sp        = -1.f;
            // Views are handled kSweep at a time in two sweeps: the first projects and takes the entry slots (up to kSweep
            // returning atomics in flight per thread instead of one), the second projects again (the same arithmetic,
            // hence the same bits) and writes the entries.  Waiting for each slot before the next projection made the
            // kernel latency-bound.
            for (int vb = 0; vb < nv; vb += kSweep)
            {
                uint32_t slot[kSweep];
                unsigned vis = 0;
#pragma unroll
                for (int j = 0; j < kSweep; ++j)
                {
                    const int v = vb + j;
                    slot[j]     = 0;
                    if (v >= nv || ((skip >> v) & 1u)) continue;  // uniform
                    if (use_dropout && __ldg(sc.dropout + (size_t)(v0 + v) * sc.N + i) == 1.f) continue;
                    const Projected r = project_visible(s_cam[v], g, pr, p, raw, sp);
                    if (!r.ok) continue;
                    vis |= 1u << j;
                    slot[j] = atomicAdd(fb.bin_base + ((size_t)(v0 + v) * g.n_bins << kSubShift) + bin_key(g, r.u, r.v), 1u);
                }
                if (!vis) continue;
                fetch_point_row<C, ACT>(sc, pr, fb, i, d);
#pragma unroll
                for (int j = 0; j < kSweep; ++j)
                {
                    if (!((vis >> j) & 1u)) continue;
                    const int v       = vb + j;
                    const Projected r = project_visible(s_cam[v], g, pr, p, raw, sp);
                    write_entry<C>(fb, g, pr, s_ebase[v] + slot[j], i, p, raw, r, d);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// The same two passes for point clouds that crowd into a few screen tiles (a distant or tiny object: millions of points
// in a 64x64-pixel window).  There the per-(bin, tile) counters above become a handful of addresses that every thread
// of the machine updates, and same-address atomics are served one after the other.  These variants aggregate in shared
// memory first: a block takes a ticket of kHotTicket points, counts its visible point-views per key in a small hash
// table (linear probing, at most four probes; a key that finds no slot simply uses the global counter directly), and
// touches the global counter of every key it met once per ticket.  In the scatter pass that one returning atomic
// reserves a range of the key's entries for the whole ticket, and the slots inside the range come from the table.
// The host selects these variants when the previous call (or, in a sized call, this call's own count pass) saw more
// than kHotKey visible points in one (view, bin, tile) group; ordinary scenes never do and run the kernels above.
// ------------------------------------------------------------------------------------------------------------
constexpr int kHotTicket        = 2048;
constexpr int kHotSlots         = 2048;
constexpr uint32_t kHotEmpty    = 0xffffffffu;

__device__ __forceinline__ uint32_t hot_hash(uint32_t key) { return (key * 2654435761u) >> 21; }  // 11 bits

__device__ __forceinline__ int hot_find_or_insert(uint32_t* tag, uint32_t key)
{
    const uint32_t h = hot_hash(key);
#pragma unroll
    for (int probe = 0; probe < 4; ++probe)
    {
        const uint32_t s   = (h + probe) & (kHotSlots - 1);
        const uint32_t old = atomicCAS(tag + s, kHotEmpty, key);
        if (old == kHotEmpty || old == key) return (int)s;
    }
    return -1;
}

__device__ __forceinline__ int hot_find(const uint32_t* tag, uint32_t key)
{
    const uint32_t h = hot_hash(key);
#pragma unroll
    for (int probe = 0; probe < 4; ++probe)
    {
        const uint32_t s = (h + probe) & (kHotSlots - 1);
        const uint32_t t = tag[s];
        if (t == key) return (int)s;
        if (t == kHotEmpty) return -1;
    }
    return -1;
}

__device__ __forceinline__ bool next_hot_ticket(unsigned* ticket, int N, unsigned* s_ticket, int& first, int& last)
{
    __syncthreads();
    if (threadIdx.x == 0) *s_ticket = atomicAdd(ticket, 1u);
    __syncthreads();
    const unsigned t = *s_ticket;
    if (t >= ((unsigned)N + kHotTicket - 1) / kHotTicket) return false;
    first = (int)(t * kHotTicket);
    last  = min(N, first + kHotTicket);
    return true;
}

template <bool ACT>
__global__ __launch_bounds__(kBinThreads) void bin_count_hot_kernel(ScenePtrs sc, const CamConst* __restrict__ cams, const __grid_constant__ Geom g,
                                                                    TripsRenderParams pr, FwdBuffers fb, int v0, int nv, unsigned* ticket)
{
    __shared__ CamConst s_cam[kViewGroup];
    __shared__ uint32_t s_tag[kHotSlots], s_cnt[kHotSlots];
    __shared__ unsigned s_ticket;
    for (int k = threadIdx.x; k < nv * (int)(sizeof(CamConst) / 4); k += kBinThreads) ((int*)s_cam)[k] = ((const int*)(cams + v0))[k];
    const bool use_dropout = pr.train && sc.dropout;
    const uint32_t n_keys  = (uint32_t)g.n_bins << kSubShift;
    uint32_t* counters     = fb.bin_count + (size_t)v0 * n_keys;  // counter of (view v0 + v, key) at [v * n_keys + key]
    int first, last;
    while (next_hot_ticket(ticket, sc.N, &s_ticket, first, last))
    {
        for (int k = threadIdx.x; k < kHotSlots; k += kBinThreads) s_tag[k] = kHotEmpty, s_cnt[k] = 0u;
        __syncthreads();
        for (int i = first + threadIdx.x; i < last; i += kBinThreads)
        {
            const int tex = sc.index ? __ldg(sc.index + i) : i;
            if (discarded_for_confidence<ACT>(sc, pr, tex)) continue;
            const float4 p  = __ldg(sc.position + i);
            const float raw = __ldg(sc.point_size + i);
            float sp        = -1.f;
            for (int v = 0; v < nv; ++v)
            {
                if (use_dropout && __ldg(sc.dropout + (size_t)(v0 + v) * sc.N + i) == 1.f) continue;
                const Projected r = project_visible(s_cam[v], g, pr, p, raw, sp);
                if (!r.ok) continue;
                const uint32_t key = (uint32_t)v * n_keys + (uint32_t)bin_key(g, r.u, r.v);
                const int s        = hot_find_or_insert(s_tag, key);
                if (s >= 0)
                    atomicAdd(s_cnt + s, 1u);
                else
                    atomicAdd(counters + key, 1u);
            }
        }
        __syncthreads();
        for (int k = threadIdx.x; k < kHotSlots; k += kBinThreads)
            if (s_tag[k] != kHotEmpty) atomicAdd(counters + s_tag[k], s_cnt[k]);
    }
}

template <int C, bool ACT>
__global__ __launch_bounds__(kBinThreads) void bin_scatter_hot_kernel(ScenePtrs sc, const CamConst* __restrict__ cams, const __grid_constant__ Geom g,
                                                                      TripsRenderParams pr, FwdBuffers fb, int v0, int nv, unsigned* ticket)
{
    __shared__ CamConst s_cam[kViewGroup];
    __shared__ unsigned long long s_ebase[kViewGroup + 1];
    __shared__ uint32_t s_tag[kHotSlots], s_cnt[kHotSlots], s_base[kHotSlots];
    __shared__ unsigned s_ticket;
    for (int k = threadIdx.x; k < nv * (int)(sizeof(CamConst) / 4); k += kBinThreads) ((int*)s_cam)[k] = ((const int*)(cams + v0))[k];
    if (threadIdx.x <= nv) s_ebase[threadIdx.x] = fb.entry_base[v0 + threadIdx.x];
    __syncthreads();
    unsigned no_room = 0;  // views without entries: nothing visible, or the view did not fit the entry arrays
    for (int v = 0; v < nv; ++v) no_room |= (s_ebase[v + 1] == s_ebase[v] ? 1u : 0u) << v;
    const bool use_dropout = pr.train && sc.dropout;
    const uint32_t n_keys  = (uint32_t)g.n_bins << kSubShift;
    uint32_t* cursors      = fb.bin_base + (size_t)v0 * n_keys;
    int first, last;
    while (next_hot_ticket(ticket, sc.N, &s_ticket, first, last))
    {
        for (int k = threadIdx.x; k < kHotSlots; k += kBinThreads) s_tag[k] = kHotEmpty, s_cnt[k] = 0u;
        __syncthreads();
        // ---- the ticket's visible point-views per key ----
        for (int i = first + threadIdx.x; i < last; i += kBinThreads)
        {
            const int tex = sc.index ? __ldg(sc.index + i) : i;
            if (discarded_for_confidence<ACT>(sc, pr, tex)) continue;
            const float4 p  = __ldg(sc.position + i);
            const float raw = __ldg(sc.point_size + i);
            float sp        = -1.f;
            for (int v = 0; v < nv; ++v)
            {
                if ((no_room >> v) & 1u) continue;  // uniform
                if (use_dropout && __ldg(sc.dropout + (size_t)(v0 + v) * sc.N + i) == 1.f) continue;
                const Projected r = project_visible(s_cam[v], g, pr, p, raw, sp);
                if (!r.ok) continue;
                const int s = hot_find_or_insert(s_tag, (uint32_t)v * n_keys + (uint32_t)bin_key(g, r.u, r.v));
                if (s >= 0) atomicAdd(s_cnt + s, 1u);
            }
        }
        __syncthreads();
        // ---- one returning atomic per key reserves the ticket's range of that key's entries ----
        for (int k = threadIdx.x; k < kHotSlots; k += kBinThreads)
            if (s_tag[k] != kHotEmpty)
            {
                s_base[k] = atomicAdd(cursors + s_tag[k], s_cnt[k]);
                s_cnt[k]  = 0u;
            }
        __syncthreads();
        // ---- the same point-views again (the same arithmetic, hence the same keys): slots from the table, entries out ----
        for (int i = first + threadIdx.x; i < last; i += kBinThreads)
        {
            PointRow<C> d;
            d.tex    = sc.index ? __ldg(sc.index + i) : i;
            d.tex_ok = (unsigned)d.tex < (unsigned)sc.n_tex;
            if (discarded_for_confidence<ACT>(sc, pr, d.tex)) continue;
            const float4 p  = __ldg(sc.position + i);
            const float raw = __ldg(sc.point_size + i);
            float sp        = -1.f;
            for (int v = 0; v < nv; ++v)
            {
                if ((no_room >> v) & 1u) continue;  // uniform
                if (use_dropout && __ldg(sc.dropout + (size_t)(v0 + v) * sc.N + i) == 1.f) continue;
                const Projected r = project_visible(s_cam[v], g, pr, p, raw, sp);
                if (!r.ok) continue;
                fetch_point_row<C, ACT>(sc, pr, fb, i, d);
                const uint32_t key  = (uint32_t)v * n_keys + (uint32_t)bin_key(g, r.u, r.v);
                const int s         = hot_find(s_tag, key);
                const uint32_t slot = s >= 0 ? s_base[s] + atomicAdd(s_cnt + s, 1u) : atomicAdd(cursors + key, 1u);
                write_entry<C>(fb, g, pr, s_ebase[v] + slot, i, p, raw, r, d);
            }
        }
    }
}

// Count pass of the binning stage: bounding boxes, visible points per (view, bin, tile), their exclusive scan and the
// first entry of every view.  After it fb.view_total / stats->visible say how many entries the scatter pass will write.
cudaError_t launch_bin_count(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr, int B,
                             const FwdBuffers& fb, unsigned long long entry_cap, bool hot, int sm_count, cudaStream_t st)
{
    const int n_keys   = g.n_bins << kSubShift;
    const int grid     = sm_count * kBinBlocksPerSM;
    const int n_groups = (B + kViewGroup - 1) / kViewGroup;
    cudaError_t e      = cudaMemsetAsync(fb.bin_count, 0, sizeof(uint32_t) * (size_t)B * n_keys, st);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(fb.ticket, 0, 2 * n_groups * sizeof(unsigned), st);  // one counter per pass and view group
    if (e != cudaSuccess) return e;
    if (sc.N > 0 && fb.block_box && fb.block_skip)
    {
        const int nbk = (sc.N + kBinChunk - 1) / kBinChunk;
        block_box_kernel<<<nbk, 256, 0, st>>>(sc.position, sc.N, const_cast<float*>(fb.block_box));
        block_visibility_kernel<<<(B * nbk + 127) / 128, 128, 0, st>>>(cams, g, B, nbk, fb.block_box, const_cast<uint8_t*>(fb.block_skip), fb.stats);
    }
    const bool act = pr.confidence_is_raw || pr.texture_abs;
    if (sc.N > 0)
        for (int gi = 0; gi < n_groups; ++gi)
        {
            const int v0 = gi * kViewGroup, nv = min(kViewGroup, B - v0);
            if (hot && act)
                bin_count_hot_kernel<true><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, fb.ticket + gi);
            else if (hot)
                bin_count_hot_kernel<false><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, fb.ticket + gi);
            else if (act)
                bin_count_kernel<true><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, fb.ticket + gi);
            else
                bin_count_kernel<false><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, fb.ticket + gi);
        }
    bin_scan_kernel<<<B, 1024, 0, st>>>(fb.bin_count, fb.bin_base, fb.bin_cursor, n_keys, 1, fb.view_total, kSubShift, fb.stats);
    entry_base_kernel<<<1, 32, 0, st>>>(fb.view_total, B, entry_cap, fb.entry_base, fb.stats);
    return cudaGetLastError();
}

int bin_count_launches(int N, int B) { return 2 + (N > 0 ? 2 + (B + kViewGroup - 1) / kViewGroup : 0); }
int bin_scatter_launches(int N, int B) { return N > 0 ? (B + kViewGroup - 1) / kViewGroup : 0; }

// Scatter pass of the binning stage: writes the entries (the arrays must hold fb.entry_base[B] entries).
cudaError_t launch_bin_scatter(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr, int B,
                               const FwdBuffers& fb, bool hot, int sm_count, cudaStream_t st)
{
    if (sc.N <= 0) return cudaSuccess;
    const int grid     = sm_count * kBinBlocksPerSM;
    const int n_groups = (B + kViewGroup - 1) / kViewGroup;
    const bool act     = pr.confidence_is_raw || pr.texture_abs;
    for (int gi = 0; gi < n_groups; ++gi)
    {
        const int v0 = gi * kViewGroup, nv = min(kViewGroup, B - v0);
        unsigned* tk = fb.ticket + n_groups + gi;
#define TRIPS_SCATTER_CASE(CC)                                                                                    \
    case CC:                                                                                                      \
        if (hot && act)                                                                                           \
            bin_scatter_hot_kernel<CC, true><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, tk);     \
        else if (hot)                                                                                             \
            bin_scatter_hot_kernel<CC, false><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, tk);    \
        else if (act)                                                                                             \
            bin_scatter_kernel<CC, true><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, tk);         \
        else                                                                                                      \
            bin_scatter_kernel<CC, false><<<grid, kBinThreads, 0, st>>>(sc, cams, g, pr, fb, v0, nv, tk);        \
        break;
        switch (sc.C)
        {
            TRIPS_SCATTER_CASE(3)
            TRIPS_SCATTER_CASE(4)
            TRIPS_SCATTER_CASE(6)
            TRIPS_SCATTER_CASE(8)
            TRIPS_SCATTER_CASE(16)
            default: return cudaErrorInvalidValue;
        }
#undef TRIPS_SCATTER_CASE
    }
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// exclusive scan of the list lengths of every view (three small kernels, no spin-waits)
// ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v, int lane)
{
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
    {
        uint32_t t = __shfl_up_sync(kFull, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// block of 256 threads: exclusive scan of one value per thread, returns the block total through `total`
__device__ __forceinline__ uint32_t block_excl_scan_256(uint32_t v, uint32_t* smem /*[8]*/, uint32_t& total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc   = warp_incl_scan(v, lane);
    if (lane == 31) smem[warp] = inc;
    __syncthreads();
    uint32_t wsum = (lane < 8) ? smem[lane] : 0;
    uint32_t winc = warp_incl_scan(wsum, lane);
    total         = __shfl_sync(kFull, winc, 7);
    uint32_t woff = __shfl_sync(kFull, winc - wsum, warp);
    __syncthreads();
    return woff + inc - v;
}

__global__ __launch_bounds__(256) void scan_reduce_kernel(const uint32_t* __restrict__ counts, int P, int nchunks, int k_keep,
                                                          uint32_t* __restrict__ partial, DevStats* stats, uint2* __restrict__ heavy)
{
    __shared__ uint32_t sm[8];
    const int b           = blockIdx.y;
    const uint32_t* c     = counts + (size_t)b * P;
    const int start       = blockIdx.x * kScanChunk + threadIdx.x * 8;
    uint32_t sum = 0, kept = 0, mx = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k)
    {
        int i      = start + k;
        uint32_t v = (i < P) ? c[i] : 0u;
        sum += v;
        kept += min(v, (uint32_t)k_keep);
        mx = max(mx, v);
        if (v > (uint32_t)kHeavyList)  // a list worth a block of its own (heavy_topk_kernel); rare
        {
            const unsigned slot = atomicAdd(&stats->n_heavy, 1u);
            if (slot < (unsigned)kHeavyCap) heavy[slot] = make_uint2((unsigned)b, (unsigned)i);
        }
    }
    uint32_t total;
    block_excl_scan_256(sum, sm, total);
    uint32_t kept_total;
    block_excl_scan_256(kept, sm, kept_total);
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(kFull, mx, o));
    if ((threadIdx.x & 31) == 0 && mx) atomicMax(&stats->max_len, mx);
    if (threadIdx.x == 0)
    {
        partial[(size_t)b * nchunks + blockIdx.x] = total;
        if (kept_total) atomicAdd(&stats->kept, (unsigned long long)kept_total);
    }
}

// one block: per view, exclusive scan of the chunk totals in place; view_base = running 64-bit fragment offset
__global__ __launch_bounds__(1024) void scan_partials_kernel(uint32_t* __restrict__ partial, int nchunks, int B,
                                                             unsigned long long* __restrict__ view_base,
                                                             unsigned long long frag_cap, DevStats* stats)
{
    __shared__ uint32_t sm[32];
    __shared__ uint32_t carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long base = 0, need = 0;
    for (int b = 0; b < B; ++b)
    {
        uint32_t* p = partial + (size_t)b * nchunks;
        if (threadIdx.x == 0) carry_s = 0;
        __syncthreads();
        for (int s = 0; s < nchunks; s += 1024)
        {
            int i        = s + threadIdx.x;
            uint32_t v   = (i < nchunks) ? p[i] : 0u;
            uint32_t inc = warp_incl_scan(v, lane);
            if (lane == 31) sm[warp] = inc;
            __syncthreads();
            uint32_t wsum = sm[lane];
            uint32_t winc = warp_incl_scan(wsum, lane);
            uint32_t tot  = __shfl_sync(kFull, winc, 31);
            uint32_t woff = __shfl_sync(kFull, winc - wsum, warp);
            uint32_t carry = carry_s;
            if (i < nchunks) p[i] = carry + woff + inc - v;
            __syncthreads();
            if (threadIdx.x == 0) carry_s = carry + tot;
            __syncthreads();
        }
        if (threadIdx.x == 0)
        {
            // a view that does not fit the list buffer (sized from the previous call) gets no fragments at all: the
            // collect pass skips it and the blend treats its lists as empty
            view_base[b] = base;
            need += carry_s;
            if (base + carry_s <= frag_cap)
                base += carry_s;
            else
                atomicOr(&stats->status, TRIPS_DEV_FRAGMENT_OVERFLOW);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0)
    {
        view_base[B]     = base;
        stats->frag_need = need;
    }
}

__global__ __launch_bounds__(256) void scan_apply_kernel(const uint32_t* __restrict__ counts, int P, int nchunks,
                                                         const uint32_t* __restrict__ partial, uint32_t* __restrict__ offsets)
{
    __shared__ uint32_t sm[8];
    const int b       = blockIdx.y;
    const uint32_t* c = counts + (size_t)b * P;
    uint32_t* o       = offsets + (size_t)b * P;
    const int start   = blockIdx.x * kScanChunk + threadIdx.x * 8;
    uint32_t v[8];
    uint32_t sum = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k)
    {
        int i = start + k;
        v[k]  = (i < P) ? c[i] : 0u;
        sum += v[k];
    }
    uint32_t total;
    uint32_t run = block_excl_scan_256(sum, sm, total) + partial[(size_t)b * nchunks + blockIdx.x];
#pragma unroll
    for (int k = 0; k < 8; ++k)
    {
        int i = start + k;
        if (i < P) o[i] = run;
        run += v[k];
    }
}

cudaError_t launch_scan(const Geom& g, int B, int k_keep, const FwdBuffers& fb, int nchunks, cudaStream_t st)
{
    scan_reduce_kernel<<<dim3(nchunks, B), 256, 0, st>>>(fb.counts, g.P, nchunks, k_keep, fb.partial, fb.stats, fb.heavy);
    scan_partials_kernel<<<1, 1024, 0, st>>>(fb.partial, nchunks, B, fb.view_base, fb.frag_cap, fb.stats);
    scan_apply_kernel<<<dim3(nchunks, B), 256, 0, st>>>(fb.counts, g.P, nchunks, fb.partial, fb.offsets);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// count and collect: fragments into per-pixel lists, with the list counters of a screen bin held in shared memory
//
// Entries are in bin order, and every fragment of a bin's points lands inside the bin's window: on layer l the
// pixels [x0, x0 + w_l) x [y0, y0 + w_l) with x0 = (32 bx) >> l and w_l = (31 >> l) + 3 (the 2x2 footprint adds one
// pixel).  A block takes a chunk of consecutive entries, and for each bin the chunk touches it
//   count pass:   counts the fragments per window pixel with shared-memory atomics and adds every non-zero window
//                 counter to the global list length once;
//   collect pass: counts the same way, reserves for each window pixel a contiguous range of its list with ONE
//                 returning global atomic, then hands out slots inside the ranges with shared-memory atomics and
//                 writes the 16-byte fragments: the 64-bit sort key (depth bits << 32 | point id), alpha and the
//                 entry index.
// This replaces one global atomic per fragment (SplattingPass, RenderForward.cu:368-436, and the counting half of
// CountAndCollectTiled, :347-362) by one per (chunk, touched pixel).  alpha = bilinear * confidence * layer factor
// in the operation order of FastSortFusedNew (RenderForward.cu:882-899) is computed here, where every thread holds
// a whole point, and travels with the fragment.
// ------------------------------------------------------------------------------------------------------------
constexpr int kWinChunkCount   = 4096;  // entries per block ticket, counting pass
constexpr int kWinSparse       = 512;   // entries of a bin up to which the window of shared-memory counters is bypassed
constexpr int kWinChunkCountFew = 1024;  // the same when the call has too few entries for kWinTicketsPerBlock tickets of 4096 per resident block:
constexpr int kWinTicketsPerBlock = 6;   // measured count pass, tickets of 4096 / 1024: config 4 (2 views, 16 M entries) 0.58 / 0.25 ms, config 2
                                         // (4 M) 0.093 / 0.09 ms; config 3 (27 M) 0.31 / 0.52 ms, config 5 (39 M) 0.40 / 0.53 ms
constexpr int kWinChunkCollect = 1024;  // and collecting pass: the lists a chunk writes to must stay in L2 until complete (measured with tile-ordered entries: 256 1.80 ms, 512 1.46 ms, 1024 1.35 ms, 2048 1.47 ms)
constexpr int kWinThreads    = 256;
constexpr int kWinBlocksPerSM = 8;  // grid size of the window kernels, in blocks per SM
constexpr int kWinMinBlocks  = 5;  // resident blocks the register allocation leaves room for
constexpr int kWinMax     = 34 * 34 + 18 * 18 + 10 * 10 + 6 * 6 + 4 * 4 + 3 * 3 * 3;  // 1659 window pixels over 8 layers

// Window of a bin: on layer l it starts at ((32 bx) >> l, (32 by) >> l) and is win_w(l) pixels wide; the counters of
// the layers follow one another in shared memory.  Everything is computed from (bx32, by32) with shifts and selects:
// arrays indexed by the layer would live in local memory.
struct Window
{
    int bx32, by32;
    __device__ __forceinline__ int x0(int l) const { return bx32 >> l; }
    __device__ __forceinline__ int y0(int l) const { return by32 >> l; }
};

__device__ __forceinline__ int win_w(int l) { return (31 >> l) + 3; }

// first counter of layer l: sum of win_w(k)^2 over k < l = 0, 1156, 1480, 1580, 1616, 1632, 1641, 1650, 1659
__device__ __forceinline__ int win_off(int l)
{
    return l < 4 ? (l < 2 ? (l == 0 ? 0 : 1156) : (l == 2 ? 1480 : 1580)) : (l < 6 ? (l == 4 ? 1616 : 1632) : (l == 6 ? 1641 : (l == 7 ? 1650 : 1659)));
}

__device__ __forceinline__ Window make_window(const Geom& g, int bin)
{
    Window w;
    const int by = bin / g.bins_x, bx = bin - by * g.bins_x;
    w.bx32 = bx << kBinShift;
    w.by32 = by << kBinShift;
    return w;
}

// window counter -> global pixel index of the view, -1 if outside the layer
__device__ __forceinline__ int window_pixel(const Geom& g, const Window& w, int i)
{
    int l = 0;
#pragma unroll
    for (int k = 1; k < TRIPS_MAX_LAYERS; ++k)
        if (i >= win_off(k)) l = k;
    const int r  = i - win_off(l);
    const int ww = win_w(l);
    const int dy = r / ww, dx = r - dy * ww;
    const int x = w.x0(l) + dx, y = w.y0(l) + dy;
    return (l < g.L && x < g.W[l] && y < g.H[l]) ? g.base[l] + y * g.W[l] + x : -1;
}

// the chunk [c0, c1) of the view's entries and the first bin it touches; false when the view has no more chunks
__device__ __forceinline__ bool next_chunk(const FwdBuffers& fb, const Geom& g, int b, uint32_t n_entry, uint32_t* s_tmp, int kWinChunk,
                                           uint32_t& c0, uint32_t& c1, int& first_bin)
{
    __syncthreads();
    if (threadIdx.x == 0)
    {
        const uint32_t t = atomicAdd(fb.ticket + b, 1u);
        uint32_t lo      = (uint32_t)min((unsigned long long)t * kWinChunk, (unsigned long long)n_entry);
        s_tmp[0]         = lo;
        // last bin whose first entry is <= lo (empty bins share their first entry with the next non-empty one)
        const uint32_t* bf = fb.bin_cursor + (size_t)b * g.n_bins;
        int a = 0, z = g.n_bins;  // invariant: bf[a] <= lo
        while (z - a > 1)
        {
            const int mid = (a + z) >> 1;
            if (bf[mid] <= lo)
                a = mid;
            else
                z = mid;
        }
        s_tmp[1] = (uint32_t)a;
    }
    __syncthreads();
    c0        = s_tmp[0];
    first_bin = (int)s_tmp[1];
    c1        = min(n_entry, c0 + (uint32_t)kWinChunk);
    return c0 < n_entry;
}


// Calls body(e0, e1, x, y, layer, entry) for every (entry, layer) pair of the entries [lo, hi), with (x, y) the entry's
// position on that layer.  A warp takes 32 entries at a time: layer 0 directly (every entry has it), the higher layers
// through a per-warp queue of (lane, layer) items that all 32 lanes drain together, so that an entry with many layers
// does not hold up the 31 other lanes.  WITH_E1 = false: body only needs x, y, layer.
// First layer of an entry written by the strict two-layer rule: the layer below log2(size), as write_entry computed it.
__device__ __forceinline__ int strict_first_layer(float ps, int L) { return ps > 1.f ? min(tm_floor_log2(ps), L - 1) : 0; }

template <bool WITH_E1, bool STRICT, class Body>
__device__ __forceinline__ void for_each_footprint(const float4* __restrict__ head, uint32_t lo, uint32_t hi, uint8_t* queue, int L, Body&& body)
{
    const int lane = threadIdx.x & 31;
    uint32_t base  = lo + (threadIdx.x & ~31);
    float4 e0n = make_float4(0.f, 0.f, 0.f, 0.f), e1n = e0n;
    if (base + lane < hi)
    {
        e0n = head[2 * (size_t)(base + lane)];      // u v ps conf
        e1n = head[2 * (size_t)(base + lane) + 1];  // pid z raw nl|rank
    }
    for (; base < hi; base += kWinThreads)
    {
        const uint32_t ei = base + lane;
        const float4 e0 = e0n, e1 = e1n;
        const int nl = ei < hi ? (__float_as_int(e1.w) & ((1 << kRankShift) - 1)) : 0;
        if (base + kWinThreads + lane < hi)  // the next round's entry travels while this one is processed
        {
            e0n = head[2 * (size_t)(ei + kWinThreads)];
            e1n = head[2 * (size_t)(ei + kWinThreads) + 1];
        }
        int first = 0;
        if constexpr (STRICT)
        {
            first = strict_first_layer(e0.z, L);
            const float sc = __int_as_float((127 - first) << 23);
            if (nl > 0) body(e0, e1, e0.x * sc, e0.y * sc, first, ei);
        }
        else if (nl > 0)
            body(e0, e1, e0.x, e0.y, 0, ei);
        const int extra = max(nl - 1, 0);
        int incl = extra;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            const int t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        const int total = __shfl_sync(kFull, incl, 31);
        if (total == 0) continue;  // uniform
        int pos = incl - extra;
        for (int l = 1; l < nl; ++l) queue[pos++] = (uint8_t)(lane | ((first + l) << 5));
        __syncwarp();
        for (int i0 = 0; i0 < total; i0 += 32)
        {
            const int i        = i0 + lane;
            const unsigned it  = i < total ? queue[i] : 0u;
            const int src = it & 31, layer = it >> 5;
            float4 s0, s1 = make_float4(0.f, 0.f, 0.f, 0.f);
            s0.x = __shfl_sync(kFull, e0.x, src);
            s0.y = __shfl_sync(kFull, e0.y, src);
            s0.z = s0.w = 0.f;
            if (WITH_E1)
            {
                s0.z = __shfl_sync(kFull, e0.z, src);
                s0.w = __shfl_sync(kFull, e0.w, src);
                s1.x = __shfl_sync(kFull, e1.x, src);
                s1.y = __shfl_sync(kFull, e1.y, src);
            }
            if (i < total)
            {
                const float sc = __int_as_float((127 - layer) << 23);  // 2^-layer: the same value as `layer` halvings
                body(s0, s1, s0.x * sc, s0.y * sc, layer, base + src);
            }
        }
        __syncwarp();
    }
}


// 16-byte store that asks L2 to keep the line: a pixel's list is written 16 bytes at a time by many threads, and a
// sector that leaves L2 half written costs a read-modify-write in DRAM.
__device__ __forceinline__ void store_frag(uint4* p, const uint4& v, uint64_t policy)
{
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t evict_last_policy()
{
    uint64_t policy = 0;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// A bin with few entries inside a ticket (sky, far ground: a ticket can span hundreds of such bins) is not worth clearing
// and flushing a window of shared-memory counters with three block barriers: its footprints go straight to the pixels'
// global counters.  (On a 2560x1440 view of 20 M points with half of the bins nearly empty, the blocks that drew the
// sparse tickets ran 12 times longer than the others.)  Not inlined: the dense path keeps its registers.
template <bool COLLECT, bool STRICT>
__device__ __noinline__ void sparse_bin_footprints(const Geom& g, const float4* __restrict__ head, uint32_t lo, uint32_t hi, uint8_t* queue,
                                                   uint32_t* pixel_ctr, uint4* frags, uint64_t keep)
{
    for_each_footprint<COLLECT, STRICT>(head, lo, hi, queue, g.L, [&](const float4& e0, const float4& e1, float x, float y, int layer, uint32_t ei) {
        const int px = __float2int_rd(x), py = __float2int_rd(y);
        const int Wl = g.W[layer];
        uint32_t* c  = pixel_ctr + g.base[layer] + py * Wl + px;
        if constexpr (!COLLECT)
        {
            atomicAdd(c, 1u);
            atomicAdd(c + 1, 1u);
            atomicAdd(c + Wl, 1u);
            atomicAdd(c + Wl + 1, 1u);
        }
        else
        {
            const float conf   = e0.w;
            const uint32_t pid = __float_as_uint(e1.x), zb = __float_as_uint(e1.y);
            const float lf  = layer_factor(e0.z, layer, g.L, nullptr);
            const float dx0 = fabsf(x - (float)px), dx1 = fabsf(x - (float)(px + 1));
            const float dy0 = fabsf(y - (float)py), dy1 = fabsf(y - (float)(py + 1));
            auto alpha = [&](float dx, float dy) {
                float bl = (1.f - dx) * (1.f - dy);
                if (dx > 1.f || dy > 1.f) bl = 0.f;
                float a = bl * conf;
                a *= lf;
                return __float_as_uint(a);
            };
            const uint32_t s00 = atomicAdd(c, 1u);
            const uint32_t s10 = atomicAdd(c + 1, 1u);
            const uint32_t s01 = atomicAdd(c + Wl, 1u);
            const uint32_t s11 = atomicAdd(c + Wl + 1, 1u);
            store_frag(frags + s00, make_uint4(pid, zb, alpha(dx0, dy0), ei), keep);
            store_frag(frags + s10, make_uint4(pid, zb, alpha(dx1, dy0), ei), keep);
            store_frag(frags + s01, make_uint4(pid, zb, alpha(dx0, dy1), ei), keep);
            store_frag(frags + s11, make_uint4(pid, zb, alpha(dx1, dy1), ei), keep);
        }
    });
}

template <bool COLLECT, bool STRICT>
__global__ __launch_bounds__(kWinThreads, kWinMinBlocks) void window_kernel(const __grid_constant__ Geom g, FwdBuffers fb, int B, int chunk)
{
    __shared__ uint32_t s_cnt[kWinMax];
    __shared__ uint32_t s_base[COLLECT ? kWinMax : 1];
    __shared__ uint32_t s_tmp[2];
    const uint64_t keep = evict_last_policy();
    __shared__ uint8_t s_queue[kWinThreads / 32][32 * (TRIPS_MAX_LAYERS - 1)];
    // all blocks walk the views in the same order: the lists, counters and entries in flight belong to one view (or two,
    // where blocks cross over), which keeps the partially written list sectors of a view in L2 until they are complete
    for (int b = 0; b < B; ++b)
    {
    if (COLLECT && fb.view_base[b + 1] == fb.view_base[b]) continue;  // no fragments, or the view did not fit the list buffer (status bit raised by the scan)
    uint32_t* pixel_ctr   = (COLLECT ? fb.offsets : fb.counts) + (size_t)b * g.P;
    uint4* frags          = fb.frags + fb.view_base[COLLECT ? b : 0];
    const uint32_t n_entry = (uint32_t)(fb.entry_base[b + 1] - fb.entry_base[b]);
    const float4* head     = fb.ent_head + fb.entry_base[b] * 2;
    const uint32_t* bfirst = fb.bin_cursor + (size_t)b * g.n_bins;
    uint32_t c0, c1;
    int bin;
    while (next_chunk(fb, g, b, n_entry, s_tmp, chunk, c0, c1, bin))
    {
        for (; bin < g.n_bins && bfirst[bin] < c1; ++bin)
        {
            const uint32_t bin_end = (bin + 1 < g.n_bins) ? bfirst[bin + 1] : n_entry;
            const uint32_t lo = max(c0, bfirst[bin]), hi = min(c1, bin_end);
            if (lo >= hi) continue;  // uniform: all threads read the same values
            if (bin_end - bfirst[bin] <= (uint32_t)kWinSparse)  // the whole bin is sparse (a short piece of a dense bin still pays off in the window)
            {
                sparse_bin_footprints<COLLECT, STRICT>(g, head, lo, hi, s_queue[threadIdx.x >> 5], pixel_ctr, frags, keep);
                continue;
            }
            const Window w = make_window(g, bin);
            const int n_win = win_off(g.L);
            for (int i = threadIdx.x; i < n_win; i += kWinThreads) s_cnt[i] = 0;
            __syncthreads();
            // ---- fragments per window pixel ----
            for_each_footprint<false, STRICT>(head, lo, hi, s_queue[threadIdx.x >> 5], g.L,
                                      [&](const float4&, const float4&, float x, float y, int layer, uint32_t) {
                                          const int ww = win_w(layer);
                                          uint32_t* c  = s_cnt + win_off(layer) + (__float2int_rd(y) - w.y0(layer)) * ww + (__float2int_rd(x) - w.x0(layer));
                                          atomicAdd(c, 1u);
                                          atomicAdd(c + 1, 1u);
                                          atomicAdd(c + ww, 1u);
                                          atomicAdd(c + ww + 1, 1u);
                                      });
            __syncthreads();
            // ---- one global atomic per touched pixel ----
            for (int i = threadIdx.x; i < n_win; i += kWinThreads)
            {
                const uint32_t c = s_cnt[i];
                if (c)
                {
                    const int pix = window_pixel(g, w, i);
                    if (COLLECT)
                    {
                        s_base[i] = (pix >= 0) ? atomicAdd(pixel_ctr + pix, c) : 0u;
                        s_cnt[i]  = 0;
                    }
                    else if (pix >= 0)
                        atomicAdd(pixel_ctr + pix, c);
                }
            }
            __syncthreads();
            if (COLLECT)
            {
                // ---- slots inside the reserved ranges; alpha and the fragment itself ----
                for_each_footprint<true, STRICT>(head, lo, hi, s_queue[threadIdx.x >> 5], g.L,
                                         [&](const float4& e0, const float4& e1, float x, float y, int layer, uint32_t ei) {
                                             // x, y equal (u, v) * 2^-layer exactly (power-of-two scaling)
                                             const float conf   = e0.w;
                                             const uint32_t pid = __float_as_uint(e1.x), zb = __float_as_uint(e1.y);
                                             const int px = __float2int_rd(x), py = __float2int_rd(y);
                                             const int ww = win_w(layer);
                                             const int li = win_off(layer) + (py - w.y0(layer)) * ww + (px - w.x0(layer));
                                             const float lf  = layer_factor(e0.z, layer, g.L, nullptr);
                                             const float dx0 = fabsf(x - (float)px), dx1 = fabsf(x - (float)(px + 1));
                                             const float dy0 = fabsf(y - (float)py), dy1 = fabsf(y - (float)(py + 1));
                                             auto alpha = [&](float dx, float dy) {
                                                 float bl = (1.f - dx) * (1.f - dy);
                                                 if (dx > 1.f || dy > 1.f) bl = 0.f;
                                                 float a = bl * conf;
                                                 a *= lf;
                                                 return __float_as_uint(a);
                                             };
                                             // the four slots first, then the four stores: the shared-memory atomics do not wait for one another
                                             const uint32_t s00 = s_base[li] + atomicAdd(s_cnt + li, 1u);
                                             const uint32_t s10 = s_base[li + 1] + atomicAdd(s_cnt + li + 1, 1u);
                                             const uint32_t s01 = s_base[li + ww] + atomicAdd(s_cnt + li + ww, 1u);
                                             const uint32_t s11 = s_base[li + ww + 1] + atomicAdd(s_cnt + li + ww + 1, 1u);
                                             store_frag(frags + s00, make_uint4(pid, zb, alpha(dx0, dy0), ei), keep);
                                             store_frag(frags + s10, make_uint4(pid, zb, alpha(dx1, dy0), ei), keep);
                                             store_frag(frags + s01, make_uint4(pid, zb, alpha(dx0, dy1), ei), keep);
                                             store_frag(frags + s11, make_uint4(pid, zb, alpha(dx1, dy1), ei), keep);
                                         });
                __syncthreads();  // the next bin of this chunk reuses s_cnt / s_base
            }
        }
    }
    }
}

cudaError_t launch_count(const ScenePtrs& sc, const Geom& g, int B, const FwdBuffers& fb, bool strict, unsigned long long entries_hint, int sm_count,
                         cudaStream_t st)
{
    cudaError_t e = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned) * B, st);
    if (e != cudaSuccess) return e;
    // entries_hint: the number of entries of the call as far as the host knows it (the previous call's, or this call's own count)
    const bool few  = entries_hint / kWinChunkCount < (unsigned long long)kWinTicketsPerBlock * sm_count * kWinMinBlocks;
    const int chunk = few ? kWinChunkCountFew : kWinChunkCount;
    if (strict)
        window_kernel<false, true><<<sm_count * kWinBlocksPerSM, kWinThreads, 0, st>>>(g, fb, B, chunk);
    else
        window_kernel<false, false><<<sm_count * kWinBlocksPerSM, kWinThreads, 0, st>>>(g, fb, B, chunk);
    return cudaGetLastError();
}

cudaError_t launch_collect(const ScenePtrs& sc, const Geom& g, int B, const FwdBuffers& fb, bool strict, int sm_count, cudaStream_t st)
{
    cudaError_t e = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned) * B, st);
    if (e != cudaSuccess) return e;
    if (strict)
        window_kernel<true, true><<<sm_count * kWinBlocksPerSM, kWinThreads, 0, st>>>(g, fb, B, kWinChunkCollect);
    else
        window_kernel<true, false><<<sm_count * kWinBlocksPerSM, kWinThreads, 0, st>>>(g, fb, B, kWinChunkCollect);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// per-pixel top-K selection + front-to-back blend
//
// One warp renders an 8x4 pixel tile of one view.
//   phase A (lane = fragment, lanes densely packed over the tile's fragments): every fragment finds its pixel by a
//     binary search over the tile's list lengths and its rank in the pixel's list by counting the smaller 64-bit
//     keys; ranks below K go to shared memory in sorted order together with the descriptor row of their entry (and,
//     when training, to the backward records).  Lists longer than kRankMax take the streaming path instead: a
//     half-warp keeps the 16 nearest fragments in registers and merges the list in chunks of 16 with bitonic
//     compare-exchange steps over warp shuffles.
//   phase B (lane = pixel): the sequential transmittance recurrence and the colour sum over the kept fragments.
// Replaces FastSortFusedNew (RenderForward.cu:474-1059).
// ------------------------------------------------------------------------------------------------------------
typedef unsigned long long u64;
constexpr u64 kInfKey    = 0xffffffffffffffffull;
constexpr int kSbRing    = 2;    // descriptor rows requested ahead of their use in the blend loop (C <= 4)
constexpr int kRankMax   = 32;   // longest list ranked by counting; longer lists use the streaming path (measured: 16 3.12 ms, 24 3.03, 32 3.02, 48 3.08, 64 3.15)
constexpr int kSortedPad = 17;   // row pitch (entries) of the per-pixel sorted lists in shared memory
constexpr int kSbStageMaxC = 0;  // widest descriptor whose rows are staged in shared memory by phase A (0: none; staging cost more L1 than it saved)
constexpr int kSbThreads = 128;
constexpr int kSbWarps   = kSbThreads / 32;

struct KeyVal
{
    u64 key;
    uint32_t alpha;
    uint32_t eidx;
};

__device__ __forceinline__ KeyVal cmpx(KeyVal v, int j_mask, bool keep_min)
{
    KeyVal o;
    o.key         = __shfl_xor_sync(kFull, v.key, j_mask);
    o.alpha       = __shfl_xor_sync(kFull, v.alpha, j_mask);
    o.eidx        = __shfl_xor_sync(kFull, v.eidx, j_mask);
    const bool lt = v.key < o.key;
    return (lt == keep_min) ? v : o;
}

// ascending bitonic sort of 16 fragments held one per lane by each half-warp (10 compare-exchange steps)
__device__ __forceinline__ KeyVal bitonic_sort16(KeyVal v, int j)
{
#pragma unroll
    for (int k = 2; k <= 16; k <<= 1)
    {
#pragma unroll
        for (int s = k >> 1; s > 0; s >>= 1)
        {
            const bool up    = ((j & k) == 0) || (k == 16);
            const bool lower = (j & s) == 0;
            v                = cmpx(v, s, lower == up);
        }
    }
    return v;
}

// a bitonic sequence of 16 fragments -> ascending (4 steps)
__device__ __forceinline__ KeyVal bitonic_merge16(KeyVal v, int j)
{
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) v = cmpx(v, s, (j & s) == 0);
    return v;
}

// Merges a chunk of up to 16 fragments (one per lane of a half-warp, unsorted, kInfKey = absent) into the ascending
// top-16 `v` the half-warp keeps.  Both half-warps of a warp must call this together (full-mask shuffles).
__device__ __forceinline__ void topk_merge16(KeyVal& v, KeyVal nk, int j, int hbase)
{
    const u64 cur_max = __shfl_sync(kFull, v.key, hbase | 15);
    if (__ballot_sync(kFull, nk.key < cur_max) == 0) return;  // nothing nearer in either half
    nk = bitonic_sort16(nk, j);
    KeyVal rev;
    rev.key   = __shfl_sync(kFull, nk.key, hbase | (15 - j));
    rev.alpha = __shfl_sync(kFull, nk.alpha, hbase | (15 - j));
    rev.eidx  = __shfl_sync(kFull, nk.eidx, hbase | (15 - j));
    if (rev.key < v.key) v = rev;
    v = bitonic_merge16(v, j);
}

// Pre-selection of very long lists.  A pixel list of thousands of fragments (many points projected into a few pixels)
// would keep one half-warp of the blend kernel busy on its own while the rest of the machine idles.  Here a block of
// 256 threads takes one such list: its 16 half-warps each select the 16 nearest fragments of a sixteenth of the list
// (the streaming bitonic top-16 of the blend kernel), one half-warp merges the 256 candidates, and the 16 winners are
// moved to the front of the list in depth order by swapping them with the fragments that were there - the list stays
// the same set of fragments.  The blend kernel then reads only the first 16 entries of every list longer than
// kHeavyList.  Lists are found by the scan (scan_reduce_kernel); with more than kHeavyCap of them nothing is done here
// and the blend kernel, which sees the same counter, walks them itself.
__global__ __launch_bounds__(256) void heavy_topk_kernel(const __grid_constant__ Geom g, FwdBuffers fb, int B)
{
    __shared__ u64 s_key[16][16];
    __shared__ uint32_t s_pos[16][16];
    __shared__ uint32_t s_vac[16];
    const unsigned n_heavy = fb.stats->n_heavy;
    if (n_heavy == 0 || n_heavy > (unsigned)kHeavyCap) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, j = lane & 15, hbase = lane & 16, hw = threadIdx.x >> 4;
    for (unsigned h = blockIdx.x; h < n_heavy; h += gridDim.x)
    {
        const uint2 e = fb.heavy[h];
        const int b   = (int)e.x;
        if (b >= B || fb.view_base[b + 1] == fb.view_base[b]) continue;  // uniform: the view did not fit the list buffer
        const size_t bP    = (size_t)b * g.P;
        const uint32_t cnt = fb.counts[bP + e.y];
        uint4* list        = fb.frags + fb.view_base[b] + (fb.offsets[bP + e.y] - cnt);  // offsets hold list ends after the collect pass
        const uint32_t n_chunks = (cnt + 15) / 16, per = (n_chunks + 15) / 16;
        const uint32_t c0 = hw * per, c1 = min(n_chunks, c0 + per);
        KeyVal v;
        v.key = kInfKey, v.alpha = 0u, v.eidx = 0u;
        for (uint32_t k0 = 0; k0 < per; k0 += 4)  // the same trip count for all half-warps; four chunks of keys in flight per lane
        {
            KeyVal nk[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
            {
                const uint32_t k = k0 + q, idx = (c0 + k) * 16 + j;
                nk[q].key = kInfKey, nk[q].alpha = 0u, nk[q].eidx = 0u;
                if (k < per && c0 + k < c1 && idx < cnt)
                {
                    const uint2 kk = *reinterpret_cast<const uint2*>(list + idx);
                    nk[q].key      = ((u64)kk.y << 32) | kk.x;
                    nk[q].alpha    = idx;  // the payload is the fragment's position in the list
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) topk_merge16(v, nk[q], j, hbase);
        }
        s_key[hw][j] = v.key;
        s_pos[hw][j] = v.alpha;
        __syncthreads();
        if (warp == 0)
        {
            KeyVal w;
            w.key = kInfKey, w.alpha = 0u, w.eidx = 0u;
            for (int k = 0; k < 16; k += 2)  // each half of warp 0 merges eight of the sixteen candidate lists
            {
                const int src = k + (hbase >> 4);
                KeyVal nk;
                nk.key = s_key[src][j], nk.alpha = s_pos[src][j], nk.eidx = 0u;
                topk_merge16(w, nk, j, hbase);
            }
            {
                KeyVal nk;  // the upper half's result goes into the lower half's
                nk.key   = __shfl_sync(kFull, w.key, 16 | j);
                nk.alpha = __shfl_sync(kFull, w.alpha, 16 | j);
                nk.eidx  = 0u;
                if (hbase) nk.key = kInfKey;
                topk_merge16(w, nk, j, hbase);
            }
            // lanes 0..15 hold the 16 nearest fragments in depth order (cnt > kHeavyList >= 16: all present); swap them to the front
            const bool act    = lane < 16;
            const uint32_t wp = w.alpha;
            uint4 winner = make_uint4(0u, 0u, 0u, 0u), front = winner;
            if (act)
            {
                winner = list[wp];
                front  = list[j];
            }
            bool front_is_winner = false;
            for (int k = 0; k < 16; ++k) front_is_winner |= (__shfl_sync(kFull, wp, k) == (uint32_t)j);
            const bool displaced = act && !front_is_winner;  // a fragment that has to leave the front
            const bool vacated   = act && wp >= 16u;         // a winner's old place outside the front
            const unsigned m_d = __ballot_sync(kFull, displaced) & 0xffffu, m_v = __ballot_sync(kFull, vacated) & 0xffffu;
            if (vacated) s_vac[__popc(m_v & ((1u << j) - 1u))] = wp;
            __syncwarp();  // every lane holds its two fragments in registers before anything is stored
            if (displaced) list[s_vac[__popc(m_d & ((1u << j) - 1u))]] = front;
            if (act) list[j] = winner;
        }
        __syncthreads();
    }
}

cudaError_t launch_heavy_topk(const Geom& g, int B, const FwdBuffers& fb, int sm_count, cudaStream_t st)
{
    heavy_topk_kernel<<<sm_count * 6, 256, 0, st>>>(g, fb, B);
    return cudaGetLastError();
}

// A sorted entry in shared memory is (alpha, descriptor row[C]) when the row fits the shared-memory budget (C <= 4:
// the gather happens in phase A where lanes are densely packed); for wider descriptors it is (entry index, alpha)
// and phase B gathers.
template <int C>
struct SbEntry
{
    static constexpr bool kStaged = (C <= kSbStageMaxC);
    static constexpr int kFloats  = kStaged ? (1 + C) : 2;
};

template <int C>
__device__ __forceinline__ void sb_store_entry(float* dst, const float* entries, unsigned eidx, unsigned alpha_bits)
{
    if constexpr (SbEntry<C>::kStaged)
    {
        const float4 v4 = *reinterpret_cast<const float4*>(entries + (size_t)eidx * tail_stride(C) + 4);
        dst[0]          = __uint_as_float(alpha_bits);
        dst[1]          = v4.x;
        if (C > 1) dst[2] = v4.y;
        if (C > 2) dst[3] = v4.z;
        if (C > 3) dst[4] = v4.w;
    }
    else
    {
        dst[0] = __uint_as_float(eidx);
        dst[1] = __uint_as_float(alpha_bits);
    }
}

// measured: 7 resident blocks (72 registers) 3.18 ms, 6 blocks (80) 3.46 ms, 5 blocks 3.83 ms, 8 blocks (64, spills) 3.76 ms
constexpr int kSbMinBlocks = 7;
template <int C>
__global__ __launch_bounds__(kSbThreads, (C <= 8 ? kSbMinBlocks : 1)) void sort_blend_kernel(ScenePtrs sc, const __grid_constant__ Geom g, TripsRenderParams pr,
                                                                int B, FwdBuffers fb, const __grid_constant__ LayerPtrs out,
                                                                unsigned n_tiles_total)
{
    constexpr int E  = SbEntry<C>::kFloats;
    constexpr int ES = tail_stride(C);
    __shared__ float s_sorted[kSbWarps][32 * kSortedPad * E];  // per warp: 32 pixels x K entries, nearest first
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K    = pr.k_keep;
    float* sorted  = s_sorted[warp];
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);

    const bool preselected = fb.stats->n_heavy <= (unsigned)kHeavyCap;  // heavy_topk_kernel handled every long list
    unsigned next_ticket = 0;
    if (lane == 0) next_ticket = atomicAdd(fb.ticket, 1u);
    for (;;)
    {
        // the ticket of the following tile is requested now, a whole tile ahead of its use
        const unsigned ticket = __shfl_sync(kFull, next_ticket, 0);
        if (ticket >= n_tiles_total) break;
        if (lane == 0) next_ticket = atomicAdd(fb.ticket, 1u);
        const int b          = ticket / (unsigned)g.n_tiles;
        const int tile       = ticket - b * (unsigned)g.n_tiles;
        const size_t bP      = (size_t)b * g.P;
        const uint4* frags   = fb.frags + fb.view_base[b];
        const float* entries = fb.ent_tail + fb.entry_base[b] * ES;  // (position, descriptor row) of the view's entries
        const uint32_t n_entry = (uint32_t)(fb.entry_base[b + 1] - fb.entry_base[b]);
        int layer, gx, gy, p;
        tile_pixel(g, tile, lane, layer, gx, gy, p);  // lane i owns one pixel of the tile
        uint32_t cnt_all = 0, start = 0;
        if (p >= 0 && fb.view_base[b + 1] != fb.view_base[b])  // (a view that did not fit the list buffer renders as background)
        {
            cnt_all = fb.counts[bP + p];
            start   = fb.offsets[bP + p] - cnt_all;  // offsets hold list ends after the collect pass
        }
        // of a pre-selected list (heavy_topk_kernel) only the front matters: its 16 nearest fragments in depth order
        const uint32_t cnt = (preselected && cnt_all > (uint32_t)kHeavyList) ? 16u : cnt_all;
        uint32_t incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            uint32_t t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        const uint32_t rel_start  = incl - cnt;
        const uint32_t tile_total = __shfl_sync(kFull, incl, 31);
        uint32_t max_cnt          = cnt;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) max_cnt = max(max_cnt, __shfl_xor_sync(kFull, max_cnt, o));

        if (max_cnt <= (uint32_t)kRankMax)
        {
            // ---- phase A, counting path: lane = fragment.  The fragment of the next round is fetched before the
            //      ranking loop of the current one, so that its DRAM latency hides behind the loop ----
            struct Loc
            {
                uint32_t seg_start, seg_cnt, idx;
                int seg, seg_p;
            };
            auto locate = [&](uint32_t t) {
                Loc L;
                // pixel of this fragment: the last lane whose list starts at or before t
                int seg = 0;
#pragma unroll
                for (int step = 16; step > 0; step >>= 1)
                {
                    const int probe       = seg + step;
                    const uint32_t pstart = __shfl_sync(kFull, rel_start, probe & 31);
                    if (probe < 32 && pstart <= t) seg = probe;
                }
                L.seg       = seg;
                L.idx       = t - __shfl_sync(kFull, rel_start, seg);
                L.seg_start = __shfl_sync(kFull, start, seg);
                L.seg_cnt   = __shfl_sync(kFull, cnt, seg);
                L.seg_p     = __shfl_sync(kFull, p, seg);
                return L;
            };
            // Rounds of whole lists: a round takes the lists of consecutive pixels as long as they fit 32 lanes (every
            // list has at most kRankMax = 32 fragments here), so the fragments of one pixel always sit in neighbouring
            // lanes of one round and a fragment finds its rank by reading the keys of its list from those lanes with
            // shuffles.  Reading the keys from the list in memory instead cost one gather over several 128-byte lines
            // per key and lane, and it was the load/store unit's line rate that bounded this kernel.
            static_assert(kRankMax <= 32, "a list ranked by shuffles must fit one round of 32 lanes");
            struct Round
            {
                uint32_t base, total;  // fragments of the tile before this round, fragments in it
                int end_px;            // first pixel (lane) of the next round
            };
            auto plan = [&](int first_px) {
                Round r;
                r.base              = __shfl_sync(kFull, rel_start, first_px & 31);
                const unsigned fits = __ballot_sync(kFull, lane >= first_px && incl - r.base <= 32u);  // a run of lanes from first_px on
                r.end_px            = first_px + __popc(fits);
                r.total             = __shfl_sync(kFull, incl, (r.end_px - 1) & 31) - r.base;
                return r;
            };
            Round rn     = plan(0);
            Loc nxt      = locate(rn.base + lane);
            uint4 f_next = make_uint4(kFull, kFull, 0u, 0u);
            if ((uint32_t)lane < rn.total) f_next = frags[nxt.seg_start + nxt.idx];
            for (;;)
            {
                const Round rc   = rn;
                const Loc cur    = nxt;
                const uint4 f    = f_next;
                const bool valid = (uint32_t)lane < rc.total;
                const bool more  = rc.end_px < 32 && rc.base + rc.total < tile_total;  // uniform
                if (more)
                {
                    rn     = plan(rc.end_px);
                    nxt    = locate(rn.base + lane);
                    f_next = make_uint4(kFull, kFull, 0u, 0u);
                    if ((uint32_t)lane < rn.total) f_next = frags[nxt.seg_start + nxt.idx];
                }
                const int lane0   = (int)(rc.base + lane - cur.idx - rc.base);  // lane of the first fragment of this fragment's list
                const int longest = __reduce_max_sync(kFull, valid ? (int)cur.seg_cnt : 0);
                const u64 mine    = ((u64)f.y << 32) | f.x;
                int rank          = 0;
                for (int i = 0; i < longest; ++i)
                {
                    const int src     = max(0, min(lane0 + i, 31));
                    const uint32_t oy = __shfl_sync(kFull, f.y, src), ox = __shfl_sync(kFull, f.x, src);
                    if (i < (int)cur.seg_cnt) rank += ((((u64)oy << 32) | ox) < mine) ? 1 : 0;
                }
                if (valid)
                {
                    if (f.w >= n_entry)
                        atomicOr(&fb.stats->status, TRIPS_DEV_BAD_FRAGMENT);  // corrupted list: skip instead of gathering out of bounds
                    else if (rank < K)
                    {
                        sb_store_entry<C>(sorted + (cur.seg * kSortedPad + rank) * E, entries, f.w, f.z);
                        if (pr.train) fb.records[(bP + cur.seg_p) * 16 + rank] = make_uint2(f.w, f.z);
                    }
                }
                if (!more) break;
            }
        }
        else
        {
            // ---- phase A, streaming path: a half-warp per pixel keeps the 16 nearest fragments in registers ----
            const int j     = lane & 15;
            const int hbase = lane & 16;
            for (int it = 0; it < 16; ++it)
            {
                const int src        = it * 2 + (hbase >> 4);
                const uint32_t cnt_s = __shfl_sync(kFull, cnt, src);
                const uint32_t beg_s = __shfl_sync(kFull, start, src);
                const int p_s        = __shfl_sync(kFull, p, src);
                const uint32_t cnt_o = __shfl_xor_sync(kFull, cnt_s, 16);
                KeyVal v;
                v.key   = kInfKey;
                v.alpha = 0u;
                v.eidx  = 0u;
                if (j < (int)cnt_s)
                {
                    const uint4 f = frags[beg_s + j];
                    v.key         = ((u64)f.y << 32) | f.x;
                    v.alpha       = f.z;
                    v.eidx        = f.w;
                }
                v = bitonic_sort16(v, j);
                const uint32_t cnt_max = max(cnt_s, cnt_o);
                for (uint32_t ch = 16; ch < cnt_max; ch += 16)
                {
                    KeyVal nk;
                    nk.key   = kInfKey;
                    nk.alpha = 0u;
                    nk.eidx  = 0u;
                    if (ch + j < cnt_s)
                    {
                        const uint4 f = frags[beg_s + ch + j];
                        nk.key        = ((u64)f.y << 32) | f.x;
                        nk.alpha      = f.z;
                        nk.eidx       = f.w;
                    }
                    topk_merge16(v, nk, j, hbase);
                }
                if (j < min((int)cnt_s, K))
                {
                    if (v.eidx >= n_entry)
                    {
                        atomicOr(&fb.stats->status, TRIPS_DEV_BAD_FRAGMENT);
                        v.eidx  = 0;
                        v.alpha = 0;
                    }
                    sb_store_entry<C>(sorted + (src * kSortedPad + j) * E, entries, v.eidx, v.alpha);
                    if (pr.train && p_s >= 0) fb.records[(bP + p_s) * 16 + j] = make_uint2(v.eidx, v.alpha);
                }
            }
        }
        __syncwarp();

        // ---- phase B: lane = pixel.  T_j = T_{j-1} * (1 - a_{j-1}), colour summed in the order of a 16-leaf
        //      butterfly (RenderForward.cu:940-994) so that results do not depend on how lanes are assigned ----
        const int n = min((int)cnt, K);
        int n_max   = n;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) n_max = max(n_max, __shfl_xor_sync(kFull, n_max, o));
        float run = 1.f, t_last = 1.f, tn_last = 1.f;
        int m      = 0;
        bool alive = true;
        float s0[C], s1[C], s2[C], s3[C];
#pragma unroll
        for (int c = 0; c < C; ++c) s0[c] = s1[c] = s2[c] = s3[c] = 0.f;
        const float* my_sorted = sorted + lane * kSortedPad * E;
        // descriptor rows are requested kRing entries ahead of their use (the gathers are independent of the recurrence)
        constexpr int kRows = (C + 3) / 4;
        constexpr int kRing = SbEntry<C>::kStaged ? 1 : (C <= 4 ? kSbRing : (C <= 8 ? 2 : 1));
        float4 ring[kRing][kRows];
        auto fetch_row = [&](int j, float4 (&dst)[kRows]) {
            if (!SbEntry<C>::kStaged && j < n)
            {
                unsigned eidx = __float_as_uint(my_sorted[j * E]);
                if (eidx >= n_entry) eidx = 0;  // only after a corrupted list was flagged in phase A: read in bounds
                const float* rp = entries + (size_t)eidx * ES + 4;
#pragma unroll
                for (int r = 0; r < kRows; ++r) dst[r] = *reinterpret_cast<const float4*>(rp + 4 * r);
            }
        };
#pragma unroll
        for (int d = 0; d < kRing; ++d) fetch_row(d, ring[d]);
#pragma unroll
        for (int j = 0; j < 16; ++j)
        {
            if (j >= n_max) break;
            float leaf[C];
#pragma unroll
            for (int c = 0; c < C; ++c) leaf[c] = 0.f;
            if (j < n)
            {
                const float* e = my_sorted + j * E;
                float a;
                float row[C];
                if constexpr (SbEntry<C>::kStaged)
                {
                    a = e[0];
#pragma unroll
                    for (int c = 0; c < C; ++c) row[c] = e[1 + c];
                }
                else
                {
                    a = (__float_as_uint(e[0]) < n_entry) ? e[1] : 0.f;  // a corrupted entry draws nothing
#pragma unroll
                    for (int c = 0; c < C; c += 4)
                    {
                        const float4 v4 = ring[j % kRing][c / 4];
                        row[c] = v4.x;
                        if (c + 1 < C) row[c + 1] = v4.y;
                        if (c + 2 < C) row[c + 2] = v4.z;
                        if (c + 3 < C) row[c + 3] = v4.w;
                    }
                }
                const float T_out = (j == 0 || run >= kAlphaCut) ? run : 0.f;
                const float w     = T_out * a;
#pragma unroll
                for (int c = 0; c < C; ++c) leaf[c] = w * row[c];
                if (alive && T_out >= kAlphaCut)
                    m = j + 1;
                else
                    alive = false;
                if (j == n - 1)
                {
                    t_last  = T_out;
                    tn_last = run * (1.f - a);
                }
                run = run * (1.f - a);
            }
            if (j + kRing < 16) fetch_row(j + kRing, ring[j % kRing]);
            // binary-counter accumulation = pairwise tree over leaves 0..15
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                if ((j & 1) == 0)
                    s0[c] = leaf[c];
                else
                {
                    float p1 = s0[c] + leaf[c];
                    if ((j & 2) == 0)
                        s1[c] = p1;
                    else
                    {
                        float p2 = s1[c] + p1;
                        if ((j & 4) == 0)
                            s2[c] = p2;
                        else
                        {
                            float p3 = s2[c] + p2;
                            if ((j & 8) == 0)
                                s3[c] = p3;
                            else
                                s3[c] = s3[c] + p3;  // j == 15: the root
                        }
                    }
                }
            }
        }
        if (p >= 0)
        {
            // pending partial sums of an incomplete tree: the missing leaves are zeros, which add exactly
            float col[C];
            const int jm = n_max;
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                float t = 0.f;
                if (jm >= 16)
                    t = s3[c];
                else
                {
                    if (jm & 1) t = s0[c];
                    if (jm & 2) t = s1[c] + t;
                    if (jm & 4) t = s2[c] + t;
                    if (jm & 8) t = s3[c] + t;
                }
                col[c] = t;
            }
            float wb;
            if (n == 0)
                wb = 1.f;  // the reference reads a neighbouring lane here (RenderForward.cu:1002-1003): defined as pure background
            else if (pr.bg_uses_Tn)
                wb = (t_last >= kAlphaCut && tn_last >= kAlphaCut) ? tn_last : 0.f;
            else
                wb = t_last;
            const int Wl = g.W[layer], Hl = g.H[layer];
            float* o = out.p[layer] + ((size_t)b * C * Hl + gy) * Wl + gx;
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                float v = col[c];
                if (wb >= kAlphaCut) v += bg[c] * (wb * 1.f);
                o[(size_t)c * Hl * Wl] = v;
            }
            if (pr.train) fb.rec_n[bP + p] = (uint8_t)m;
        }
        __syncwarp();
    }
}

cudaError_t launch_sort_blend(const ScenePtrs& sc, const Geom& g, const TripsRenderParams& pr, int B, const FwdBuffers& fb,
                              const LayerPtrs& out, int sm_count, cudaStream_t st)
{
    const unsigned n_tiles = (unsigned)g.n_tiles * (unsigned)B;
    cudaError_t e          = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) return e;
    int blocks = (int)min((unsigned)(sm_count * 16), (n_tiles + kSbWarps - 1) / kSbWarps);
    blocks     = max(blocks, 1);
    switch (sc.C)
    {
        case 3: sort_blend_kernel<3><<<blocks, kSbThreads, 0, st>>>(sc, g, pr, B, fb, out, n_tiles); break;
        case 4: sort_blend_kernel<4><<<blocks, kSbThreads, 0, st>>>(sc, g, pr, B, fb, out, n_tiles); break;
        case 6: sort_blend_kernel<6><<<blocks, kSbThreads, 0, st>>>(sc, g, pr, B, fb, out, n_tiles); break;
        case 8: sort_blend_kernel<8><<<blocks, kSbThreads, 0, st>>>(sc, g, pr, B, fb, out, n_tiles); break;
        case 16: sort_blend_kernel<16><<<blocks, kSbThreads, 0, st>>>(sc, g, pr, B, fb, out, n_tiles); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
}  // namespace trips
