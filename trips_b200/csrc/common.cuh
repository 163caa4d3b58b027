// Internal declarations shared by the kernels and the C ABI of libtrips_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/trips_b200.h"
#include "trips_math.h"

namespace trips
{
constexpr float kAlphaCut = 0.001f;  // ALPHA_DEST_CUTOFF, RenderForward.cu:907
constexpr unsigned kFull  = 0xffffffffu;
constexpr int kBinShift   = 5;   // visible points are bucketed by 32x32-pixel screen bins of layer 0
constexpr int kTileW      = 8;   // one warp renders / differentiates an 8x4 pixel tile
constexpr int kTileH      = 4;
constexpr int kRankShift  = 4;   // entry head: number of layers in the low 4 bits, spatial rank above
constexpr int kMaxRankedPoints = 1 << 28;
constexpr int kHeavyList  = 512;      // lists longer than this get their 16 nearest fragments moved to the front by a block of their own
constexpr int kHeavyCap   = 1 << 16;  // such lists per call the pre-selection handles; beyond that the blend walks them itself

// Pyramid geometry shared by all views of a call.
struct Geom
{
    int L;
    int W[TRIPS_MAX_LAYERS];            // ceil-halved layer sizes (PointRenderer.cu:385-389)
    int H[TRIPS_MAX_LAYERS];
    int base[TRIPS_MAX_LAYERS + 1];     // first pixel of every layer in the per-view pixel arrays (row-major)
    int P;                              // pixels per view
    // Tile order of a view: first the 64x64-pixel regions of layer 0 in row-major order, each with its tiles of
    // layers 0..reg_layers-1 (a region is (64 >> l) pixels wide on layer l), so that the entries of a region stay in L2
    // while all its fine layers are processed; then the remaining coarse layers, layer by layer.
    int reg_layers;                     // min(L, 4)
    int reg_x;                          // regions per row
    int reg_tiles;                      // tiles of one region: 128 + 32 + 8 + 2 for four layers
    int reg_total;                      // tiles of all regions of a view
    int tiles_x[TRIPS_MAX_LAYERS];      // 8x4 pixel tiles per layer row (coarse layers)
    int tile_base[TRIPS_MAX_LAYERS + 1];  // first tile of every coarse layer (layers below reg_layers: reg_total)
    int n_tiles;                        // tiles per view
    int bins_x, bins_y, n_bins;         // 32x32 screen bins of layer 0
};

// Per-view constants built on the device from the pose / intrinsics tensors (setup_cams_kernel).
struct CamConst
{
    float qx, qy, qz, qw, tx, ty, tz;
    float R[9];
    float fx, fy, cx, cy, s;
    float cfx, cfy, ccx, ccy, cs;
    float r00, r01, r10, r11;
    float cenx, ceny;
    int image_index, camera_index;
    float k1, k2, k3, k4, k5, k6, p1, p2;  // lens distortion (TripsRenderParams.distortion)
    float cut2;                            // dist_cutoff^2
    int dist;                              // apply the distortion and the cut-off radius
};

struct LayerPtrs
{
    float* p[TRIPS_MAX_LAYERS];
};
struct ConstLayerPtrs
{
    const float* p[TRIPS_MAX_LAYERS];
};

// Device-side counters of one forward call.
struct DevStats
{
    unsigned long long visible;    // visible points over all views (needed entries, whether or not they fitted)
    unsigned long long kept;
    unsigned long long frag_need;  // fragments over all views (needed list slots, whether or not they fitted)
    unsigned int max_len;
    unsigned int n_heavy;          // pixels whose list is longer than kHeavyList (they are pre-selected before the blend)
    unsigned int max_key;          // largest number of visible points in one (view, screen bin, tile) group
    unsigned int pad0;
    unsigned int status;
    unsigned int culled_blocks;  // (view, block of consecutive points) pairs skipped by the bounding-box test, counted once per pass
};

// A visible point of one view ("entry"): everything the later stages need, gathered once and stored in screen-bin
// order so that fragments of neighbouring pixels read neighbouring entries.  The fields live in two arrays, split by
// the stage that reads them, so that a stage's gathers touch fewer bytes it does not use (DRAM is read in 64-byte
// pieces), while the binning pass still writes whole 32-byte sectors:
//   head [2 x float4]     u, v (layer-0 image position), size in pixels, confidence (all the backward pass reads) |
//                         point id (bits), view-space depth, raw point size, number of layers written (bits 0-3) and
//                         spatial rank of the point (bits 4-31, see rank.cu; 0 when ranks are not in use)
//   tail [1 + C4/4 float4] world position x, y, z, texture index (bits) | descriptor row (C floats, padded to 4)
__host__ __device__ constexpr int tail_stride(int C) { return 4 + ((C + 3) & ~3); }
__host__ __device__ constexpr int entry_stride(int C) { return 8 + tail_stride(C); }  // floats per entry over both arrays
// Gradient accumulator of an entry: sums over its fragments of (J0 gbs, J1 gbs, bf conf lf' ga, bf lf ga) | descriptor row.
__host__ __device__ constexpr int egrad_stride(int C) { return 4 + ((C + 3) & ~3); }

// Everything the forward kernels need besides the scene (all device pointers into context scratch).
struct FwdBuffers
{
    uint32_t* bin_count;              // [B,n_bins,32] visible points per (screen bin, 8x4 tile of the bin)
    uint32_t* bin_base;               // [B,n_bins,32] next free entry (within the view) of every (bin, tile) group
    uint32_t* view_total;             // [B] visible points per view
    uint32_t* bin_cursor;             // [B,n_bins] first entry of every bin within the view
    unsigned long long* entry_base;   // [B+1] first entry of each view
    float4* ent_head;                 // [sum V_b, 2]
    float* ent_tail;                  // [sum V_b, tail_stride]
    uint32_t* counts;                 // [B,P] list lengths
    uint32_t* offsets;                // [B,P] list start within the view (list end after the collect pass)
    uint32_t* partial;                // [B,nchunks] scan partials
    unsigned long long* view_base;    // [B+1] first fragment of each view in `frags`
    uint4* frags;                     // [frag_cap] x = point id, y = depth bits (y:x = 64-bit sort key), z = alpha bits, w = entry index within the view
    unsigned long long frag_cap;
    uint8_t* rec_n;                   // [B,P] records kept for backward
    uint2* records;                   // [B,P,16] (entry index within the view, alpha bits)
    DevStats* stats;
    unsigned int* ticket;
    const uint32_t* point_rank;       // [N] spatial rank of every point, or nullptr: gradient rows are keyed by point id
    const float* block_box;           // [ceil(N / 8192), 6] bounding boxes (min xyz, max xyz) of blocks of consecutive points
    const uint8_t* block_skip;        // [B, ceil(N / 8192)] 1 = the block cannot hold a point visible in that view
    uint2* heavy;                     // [kHeavyCap] (view, pixel) of the lists longer than kHeavyList
};

struct ScenePtrs
{
    int N, n_tex, C;
    const float4* position;
    const float* point_size;
    const int32_t* index;
    const float* texture;
    const float* confidence;
    const float* background;
    const float* dropout;
};

struct BwdBuffers
{
    float* egrad;         // [sum V_b, egrad_stride] per-entry gradient accumulators
    float* g_point;       // [N, egrad_stride] per-point sums keyed by point id: xyz + raw size | descriptor row
    float* g_conf_pt;     // [N] confidence gradient keyed by point id
    double* g_bg;         // [C]
    double* g_pose;       // [B,6]
    double* g_k;          // [B,5]
    double* g_dis;        // [B,8] distortion coefficients
};

// The reference has two forward pipelines (PointRenderer.cu:730-731): the second (CountTiled, CollectTiled2[Pointsize],
// FastSortAndBlendWPrep2WarpSharedWork, RenderForward.cu:1401-3674) runs when one of these flags differs from its
// default.  strict_layers: a point is written to the two layers around log2(size) only (RenderForward.cu:2291-2393).
__host__ __device__ inline bool second_pipeline(const TripsRenderParams& pr)
{
    return !(pr.use_layer_point_size && pr.render_points_in_all_lower_resolutions && !pr.combine_lists);
}
__host__ __device__ inline bool strict_layers(const TripsRenderParams& pr)
{
    return pr.use_layer_point_size && !pr.render_points_in_all_lower_resolutions;
}

// ---- device helpers (op order mirrors the CPU oracle; compiled with -fmad=false) ----

__device__ __forceinline__ void transform_point(const CamConst& V, float px, float py, float pz, float& ox, float& oy,
                                                float& oz)
{
    // Sophus SE3f * p: Eigen quaternion _transformVector, then translation (PointRendererHelper.h:238)
    float ux = V.qy * pz - V.qz * py;
    float uy = V.qz * px - V.qx * pz;
    float uz = V.qx * py - V.qy * px;
    ux += ux;
    uy += uy;
    uz += uz;
    float cx = V.qy * uz - V.qz * uy;
    float cy = V.qz * ux - V.qx * uz;
    float cz = V.qx * uy - V.qy * ux;
    ox       = ((px + V.qw * ux) + cx) + V.tx;
    oy       = ((py + V.qw * uy) + cy) + V.ty;
    oz       = ((pz + V.qw * uz) + cz) + V.tz;
}

// saiga's distortNormalizedPoint restated: the 8-coefficient rational model with tangential terms (the operation order
// is the CPU oracle's).  J (optional): d(xd, yd) / d(x, y) row-major; Jk (optional): d(xd, yd) / d(k1..k6, p1, p2), two
// rows of 8.
__device__ __forceinline__ void distort_point(const CamConst& c, float x, float y, float& xd, float& yd, float* J, float* Jk)
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

// ProjectPointPinholeWoNormal + crop transform + crop rotation
// (PointRendererHelper.h:232-253, RenderForward.cu:302-303,69-76).
__device__ __forceinline__ void project_point(const CamConst& c, float px, float py, float pz, float& u, float& v, float& z)
{
    float vx, vy, vz;
    transform_point(c, px, py, pz, vx, vy, vz);
    z        = fmaxf(vz, 0.f);
    float iz = 1.f / vz;
    float nx = vx * iz;
    float ny = vy * iz;
    if (c.dist)  // uniform per view
    {
        // outside the cut-off radius distortNormalizedPoint returns (100000, 100000) and the caller sets z = 0
        // (PointRendererHelper.h:246-249)
        if (nx * nx + ny * ny > c.cut2) z = 0.f;
        float xd, yd;
        distort_point(c, nx, ny, xd, yd, nullptr, nullptr);
        nx = xd, ny = yd;
    }
    float ix = (c.fx * nx + c.s * ny) + c.cx;
    float iy = c.fy * ny + c.cy;
    float jx = (c.cfx * ix + c.cs * iy) + c.ccx;
    float jy = c.cfy * iy + c.ccy;
    float dx = jx - c.cenx;
    float dy = jy - c.ceny;
    float rx = c.r00 * dx + c.r01 * dy;
    float ry = c.r10 * dx + c.r11 * dy;
    u        = rx + c.cenx;
    v        = ry + c.ceny;
}

// compute_point_size_fac (PointBlending.h:81-149); floor / ceil of log2 taken from the float's bits.
// FAST_EXP: the hardware exponential (about 2 ulp) instead of the reproducible one; only for values that do not decide
// list membership, i.e. in the backward pass (gradient tolerance 1e-4), never in the forward pass.
template <bool FAST_EXP = false>
__device__ __forceinline__ float layer_factor(float ps, int layer, int L, float* grad)
{
    int lo = 0, hi = 0;
    if (ps > 1.f)
    {
        lo = min(max(0, tm_floor_log2(ps)), L - 1);
        hi = min(max(0, tm_ceil_log2(ps)), L - 1);
    }
    if (layer < lo)
    {
        if (grad) *grad = 0.f;
        return 1.f;
    }
    float f = 1.f;
    if (hi == 0)
    {
        f = 0.75f * (FAST_EXP ? __expf(ps - 1.f) : tm_expf(ps - 1.f)) + 0.25f;
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

// Pixel handled by `lane` of the warp that owns 8x4 tile `tile` of a view; p = -1 outside the image.
__device__ __forceinline__ void tile_pixel(const Geom& g, int tile, int lane, int& layer, int& gx, int& gy, int& p)
{
    int l, tx, ty;
    if (tile < g.reg_total)
    {
        const int r = tile / g.reg_tiles, k = tile - r * g.reg_tiles;
        l           = k < 128 ? 0 : (k < 160 ? 1 : (k < 168 ? 2 : 3));
        const int kk = k - (l == 0 ? 0 : (l == 1 ? 128 : (l == 2 ? 160 : 168)));
        const int ry = r / g.reg_x, rx = r - ry * g.reg_x;
        tx = rx * (8 >> l) + (kk & ((8 >> l) - 1));   // a region is 8 >> l tiles wide and 16 >> l tiles high on layer l
        ty = ry * (16 >> l) + (kk >> (3 - l));
    }
    else
    {
        l = g.reg_layers;
#pragma unroll
        for (int i = 1; i < TRIPS_MAX_LAYERS; ++i)
            if (i > g.reg_layers && i < g.L && tile >= g.tile_base[i]) l = i;
        const int t = tile - g.tile_base[l];
        ty          = t / g.tiles_x[l];
        tx          = t - ty * g.tiles_x[l];
    }
    layer        = l;
    gx           = tx * kTileW + (lane & (kTileW - 1));
    gy           = ty * kTileH + (lane >> 3);
    p            = (gx < g.W[l] && gy < g.H[l]) ? g.base[l] + gy * g.W[l] + gx : -1;
}

// ---- launchers (forward.cu / backward.cu / adam.cu) ----
cudaError_t launch_setup_cams(const TripsView* d_views, int B, const double* poses, int n_images, const float* intrinsics,
                              int n_cameras, int distortion, float dist_cutoff, CamConst* cams, DevStats* stats, cudaStream_t st);
cudaError_t launch_bin_count(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr, int B,
                             const FwdBuffers& fb, unsigned long long entry_cap, bool hot, int sm_count, cudaStream_t st);
cudaError_t launch_bin_scatter(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr, int B,
                               const FwdBuffers& fb, bool hot, int sm_count, cudaStream_t st);
constexpr unsigned kHotKey = 4096;  // visible points in one (view, bin, tile) group beyond which the binning passes aggregate in shared memory
int bin_count_launches(int N, int B);
int bin_scatter_launches(int N, int B);
size_t resize_scratch_bytes(int64_t n_points);
cudaError_t launch_resize_points(const int64_t* remove, int64_t n_remove, int64_t n_points, int64_t n_new, const TripsPointTensor* tensors,
                                 int n_tensors, void* scratch, DevStats* stats, int sm_count, cudaStream_t st);
size_t rank_temp_bytes(int N);
cudaError_t launch_point_rank(const float4* position, int N, unsigned* scratch, void* temp, size_t temp_bytes, unsigned* rank,
                              int sm_count, cudaStream_t st);
cudaError_t launch_scan(const Geom& g, int B, int k_keep, const FwdBuffers& fb, int nchunks, cudaStream_t st);
// strict: an entry's layers start at the layer below log2(size) instead of layer 0 (strict_layers above)
// entries_hint: the number of entries of the call as far as the host knows it (selects the size of the work tickets)
cudaError_t launch_count(const ScenePtrs& sc, const Geom& g, int B, const FwdBuffers& fb, bool strict, unsigned long long entries_hint, int sm_count,
                         cudaStream_t st);
cudaError_t launch_collect(const ScenePtrs& sc, const Geom& g, int B, const FwdBuffers& fb, bool strict, int sm_count, cudaStream_t st);
// top-K + blend by the rules of the reference's second forward pipeline (one thread per pixel)
cudaError_t launch_second_blend(const ScenePtrs& sc, const Geom& g, const TripsRenderParams& pr, int B, const FwdBuffers& fb,
                                const LayerPtrs& out, int sm_count, cudaStream_t st);
cudaError_t launch_heavy_topk(const Geom& g, int B, const FwdBuffers& fb, int sm_count, cudaStream_t st);
cudaError_t launch_sort_blend(const ScenePtrs& sc, const Geom& g, const TripsRenderParams& pr, int B, const FwdBuffers& fb,
                              const LayerPtrs& out, int sm_count, cudaStream_t st);
cudaError_t launch_zero_entry_rows(int C, int B, const FwdBuffers& fb, const BwdBuffers& bb, int sm_count, cudaStream_t st);
cudaError_t launch_blend_backward(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr,
                                  int B, const FwdBuffers& fb, const BwdBuffers& bb, const ConstLayerPtrs& grad_in,
                                  bool want_cam_grads, int sm_count, cudaStream_t st);
cudaError_t launch_unpack_grads(const ScenePtrs& sc, const CamConst* cams, int B, const FwdBuffers& fb, const BwdBuffers& bb,
                                const TripsGrads& out, const TripsRenderParams& pr, int sm_count, cudaStream_t st);
cudaError_t launch_adam(const TripsAdamTensor* d_tensors, const int64_t* d_block_start, int n_tensors, int64_t total_blocks,
                        cudaStream_t st);
cudaError_t launch_fused_reduce_adam(const float* const* grad_ptrs, float* const* param_ptrs, int world, int rank,
                                     const TripsAdamSegment* segs, int n_seg, int64_t lo, int64_t hi, float* m_state,
                                     float* v_state, int32_t* steps, int sm_count, cudaStream_t st);
cudaError_t launch_fused_multicast_adam(const float* grad_mc, float* param_mc, const float* param, const TripsAdamSegment* segs, int n_seg,
                                        int64_t lo, int64_t hi, float* m_state, float* v_state, int32_t* steps, int sm_count, cudaStream_t st);
struct L1Args
{
    const float* out[TRIPS_MAX_LAYERS];
    const float* target[TRIPS_MAX_LAYERS];
    float* grad[TRIPS_MAX_LAYERS];
    int64_t start[TRIPS_MAX_LAYERS + 1];
    int L;
};
cudaError_t launch_l1_loss(const L1Args& a, int64_t total, double* loss_out, int sm_count, cudaStream_t st);
constexpr int kScanChunk    = 2048;
constexpr int kAdamPerBlock = 1024 * 4;  // elements handled by one Adam block
}  // namespace trips
