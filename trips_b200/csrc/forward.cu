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
                                  const float* __restrict__ intrinsics, int n_cameras, CamConst* __restrict__ cams,
                                  DevStats* stats)
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
    if (dist) atomicOr(&stats->status, TRIPS_DEV_NONZERO_DISTORTION);
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
                              int n_cameras, CamConst* cams, DevStats* stats, cudaStream_t st)
{
    setup_cams_kernel<<<(B + 63) / 64, 64, 0, st>>>(d_views, B, poses, n_images, intrinsics, n_cameras, cams, stats);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// project + cull + layer select, bucket the visible points of every view by 32x32 screen bin, count fragments
//
// Three kernels: (1) count visible points per (view, bin); (2) exclusive scan of the bin counts; (3) project again,
// take a slot in the bin, write the point's 16-byte-aligned entry there and add 1 to the list length of every
// pixel its 2x2 footprints touch, on each pyramid layer it is drawn into.  Replaces CountAndCollectTiled
// (RenderForward.cu:168-366).  Projecting twice costs two coalesced reads of position + size per view and avoids
// writing and re-reading a per-point record for all N points.
// ------------------------------------------------------------------------------------------------------------
struct Projected
{
    float u, v, z, ps, rad;
    int tex;
    bool ok;
};

__device__ __forceinline__ Projected project_visible(const ScenePtrs& sc, const CamConst& cam, const Geom& g,
                                                     const TripsRenderParams& pr, size_t bN, int i, float fxc)
{
    Projected r;
    r.ok  = false;
    r.tex = sc.index ? __ldg(sc.index + i) : i;
    if (pr.viewer_only)
    {
        // discard_point_for_confidence, RenderForward.cu:122-130
        if ((unsigned)r.tex < (unsigned)sc.n_tex && __ldg(sc.confidence + r.tex) < pr.stability_cutoff_value) return r;
    }
    else if (pr.train && sc.dropout)
    {
        if (__ldg(sc.dropout + bN + i) == 1.f) return r;
    }
    const float4 p = __ldg(sc.position + i);
    const float s  = tm_softplus(__ldg(sc.point_size + i));
    project_point(cam, p.x, p.y, p.z, r.u, r.v, r.z);
    r.rad = fxc * p.w / r.z;
    r.ps  = fxc * s / r.z;
    bool ok = !(r.z <= 0.f || r.u < 0.f || r.u >= (float)(g.W[0] - 1) || r.v < 0.f || r.v >= (float)(g.H[0] - 1));
    if (ok && pr.drop_out_points_by_radius && (float)(int)r.rad < pr.drop_out_radius_threshold) ok = false;
    r.ok = ok;
    return r;
}

__global__ __launch_bounds__(256) void bin_count_kernel(ScenePtrs sc, const CamConst* __restrict__ cams,
                                                        const __grid_constant__ Geom g, TripsRenderParams pr, FwdBuffers fb)
{
    __shared__ CamConst cam;
    const int b = blockIdx.y;
    if (threadIdx.x < sizeof(CamConst) / 4) ((int*)&cam)[threadIdx.x] = ((const int*)&cams[b])[threadIdx.x];
    __syncthreads();
    const size_t bN = (size_t)b * sc.N;
    const float fxc = cam.fx * cam.cfx;
    uint32_t* bins  = fb.bin_count + (size_t)b * g.n_bins;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < sc.N; i += gridDim.x * blockDim.x)
    {
        const Projected r = project_visible(sc, cam, g, pr, bN, i, fxc);
        if (r.ok) atomicAdd(bins + (__float2int_rd(r.v) >> kBinShift) * g.bins_x + (__float2int_rd(r.u) >> kBinShift), 1u);
    }
}

// one block: per view, exclusive scan of the bin counts -> first entry of every bin; entry_base = running total
__global__ __launch_bounds__(1024) void bin_scan_kernel(const uint32_t* __restrict__ bin_count, uint32_t* __restrict__ bin_cursor,
                                                        int n_bins, int B, unsigned long long* __restrict__ entry_base,
                                                        DevStats* stats)
{
    __shared__ uint32_t sm[32];
    __shared__ uint32_t carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long base = 0;
    for (int b = 0; b < B; ++b)
    {
        const uint32_t* c = bin_count + (size_t)b * n_bins;
        uint32_t* o       = bin_cursor + (size_t)b * n_bins;
        if (threadIdx.x == 0) carry_s = 0;
        __syncthreads();
        for (int s = 0; s < n_bins; s += 1024)
        {
            const int i  = s + threadIdx.x;
            uint32_t v   = (i < n_bins) ? c[i] : 0u;
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
            if (i < n_bins) o[i] = carry + woff + inc - v;
            __syncthreads();
            if (threadIdx.x == 0) carry_s = carry + tot;
            __syncthreads();
        }
        if (threadIdx.x == 0)
        {
            entry_base[b] = base;
            base += carry_s;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0)
    {
        entry_base[B]  = base;
        stats->visible = base;
    }
}

template <int C>
__global__ __launch_bounds__(256) void bin_scatter_kernel(ScenePtrs sc, const CamConst* __restrict__ cams,
                                                          const __grid_constant__ Geom g, TripsRenderParams pr, FwdBuffers fb)
{
    constexpr int ES = entry_stride(C);
    __shared__ CamConst cam;
    const int b = blockIdx.y;
    if (threadIdx.x < sizeof(CamConst) / 4) ((int*)&cam)[threadIdx.x] = ((const int*)&cams[b])[threadIdx.x];
    __syncthreads();
    const size_t bN  = (size_t)b * sc.N;
    const float fxc  = cam.fx * cam.cfx;
    uint32_t* cursor = fb.bin_cursor + (size_t)b * g.n_bins;
    uint32_t* counts = fb.counts + (size_t)b * g.P;
    float* entries   = fb.entries + fb.entry_base[b] * ES;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < sc.N; i += gridDim.x * blockDim.x)
    {
        const Projected r = project_visible(sc, cam, g, pr, bN, i, fxc);
        if (!r.ok) continue;
        const int bin       = (__float2int_rd(r.v) >> kBinShift) * g.bins_x + (__float2int_rd(r.u) >> kBinShift);
        const uint32_t slot = atomicAdd(cursor + bin, 1u);
        // layers 0..hi, stopping where the 2x2 footprint leaves the layer (RenderForward.cu:342-363)
        int hi = 0;
        if (r.ps > 1.f) hi = min(tm_ceil_log2(r.ps), g.L - 1);
        int layer = 0;
        float x = r.u, y = r.v, rad = r.rad;
        for (; layer < hi + 1; ++layer, x *= 0.5f, y *= 0.5f, rad *= 0.5f)
        {
            const int px = __float2int_rd(x), py = __float2int_rd(y);
            if (px < 0 || px >= g.W[layer] - 1 || py < 0 || py >= g.H[layer] - 1) break;
            if (pr.drop_out_points_by_radius && (float)(int)rad < pr.drop_out_radius_threshold) break;
            uint32_t* c0 = counts + g.base[layer] + py * g.W[layer] + px;
            atomicAdd(c0, 1u);
            atomicAdd(c0 + 1, 1u);
            atomicAdd(c0 + g.W[layer], 1u);
            atomicAdd(c0 + g.W[layer] + 1, 1u);
        }
        float conf = 0.f;
        const bool tex_ok = (unsigned)r.tex < (unsigned)sc.n_tex;
        if (tex_ok)
            conf = __ldg(sc.confidence + r.tex);
        else
            atomicOr(&fb.stats->status, TRIPS_DEV_BAD_TEXTURE_INDEX);  // the point is drawn with alpha 0
        const float4 p = __ldg(sc.position + i);
        float4* e      = reinterpret_cast<float4*>(entries + (size_t)slot * ES);
        e[0]           = make_float4(r.u, r.v, r.ps, r.z);
        e[1]           = make_float4(__int_as_float(i), conf, __ldg(sc.point_size + i), __int_as_float(layer));
        e[2]           = make_float4(p.x, p.y, p.z, __int_as_float(tex_ok ? r.tex : -1));
        float row[(C + 3) & ~3];
#pragma unroll
        for (int c = 0; c < ((C + 3) & ~3); ++c) row[c] = (c < C && tex_ok) ? __ldg(sc.texture + (size_t)c * sc.n_tex + r.tex) : 0.f;
#pragma unroll
        for (int c = 0; c < ((C + 3) & ~3); c += 4) e[3 + c / 4] = make_float4(row[c], row[c + 1], row[c + 2], row[c + 3]);
    }
}

cudaError_t launch_bin_points(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr, int B,
                              const FwdBuffers& fb, cudaStream_t st)
{
    cudaError_t e = cudaMemsetAsync(fb.bin_count, 0, sizeof(uint32_t) * (size_t)B * g.n_bins, st);
    if (e != cudaSuccess) return e;
    int bx = max(1, min((sc.N + 255) / 256, 148 * 8));
    if (sc.N > 0) bin_count_kernel<<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb);
    bin_scan_kernel<<<1, 1024, 0, st>>>(fb.bin_count, fb.bin_cursor, g.n_bins, B, fb.entry_base, fb.stats);
    if (sc.N > 0)
    {
        switch (sc.C)
        {
            case 3: bin_scatter_kernel<3><<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb); break;
            case 4: bin_scatter_kernel<4><<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb); break;
            case 6: bin_scatter_kernel<6><<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb); break;
            case 8: bin_scatter_kernel<8><<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb); break;
            case 16: bin_scatter_kernel<16><<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb); break;
            default: return cudaErrorInvalidValue;
        }
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
                                                          uint32_t* __restrict__ partial, DevStats* stats)
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
    unsigned long long base = 0;
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
            view_base[b] = base;
            base += carry_s;
            if (base > frag_cap) atomicOr(&stats->status, TRIPS_DEV_FRAGMENT_OVERFLOW);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) view_base[B] = base;
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
    scan_reduce_kernel<<<dim3(nchunks, B), 256, 0, st>>>(fb.counts, g.P, nchunks, k_keep, fb.partial, fb.stats);
    scan_partials_kernel<<<1, 1024, 0, st>>>(fb.partial, nchunks, B, fb.view_base, fb.frag_cap, fb.stats);
    scan_apply_kernel<<<dim3(nchunks, B), 256, 0, st>>>(fb.counts, g.P, nchunks, fb.partial, fb.offsets);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// collect: four threads per visible point (entry) write one 16-byte fragment per (layer, footprint pixel) into the
// per-pixel lists: the 64-bit sort key (depth bits << 32 | point id), the fragment's alpha and the entry index.
// Computing alpha here, where every lane holds a fragment, keeps the per-fragment arithmetic (bilinear weight,
// confidence, layer factor) out of the per-pixel blend.  alpha = bilinear * confidence * layer factor, in the
// operation order of FastSortFusedNew (RenderForward.cu:882-899).  Replaces SplattingPass (RenderForward.cu:368-436).
// Entries are in screen-bin order, so the list cursors and the fragment stores of a block stay within a small
// window of the pixel arrays.
// ------------------------------------------------------------------------------------------------------------
__global__ __launch_bounds__(256) void collect_kernel(int ES, const __grid_constant__ Geom g, FwdBuffers fb)
{
    const int b      = blockIdx.y;
    uint32_t* cursor = fb.offsets + (size_t)b * g.P;
    const unsigned long long vbase = fb.view_base[b];
    const unsigned long long vend  = fb.view_base[b + 1];
    if (vend > fb.frag_cap) return;  // list buffer too small: the overflow status bit is already raised
    uint4* frags         = fb.frags + vbase;
    const size_t n_entry = (size_t)(fb.entry_base[b + 1] - fb.entry_base[b]);
    const float* entries = fb.entries + fb.entry_base[b] * ES;
    const size_t total   = n_entry * 4;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x)
    {
        const size_t ei = t >> 2;
        const int sub   = (int)(t & 3);
        const float4 e0 = *reinterpret_cast<const float4*>(entries + ei * ES);      // u v ps z
        const float4 e1 = *reinterpret_cast<const float4*>(entries + ei * ES + 4);  // pid conf raw nl
        const int nl     = __float_as_int(e1.w);
        const float conf = e1.y;
        float x = e0.x, y = e0.y;
        for (int layer = 0; layer < nl; ++layer, x *= 0.5f, y *= 0.5f)
        {
            const int px = __float2int_rd(x) + (sub & 1), py = __float2int_rd(y) + (sub >> 1);
            const uint32_t slot = atomicAdd(cursor + g.base[layer] + py * g.W[layer] + px, 1u);
            // x, y equal (u, v) * 2^-layer exactly (power-of-two scaling)
            const float dx = fabsf(x - (float)px), dy = fabsf(y - (float)py);
            float bl = (1.f - dx) * (1.f - dy);
            if (dx > 1.f || dy > 1.f) bl = 0.f;
            float a = bl * conf;
            a *= layer_factor(e0.z, layer, g.L, nullptr);
            frags[slot] = make_uint4(__float_as_uint(e1.x), __float_as_uint(e0.w), __float_as_uint(a), (unsigned)ei);
        }
    }
}

cudaError_t launch_collect(const ScenePtrs& sc, const Geom& g, int B, const FwdBuffers& fb, int sm_count, cudaStream_t st)
{
    collect_kernel<<<dim3(sm_count * 8 / max(1, min(B, 8)) + 1, B), 256, 0, st>>>(entry_stride(sc.C), g, fb);
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
constexpr int kRankMax   = 192;  // longest list ranked by counting; longer lists use the streaming path
constexpr int kSortedPad = 17;   // row pitch (entries) of the per-pixel sorted lists in shared memory
#ifndef TRIPS_SB_STAGE_MAX_C
#define TRIPS_SB_STAGE_MAX_C 0
#endif
#ifndef TRIPS_SB_THREADS
#define TRIPS_SB_THREADS 128
#endif
constexpr int kSbThreads = TRIPS_SB_THREADS;
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

// A sorted entry in shared memory is (alpha, descriptor row[C]) when the row fits the shared-memory budget (C <= 4:
// the gather happens in phase A where lanes are densely packed); for wider descriptors it is (entry index, alpha)
// and phase B gathers.
template <int C>
struct SbEntry
{
    static constexpr bool kStaged = (C <= TRIPS_SB_STAGE_MAX_C);
    static constexpr int kFloats  = kStaged ? (1 + C) : 2;
};

template <int C>
__device__ __forceinline__ void sb_store_entry(float* dst, const float* entries, unsigned eidx, unsigned alpha_bits)
{
    if constexpr (SbEntry<C>::kStaged)
    {
        const float4 v4 = *reinterpret_cast<const float4*>(entries + (size_t)eidx * entry_stride(C) + 12);
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

template <int C>
__global__ __launch_bounds__(kSbThreads) void sort_blend_kernel(ScenePtrs sc, const __grid_constant__ Geom g, TripsRenderParams pr,
                                                                int B, FwdBuffers fb, const __grid_constant__ LayerPtrs out,
                                                                unsigned n_tiles_total)
{
    constexpr int E  = SbEntry<C>::kFloats;
    constexpr int ES = entry_stride(C);
    __shared__ float s_sorted[kSbWarps][32 * kSortedPad * E];  // per warp: 32 pixels x K entries, nearest first
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K    = pr.k_keep;
    float* sorted  = s_sorted[warp];
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);

    for (;;)
    {
        unsigned ticket = 0;
        if (lane == 0) ticket = atomicAdd(fb.ticket, 1u);
        ticket = __shfl_sync(kFull, ticket, 0);
        if (ticket >= n_tiles_total) break;
        const int b          = ticket / (unsigned)g.n_tiles;
        const int tile       = ticket - b * (unsigned)g.n_tiles;
        const size_t bP      = (size_t)b * g.P;
        const uint4* frags   = fb.frags + fb.view_base[b];
        const float* entries = fb.entries + fb.entry_base[b] * ES;
        int layer, gx, gy, p;
        tile_pixel(g, tile, lane, layer, gx, gy, p);  // lane i owns one pixel of the tile
        uint32_t cnt = 0, start = 0;
        if (p >= 0)
        {
            cnt   = fb.counts[bP + p];
            start = fb.offsets[bP + p] - cnt;  // offsets hold list ends after the collect pass
        }
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
            // ---- phase A, counting path: lane = fragment ----
            for (uint32_t t0 = 0; t0 < tile_total; t0 += 32)
            {
                const uint32_t t = t0 + lane;
                const bool valid = t < tile_total;
                // pixel of this fragment: the last lane whose list starts at or before t
                int seg = 0;
#pragma unroll
                for (int step = 16; step > 0; step >>= 1)
                {
                    const int probe       = seg + step;
                    const uint32_t pstart = __shfl_sync(kFull, rel_start, probe & 31);
                    if (probe < 32 && pstart <= t) seg = probe;
                }
                const uint32_t seg_rel   = __shfl_sync(kFull, rel_start, seg);
                const uint32_t seg_start = __shfl_sync(kFull, start, seg);
                const uint32_t seg_cnt   = __shfl_sync(kFull, cnt, seg);
                const int seg_p          = __shfl_sync(kFull, p, seg);
                if (valid)
                {
                    const uint4 f   = frags[seg_start + (t - seg_rel)];
                    const u64 mine  = ((u64)f.y << 32) | f.x;
                    const uint2* kp = reinterpret_cast<const uint2*>(frags + seg_start);
                    int rank        = 0;
                    for (uint32_t i = 0; i < seg_cnt; ++i)
                    {
                        const uint2 o = kp[(size_t)i * 2];
                        rank += ((((u64)o.y << 32) | o.x) < mine) ? 1 : 0;
                    }
                    if (rank < K)
                    {
                        sb_store_entry<C>(sorted + (seg * kSortedPad + rank) * E, entries, f.w, f.z);
                        if (pr.train) fb.records[(bP + seg_p) * 16 + rank] = make_uint2(f.w, f.z);
                    }
                }
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
                    const u64 cur_max = __shfl_sync(kFull, v.key, hbase | 15);
                    if (__ballot_sync(kFull, nk.key < cur_max) == 0) continue;  // nothing nearer in either half
                    nk = bitonic_sort16(nk, j);
                    KeyVal rev;
                    rev.key   = __shfl_sync(kFull, nk.key, hbase | (15 - j));
                    rev.alpha = __shfl_sync(kFull, nk.alpha, hbase | (15 - j));
                    rev.eidx  = __shfl_sync(kFull, nk.eidx, hbase | (15 - j));
                    if (rev.key < v.key) v = rev;
                    v = bitonic_merge16(v, j);
                }
                if (j < min((int)cnt_s, K))
                {
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
                    const unsigned eidx = __float_as_uint(e[0]);
                    a                   = e[1];
                    const float* rp     = entries + (size_t)eidx * ES + 12;
#pragma unroll
                    for (int c = 0; c < C; c += 4)
                    {
                        const float4 v4 = *reinterpret_cast<const float4*>(rp + c);
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
