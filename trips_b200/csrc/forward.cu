// Forward rasterizer: project + count, scan, collect, per-pixel top-K sort and front-to-back blend.
//
// Stage map to the reference (src/lib/rendering/RenderForward.cu):
//   project_count_kernel  <- CountAndCollectTiled        (:168-366)
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
// descriptor repack: texture [C,n_tex] -> rows [n_tex,C] so that one fragment gathers one 4C-byte row
// ------------------------------------------------------------------------------------------------------------
template <int C>
__global__ void pack_texture_kernel(const float* __restrict__ tex, int n_tex, float* __restrict__ out)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n_tex; i += (size_t)gridDim.x * blockDim.x)
    {
        float v[C];
#pragma unroll
        for (int c = 0; c < C; ++c) v[c] = __ldg(tex + (size_t)c * n_tex + i);
#pragma unroll
        for (int c = 0; c < C; ++c) out[i * C + c] = v[c];
    }
}

cudaError_t launch_pack_texture(const ScenePtrs& sc, float* tex_packed, cudaStream_t st)
{
    int blocks = (int)min((size_t)148 * 16, ((size_t)sc.n_tex + 255) / 256);
    if (blocks < 1) blocks = 1;
    switch (sc.C)
    {
        case 3: pack_texture_kernel<3><<<blocks, 256, 0, st>>>(sc.texture, sc.n_tex, tex_packed); break;
        case 4: pack_texture_kernel<4><<<blocks, 256, 0, st>>>(sc.texture, sc.n_tex, tex_packed); break;
        case 6: pack_texture_kernel<6><<<blocks, 256, 0, st>>>(sc.texture, sc.n_tex, tex_packed); break;
        case 8: pack_texture_kernel<8><<<blocks, 256, 0, st>>>(sc.texture, sc.n_tex, tex_packed); break;
        case 16: pack_texture_kernel<16><<<blocks, 256, 0, st>>>(sc.texture, sc.n_tex, tex_packed); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// project + cull + layer select + count
// ------------------------------------------------------------------------------------------------------------
__global__ __launch_bounds__(256) void project_count_kernel(ScenePtrs sc, const CamConst* __restrict__ cams,
                                                            const __grid_constant__ Geom g,
                                                            TripsRenderParams pr, FwdBuffers fb)
{
    __shared__ CamConst cam;
    const int b = blockIdx.y;
    if (threadIdx.x < sizeof(CamConst) / 4) ((int*)&cam)[threadIdx.x] = ((const int*)&cams[b])[threadIdx.x];
    __syncthreads();
    const int N        = sc.N;
    const size_t bN    = (size_t)b * N;
    uint32_t* counts   = fb.counts + (size_t)b * g.P;
    const float fxc    = cam.fx * cam.cfx;
    const float w_hi   = (float)(g.W[0] - 1);
    const float h_hi   = (float)(g.H[0] - 1);
    unsigned n_visible = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x)
    {
        float depth_out = -1.f;
        uint8_t nl_out  = 0;
        float4 rec_out  = make_float4(0.f, 0.f, 0.f, 0.f);
        bool skip       = false;
        int tex         = sc.index ? __ldg(sc.index + i) : i;
        if (pr.viewer_only)
        {
            // discard_point_for_confidence, RenderForward.cu:122-130
            if ((unsigned)tex < (unsigned)sc.n_tex && __ldg(sc.confidence + tex) < pr.stability_cutoff_value) skip = true;
        }
        else if (pr.train && sc.dropout)
        {
            if (__ldg(sc.dropout + bN + i) == 1.f) skip = true;
        }
        if (!skip)
        {
            const float4 p = __ldg(sc.position + i);
            const float s  = tm_softplus(__ldg(sc.point_size + i));
            float u, v, z;
            project_point(cam, p.x, p.y, p.z, u, v, z);
            float rad      = fxc * p.w / z;
            const float ps = fxc * s / z;
            bool ok        = !(z <= 0.f || u < 0.f || u >= w_hi || v < 0.f || v >= h_hi);
            if (ok && pr.drop_out_points_by_radius && (float)(int)rad < pr.drop_out_radius_threshold) ok = false;
            if (ok)
            {
                depth_out = z;
                rec_out   = make_float4(u, v, ps, __int_as_float(tex));
                int hi    = 0;
                if (ps > 1.f) hi = min(tm_ceil_log2(ps), g.L - 1);
                int layer = 0;
                float x = u, y = v;
                for (; layer < hi + 1; ++layer, x *= 0.5f, y *= 0.5f, rad *= 0.5f)
                {
                    int px = __float2int_rd(x), py = __float2int_rd(y);
                    if (px < 0 || px >= g.W[layer] - 1 || py < 0 || py >= g.H[layer] - 1) break;
                    if (pr.drop_out_points_by_radius && (float)(int)rad < pr.drop_out_radius_threshold) break;
                    uint32_t* c0 = counts + g.base[layer] + py * g.W[layer] + px;
                    atomicAdd(c0, 1u);
                    atomicAdd(c0 + 1, 1u);
                    atomicAdd(c0 + g.W[layer], 1u);
                    atomicAdd(c0 + g.W[layer] + 1, 1u);
                }
                nl_out = (uint8_t)layer;
                n_visible++;
            }
        }
        fb.depth[bN + i] = depth_out;
        fb.nlay[bN + i]  = nl_out;
        fb.rec[bN + i]   = rec_out;
    }
    // one atomic per warp for the visible-point counter
    for (int o = 16; o > 0; o >>= 1) n_visible += __shfl_xor_sync(kFull, n_visible, o);
    if ((threadIdx.x & 31) == 0 && n_visible) atomicAdd(&fb.stats->visible, (unsigned long long)n_visible);
}

cudaError_t launch_project_count(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr,
                                 int B, const FwdBuffers& fb, cudaStream_t st)
{
    int bx = (sc.N + 255) / 256;
    bx     = max(1, min(bx, 148 * 8));
    project_count_kernel<<<dim3(bx, B), 256, 0, st>>>(sc, cams, g, pr, fb);
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
// collect: four threads per point write the 64-bit fragment keys into the per-pixel lists
// ------------------------------------------------------------------------------------------------------------
__global__ __launch_bounds__(256) void collect_kernel(int N, const __grid_constant__ Geom g, FwdBuffers fb)
{
    const int b        = blockIdx.y;
    const size_t bN    = (size_t)b * N;
    uint32_t* cursor   = fb.offsets + (size_t)b * g.P;
    const unsigned long long vbase = fb.view_base[b];
    const unsigned long long vend  = fb.view_base[b + 1];
    if (vend > fb.frag_cap) return;  // list buffer too small: the overflow status bit is already raised
    unsigned long long* frags = fb.frags + vbase;
    const size_t total = (size_t)N * 4;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x)
    {
        const int i   = (int)(t >> 2);
        const int sub = (int)(t & 3);
        const float z = fb.depth[bN + i];
        if (!(z > 0.f)) continue;
        const int nl      = fb.nlay[bN + i];
        const float4 r    = fb.rec[bN + i];
        const unsigned long long key = ((unsigned long long)__float_as_uint(z) << 32) | (unsigned)i;
        float x = r.x, y = r.y;
        for (int layer = 0; layer < nl; ++layer, x *= 0.5f, y *= 0.5f)
        {
            int px = __float2int_rd(x) + (sub & 1), py = __float2int_rd(y) + (sub >> 1);
            uint32_t slot = atomicAdd(cursor + g.base[layer] + py * g.W[layer] + px, 1u);
            frags[slot]   = key;
        }
    }
}

cudaError_t launch_collect(const ScenePtrs& sc, const Geom& g, int B, const FwdBuffers& fb, cudaStream_t st)
{
    size_t threads = (size_t)sc.N * 4;
    int bx         = (int)min((size_t)148 * 32, (threads + 255) / 256);
    collect_kernel<<<dim3(max(bx, 1), B), 256, 0, st>>>(sc.N, g, fb);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// per-pixel top-K sort in registers + front-to-back blend
// ------------------------------------------------------------------------------------------------------------
typedef unsigned long long u64;
constexpr u64 kInfKey = 0xffffffffffffffffull;

__device__ __forceinline__ u64 cmpx(u64 key, int j_mask, bool keep_min)
{
    u64 other = __shfl_xor_sync(kFull, key, j_mask);
    return keep_min ? min(key, other) : max(key, other);
}

// ascending bitonic sort of 16 keys held one per lane by each half-warp (10 compare-exchange steps)
__device__ __forceinline__ u64 bitonic_sort16(u64 key, int j)
{
#pragma unroll
    for (int k = 2; k <= 16; k <<= 1)
    {
#pragma unroll
        for (int s = k >> 1; s > 0; s >>= 1)
        {
            bool up       = ((j & k) == 0) || (k == 16);
            bool lower    = (j & s) == 0;
            key           = cmpx(key, s, lower == up);
        }
    }
    return key;
}

// a bitonic sequence of 16 keys -> ascending (4 steps)
__device__ __forceinline__ u64 bitonic_merge16(u64 key, int j)
{
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) key = cmpx(key, s, (j & s) == 0);
    return key;
}

// One warp renders a tile of 32 consecutive pixels of one view, two pixels (one per half-warp) at a time:
// lane j of a half-warp holds the j-th nearest fragment of its pixel.
template <int C>
__global__ __launch_bounds__(256) void sort_blend_kernel(ScenePtrs sc, const __grid_constant__ Geom g, TripsRenderParams pr, int B, FwdBuffers fb,
                                                         const __grid_constant__ LayerPtrs out, unsigned n_tiles,
                                                         unsigned tiles_per_view)
{
    __shared__ float s_out[8][C][32];
    const int lane  = threadIdx.x & 31;
    const int warp  = threadIdx.x >> 5;
    const int j     = lane & 15;
    const int hbase = lane & 16;
    const int K     = pr.k_keep;
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);

    for (;;)
    {
        unsigned tile = 0;
        if (lane == 0) tile = atomicAdd(fb.ticket, 1u);
        tile = __shfl_sync(kFull, tile, 0);
        if (tile >= n_tiles) break;
        const int b     = tile / tiles_per_view;
        const int p0    = (tile - b * tiles_per_view) * 32;
        const size_t bP = (size_t)b * g.P;
        const size_t bN = (size_t)b * sc.N;
        const u64* frags = fb.frags + fb.view_base[b];
        // lane i owns pixel p0 + i for the coalesced loads / stores
        const int p_mine = p0 + lane;
        uint32_t cnt_mine = 0, start_mine = 0;
        int layer_mine = 0, gx_mine = 0, gy_mine = 0;
        if (p_mine < g.P)
        {
            cnt_mine   = fb.counts[bP + p_mine];
            start_mine = fb.offsets[bP + p_mine] - cnt_mine;  // offsets hold list ends after the collect pass
            pixel_to_layer(g, p_mine, layer_mine, gx_mine, gy_mine);
        }
        for (int it = 0; it < 16; ++it)
        {
            const int src        = it * 2 + (hbase >> 4);
            const uint32_t cnt   = __shfl_sync(kFull, cnt_mine, src);
            const uint32_t start = __shfl_sync(kFull, start_mine, src);
            const int layer      = __shfl_sync(kFull, layer_mine, src);
            const int gx         = __shfl_sync(kFull, gx_mine, src);
            const int gy         = __shfl_sync(kFull, gy_mine, src);
            const int p          = p0 + src;
            const uint32_t cnt_o = __shfl_xor_sync(kFull, cnt, 16);
            if (p0 + it * 2 >= g.P) break;  // warp-uniform: both pixels of this step are past the view's end

            // ---- streaming top-16: sort the first 16 fragments, then merge further chunks of 16 ----
            u64 key = (j < (int)cnt) ? frags[start + j] : kInfKey;
            key     = bitonic_sort16(key, j);
            const uint32_t cnt_max = max(cnt, cnt_o);
            for (uint32_t ch = 16; ch < cnt_max; ch += 16)
            {
                u64 nk      = (ch + j < cnt) ? frags[start + ch + j] : kInfKey;
                u64 cur_max = __shfl_sync(kFull, key, hbase | 15);
                if (__ballot_sync(kFull, nk < cur_max) == 0) continue;  // nothing nearer in either half
                nk       = bitonic_sort16(nk, j);
                u64 rev  = __shfl_sync(kFull, nk, hbase | (15 - j));
                key      = min(key, rev);
                key      = bitonic_merge16(key, j);
            }
            const int n = min((int)cnt, K);
            const bool active = j < n;

            // ---- alpha of my fragment ----
            float a = 0.f;
            int pid = -1, tex = 0;
            if (active)
            {
                pid            = (int)(unsigned)(key & 0xffffffffull);
                const float4 r = fb.rec[bN + pid];
                tex            = __float_as_int(r.w);
                const float fac = __int_as_float((127 - layer) << 23);  // 2^-layer
                const float ux = r.x * fac, uy = r.y * fac;
                const float dx = fabsf(ux - (float)gx), dy = fabsf(uy - (float)gy);
                float bl = (1.f - dx) * (1.f - dy);
                if (dx > 1.f || dy > 1.f) bl = 0.f;
                if ((unsigned)tex >= (unsigned)sc.n_tex)
                {
                    atomicOr(&fb.stats->status, TRIPS_DEV_BAD_TEXTURE_INDEX);
                    tex = 0;
                    bl  = 0.f;
                }
                a = bl * __ldg(sc.confidence + tex);
                a *= layer_factor(r.z, layer, g.L, nullptr);
            }
            // ---- transmittance chain T_j = T_{j-1} * (1 - a_{j-1}) ----
            const int n_o   = min((int)cnt_o, K);
            const int n_max = max(n, n_o);
            float run = 1.f, T = 1.f;
            for (int s = 1; s < n_max; ++s)
            {
                float am = __shfl_sync(kFull, a, hbase | (s - 1));
                run      = run * (1.f - am);
                if (j == s) T = run;
            }
            const float T_out = (j == 0 || T >= kAlphaCut) ? T : 0.f;
            // ---- colour: butterfly sum over the 16 lanes ----
            float col[C];
            {
                const float w = T_out * a;
                const float* row = fb.tex_packed + (size_t)tex * C;
#pragma unroll
                for (int c = 0; c < C; ++c) col[c] = active ? w * __ldg(row + c) : 0.f;
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1)
            {
#pragma unroll
                for (int c = 0; c < C; ++c) col[c] += __shfl_xor_sync(kFull, col[c], o);
            }
            // ---- background weight ----
            float wb;
            {
                const int last = hbase | max(n - 1, 0);
                float t_last   = __shfl_sync(kFull, T_out, last);
                float tn_last  = __shfl_sync(kFull, T * (1.f - a), last);
                if (n == 0)
                    wb = 1.f;
                else if (pr.bg_uses_Tn)
                    wb = (t_last >= kAlphaCut && tn_last >= kAlphaCut) ? tn_last : 0.f;
                else
                    wb = t_last;
            }
            if (j == 0 && p < g.P)
            {
#pragma unroll
                for (int c = 0; c < C; ++c)
                {
                    float o = col[c];
                    if (wb >= kAlphaCut) o += bg[c] * (wb * 1.f);
                    s_out[warp][c][src] = o;
                }
            }
            // ---- records for backward: the leading fragments whose transmittance is above the cut-off ----
            if (pr.train)
            {
                unsigned ok   = __ballot_sync(kFull, active && T_out >= kAlphaCut);
                unsigned half = (ok >> hbase) & 0xffffu;
                int m         = __ffs(~half) - 1;  // number of leading set bits (<= 16)
                if (p < g.P)
                {
                    if (j < m) fb.records[(bP + p) * 16 + j] = make_uint2((unsigned)pid, __float_as_uint(a));
                    if (j == 0) fb.rec_n[bP + p] = (uint8_t)m;
                }
            }
        }
        __syncwarp();
        if (p_mine < g.P)
        {
            const int Wl = g.W[layer_mine], Hl = g.H[layer_mine];
            float* o = out.p[layer_mine] + ((size_t)b * C * Hl + gy_mine) * Wl + gx_mine;
#pragma unroll
            for (int c = 0; c < C; ++c) o[(size_t)c * Hl * Wl] = s_out[warp][c][lane];
        }
        __syncwarp();
    }
}

cudaError_t launch_sort_blend(const ScenePtrs& sc, const Geom& g, const TripsRenderParams& pr, int B, const FwdBuffers& fb,
                              const LayerPtrs& out, int sm_count, cudaStream_t st)
{
    unsigned tiles_per_view = (unsigned)((g.P + 31) / 32);
    unsigned n_tiles        = tiles_per_view * (unsigned)B;
    cudaError_t e           = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) return e;
    int blocks = (int)min((unsigned)(sm_count * 8), (n_tiles + 7) / 8);
    blocks     = max(blocks, 1);
    switch (sc.C)
    {
        case 3: sort_blend_kernel<3><<<blocks, 256, 0, st>>>(sc, g, pr, B, fb, out, n_tiles, tiles_per_view); break;
        case 4: sort_blend_kernel<4><<<blocks, 256, 0, st>>>(sc, g, pr, B, fb, out, n_tiles, tiles_per_view); break;
        case 6: sort_blend_kernel<6><<<blocks, 256, 0, st>>>(sc, g, pr, B, fb, out, n_tiles, tiles_per_view); break;
        case 8: sort_blend_kernel<8><<<blocks, 256, 0, st>>>(sc, g, pr, B, fb, out, n_tiles, tiles_per_view); break;
        case 16: sort_blend_kernel<16><<<blocks, 256, 0, st>>>(sc, g, pr, B, fb, out, n_tiles, tiles_per_view); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
}  // namespace trips
