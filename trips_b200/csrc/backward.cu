// Backward rasterizer: replays the kept fragments of every pixel and scatters gradients to descriptors,
// confidences, positions, point sizes, the background colour, the camera pose and the pinhole coefficients.
//
// Replaces BlendBackwardsBilinearTiled (src/lib/rendering/RenderBackward.cu:90-618).  Differences in structure:
//   * a warp per 8x4 pixel tile; the reference's O(K^2) inner loop (RenderBackward.cu:284-301) becomes a reverse
//     running sum over the pixel's kept fragments;
//   * fragments add image-space sums to a 32-byte row of their entry (one row per visible point and view, in screen
//     order); the chain to position / size / pose is applied once per entry (entry_grad_finish_kernel), which adds to
//     a 32-byte row per point (stored by spatial rank); one pass then writes the reference's layouts
//     (unpack_point_kernel);
//   * pixels are enumerated with the ceil-halved layer sizes of the forward pass (the reference halves with
//     floor here, RenderBackward.cu:112-130, and thereby skips rows of odd-sized layers).
#include "common.cuh"

namespace trips
{
template <int C>
__device__ __forceinline__ void atomic_add_row(float* row, const float (&v)[C])
{
    if constexpr (C % 4 == 0)
    {
#pragma unroll
        for (int c = 0; c < C; c += 4) atomicAdd(reinterpret_cast<float4*>(row + c), make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]));
    }
    else if constexpr (C % 2 == 0)
    {
#pragma unroll
        for (int c = 0; c < C; c += 2) atomicAdd(reinterpret_cast<float2*>(row + c), make_float2(v[c], v[c + 1]));
    }
    else
    {
#pragma unroll
        for (int c = 0; c < C; ++c) atomicAdd(row + c, v[c]);
    }
}

__device__ __forceinline__ double warp_sum_d(double v)
{
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

constexpr int kPad        = 17;   // row pitch (entries) of the per-pixel arrays in shared memory
constexpr int kBwdThreads = 128;  // 4 warps x (32 x 17 slots x 12 bytes + fragment table + gradient tile) = 32 KB of static shared memory
constexpr int kBwdWarps   = kBwdThreads / 32;

// One warp differentiates an 8x4 pixel tile; tiles come from one ticket counter over all views, in the order of
// tile_pixel (region-major), so the entries and gradient rows a tile touches are a short, L2-resident range.
//   staging: the tile's records go to shared memory (8 lanes per pixel row: 4 lines per load instruction).
//   phase 0 (lane = kept fragment, lanes densely packed over the tile's fragments): gather the descriptor row of
//     the fragment's entry, G_j = <col_j, g> and alpha_j go to shared memory.
//   phase 1 (lane = pixel, shared memory only): the sequential recurrences over the pixel's kept fragments:
//     transmittance T_j, w_j = T_j alpha_j, and d_j = dLoss/dalpha_j = T_j G_j - (W_bg + sum_{i>j} W_i) / (1 - alpha_j + 1e-9)
//     with W_i = G_i T_i alpha_i (RenderBackward.cu:262-303; the reference's O(K^2) inner loop becomes a reverse
//     running sum).
//   phase 2 (lane = kept fragment): descriptor gradient and the image-space sums of the fragment's entry
//     (RenderBackward.cu:335-393), accumulated with two vector atomics into the per-entry gradient rows, which are
//     in screen-bin order like the entries and therefore stay hot in L2 while a region of the image is processed.
// What bounds the kernel (ncu): about 50 % of the issue slots and 48 % of the load/store unit's line rate are in use
// at 16-20 resident warps per SM; DRAM is at 20-30 %.  Hence the care for lines per instruction (entries ordered by
// tile, paired atomics, coalesced staging) and for instructions per fragment (fragment table, no shuffle searches).
constexpr int kBwdBlocksPerSM = 12;  // grid size of the persistent kernel, in blocks per SM
// measured: 5 resident blocks (96 registers) 3.59 ms, 4 blocks (108) 3.63 ms, 6 blocks (80) 3.76 ms
constexpr int kBwdMinBlocks = 5;
// SAT: saturated_alpha_accumulation as the reference's backward pass has it (RenderBackward.cu:227-259); a separate
// instantiation, so that the common case carries none of its code or registers.
template <int C, bool SAT>
__global__ __launch_bounds__(kBwdThreads, (C <= 4 ? kBwdMinBlocks : 1)) void blend_backward_kernel(ScenePtrs sc, const CamConst* __restrict__ cams,
                                                                     const __grid_constant__ Geom g, TripsRenderParams pr, int B,
                                                                     FwdBuffers fb, BwdBuffers bb,
                                                                     const __grid_constant__ ConstLayerPtrs grad_in)
{
    constexpr int DS = tail_stride(C);
    constexpr int GS = egrad_stride(C);
    __shared__ float s_g[kBwdWarps][C][32];
    __shared__ float s_d[kBwdWarps][32 * kPad];   // G_j, then dA_j = G_j T_j, finally d_j
    __shared__ float s_sum[SAT ? kBwdWarps : 1][SAT ? 32 * kPad : 1];  // SAT: sum of the descriptor channels of fragment j
    __shared__ uint16_t s_map[kBwdWarps][32 * 16];
    __shared__ uint2 s_rec[kBwdWarps][32 * kPad]; // the tile's records: (entry index, alpha_j bits; after phase 1: w_j = T_j * alpha_j)
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);

    float* my_d          = s_d[warp] + lane * kPad;
    uint2* my_rec        = s_rec[warp] + lane * kPad;

    double acc_bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) acc_bg[c] = 0.0;

    // one ticket counter over all views: the views are processed one after the other, so the entries, gradient rows and
    // records in flight belong to one view
    const unsigned n_total = (unsigned)g.n_tiles * (unsigned)B;
    unsigned next_tile = 0;
    if (lane == 0) next_tile = atomicAdd(fb.ticket, 1u);
    for (;;)
    {
        // the ticket of the following tile is requested now, a whole tile ahead of its use
        const unsigned ticket = __shfl_sync(kFull, next_tile, 0);
        if (ticket >= n_total) break;
        if (lane == 0) next_tile = atomicAdd(fb.ticket, 1u);
        const int b          = ticket / (unsigned)g.n_tiles;
        const unsigned tile  = ticket - b * (unsigned)g.n_tiles;
        const size_t bP      = (size_t)b * g.P;
        const float* desc    = fb.ent_tail + fb.entry_base[b] * DS + 4;  // descriptor row of entry e at desc + e * DS
        const float4* head   = fb.ent_head + fb.entry_base[b] * 2;
        float* egrad         = bb.egrad + fb.entry_base[b] * GS;
        const uint32_t n_ent = (uint32_t)(fb.entry_base[b + 1] - fb.entry_base[b]);
        int layer, gx, gy, p;
        tile_pixel(g, (int)tile, lane, layer, gx, gy, p);
        const int gx0 = __shfl_sync(kFull, gx, 0), gy0 = __shfl_sync(kFull, gy, 0);  // tile origin: lane l is pixel (gx0 + (l & 7), gy0 + (l >> 3))
        int m = 0;
        float gin[C];
#pragma unroll
        for (int c = 0; c < C; ++c) gin[c] = 0.f;
        if (p >= 0)
        {
            m            = fb.rec_n[bP + p];
            const int Wl = g.W[layer], Hl = g.H[layer];
            const float* gi = grad_in.p[layer] + ((size_t)b * C * Hl + gy) * Wl + gx;
#pragma unroll
            for (int c = 0; c < C; ++c) gin[c] = __ldg(gi + (size_t)c * Hl * Wl);
        }
#pragma unroll
        for (int c = 0; c < C; ++c) s_g[warp][c][lane] = gin[c];
        int m_max = m;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_max = max(m_max, __shfl_xor_sync(kFull, m_max, o));
        // lanes <-> kept fragments of the tile: exclusive prefix of the record counts
        int incl = m;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            int t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        const int rel     = incl - m;
        const int n_entry = __shfl_sync(kFull, incl, 31);
        // the tile's records (entry index, alpha) -> shared memory.  The 16 records of a pixel are one 128-byte line: eight
        // lanes read the eight 16-byte pieces of one pixel's line, so a load instruction touches 4 lines instead of 32
        // (the load/store unit handles one line per cycle); pieces beyond the pixel's record count are not read.
#pragma unroll
        for (int it = 0; it < 8; ++it)
        {
            const int q   = it * 4 + (lane >> 3);  // pixel of the tile
            const int k   = lane & 7;              // piece: records 2k, 2k+1
            const int m_q = __shfl_sync(kFull, m, q);
            const int p_q = __shfl_sync(kFull, p, q);
            if (2 * k < m_q)
            {
                const uint4 v = *(reinterpret_cast<const uint4*>(fb.records + (bP + p_q) * 16) + k);
                uint2* dst    = s_rec[warp] + q * kPad + 2 * k;
                dst[0]        = make_uint2(v.x < n_ent ? v.x : 0u, v.x < n_ent ? v.y : 0u);  // a corrupted record contributes nothing
                dst[1]        = make_uint2(v.z < n_ent ? v.z : 0u, v.z < n_ent ? v.w : 0u);
            }
        }
        __syncwarp();
        // (pixel, slot in the padded per-pixel arrays) of the e-th kept fragment of the tile: a table written by the
        // pixels' lanes replaces a binary search over warp shuffles in every round of both fragment phases
        {
            uint16_t* mp = s_map[warp] + rel;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < m) mp[j] = (uint16_t)((lane << 10) | (lane * kPad + j));
        }
        __syncwarp();
        auto locate = [&](int e, int& seg, int& slot) {
            const unsigned v = e < n_entry ? s_map[warp][e] : 0u;  // lanes beyond the last fragment point at slot 0
            seg  = v >> 10;
            slot = v & 1023;
        };

        // ---- phase 0 (lane = kept fragment): G_j = <descriptor row of the entry, g>; the row of the next round is
        //      requested before the current one is consumed ----
        {
            int seg_n, j_n;
            locate(lane, seg_n, j_n);
            float4 row_n[(C + 3) / 4];
            if (lane < n_entry)
            {
                const float* rp = desc + (size_t)s_rec[warp][j_n].x * DS;
#pragma unroll
                for (int c = 0; c < (C + 3) / 4; ++c) row_n[c] = *reinterpret_cast<const float4*>(rp + 4 * c);
            }
            for (int e0 = 0; e0 < n_entry; e0 += 32)
            {
                const int seg = seg_n, j = j_n;
                float4 row[(C + 3) / 4];
#pragma unroll
                for (int c = 0; c < (C + 3) / 4; ++c) row[c] = row_n[c];
                if (e0 + 32 < n_entry)
                {
                    locate(e0 + 32 + lane, seg_n, j_n);
                    if (e0 + 32 + lane < n_entry)
                    {
                        const float* rp = desc + (size_t)s_rec[warp][j_n].x * DS;
#pragma unroll
                        for (int c = 0; c < (C + 3) / 4; ++c) row_n[c] = *reinterpret_cast<const float4*>(rp + 4 * c);
                    }
                }
                if (e0 + lane < n_entry)
                {
                    float G = 0.f;
#pragma unroll
                    for (int c = 0; c < C; c += 4)
                    {
                        const float4 v4 = row[c / 4];
                        G += v4.x * s_g[warp][c][seg];
                        if (c + 1 < C) G += v4.y * s_g[warp][c + 1][seg];
                        if (c + 2 < C) G += v4.z * s_g[warp][c + 2][seg];
                        if (c + 3 < C) G += v4.w * s_g[warp][c + 3][seg];
                    }
                    s_d[warp][j] = G;
                    if constexpr (SAT)
                    {
                        float S = 0.f;
#pragma unroll
                        for (int c = 0; c < C; c += 4)
                        {
                            const float4 v4 = row[c / 4];
                            S += v4.x;
                            if (c + 1 < C) S += v4.y;
                            if (c + 2 < C) S += v4.z;
                            if (c + 3 < C) S += v4.w;
                        }
                        s_sum[warp][j] = S;
                    }
                }
            }
        }
        __syncwarp();

        // ---- phase 1 (lane = pixel), forward: T_j, dA_j = G_j T_j, w_j = T_j a_j.  The alphas move to registers (the
        //      reverse sweep needs them again) and w_j takes their place in shared memory. ----
        float run = 1.f;
        if constexpr (SAT)
        {
            // RenderBackward.cu:227-259 as written.  alpha_dest starts at 1 and loses every alpha; a fragment's texture
            // gradient is weighted by its alpha while alpha_dest - alpha > 0, else by what is left (the fragment that
            // fills the pixel).  d_j starts as G_j = <colour_j, g>; the filling fragment's own d is dropped and the sum
            // of its colour channels (not weighted by g) is taken from every fragment before it.  After the filling
            // fragment alpha_dest is 0 and the replay ends, so this happens at most once per pixel, possibly for the
            // background step (colour = background, alpha = 1).
            float* my_sum = s_sum[warp] + lane * kPad;
#pragma unroll
            for (int j = 0; j < 16; ++j)
            {
                if (j >= m_max) continue;  // uniform
                if (j < m && run < kAlphaCut)
                {
                    // the replay ends where alpha_dest falls below the cut-off (RenderBackward.cu:308); records behind that
                    // point exist when the forward pass blended by transmittance, which falls more slowly
                    my_rec[j].y = 0u;
                    my_d[j]     = 0.f;
                }
                else if (j < m)
                {
                    const float a    = __uint_as_float(my_rec[j].y);
                    const bool fill  = (run - a) < 0.f && run > 0.f;
                    my_rec[j].y      = __float_as_uint((run - a) > 0.f ? a : __saturatef(run));
                    if (fill)
                    {
                        const float S = my_sum[j];
                        my_d[j]       = 0.f;
                        for (int i = 0; i < j; ++i) my_d[i] -= S;
                    }
                    run = __saturatef(run - a);
                }
            }
            if (p >= 0 && run >= kAlphaCut)
            {
                // background step: alpha 1, weight saturate(alpha_dest); it fills the pixel whenever alpha_dest < 1
                float S = 0.f;
#pragma unroll
                for (int c = 0; c < C; ++c)
                {
                    acc_bg[c] += (double)(((run - 1.f) > 0.f ? 1.f : __saturatef(run)) * gin[c]);
                    S += bg[c];
                }
                if ((run - 1.f) < 0.f && run > 0.f)
                    for (int i = 0; i < m; ++i) my_d[i] -= S;
            }
        }
        else
        {
        float al[16];
#pragma unroll
        for (int j = 0; j < 16; ++j)
        {
            al[j] = 0.f;
            if (j >= m_max) continue;  // uniform
            if (j < m)
            {
                const float a = __uint_as_float(my_rec[j].y);
                al[j]         = a;
                my_d[j]       = my_d[j] * run;
                my_rec[j].y   = __float_as_uint(run * a);
                run           = (1.f - a) * run;
            }
        }
        // background step with alpha = 1 while the transmittance is above the cut-off (RenderBackward.cu:205-210,308)
        float R = 0.f;
        if (p >= 0 && run >= kAlphaCut)
        {
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                R += gin[c] * bg[c] * run * 1.f;
                acc_bg[c] += (double)(run * 1.f * gin[c]);
            }
        }
        // ---- phase 1, reverse: d_j = dA_j - R_j / (1 - a_j + eps), R_j = W_bg + sum_{i>j} W_i, W_i = dA_i a_i ----
#pragma unroll
        for (int j = 15; j >= 0; --j)
        {
            if (j < m)
            {
                const float a   = al[j];
                const float dA  = my_d[j];
                const float dem = 1.f / (1.f - a + 1e-9f);
                my_d[j]         = dA - R * dem;
                R += dA * a;
            }
        }
        }
        __syncwarp();

        // ---- phase 2 (lane = kept fragment): the header of the next round's entry is requested early ----
        {
            int seg_n, j_n;
            locate(lane, seg_n, j_n);
            float4 e0_n = make_float4(0.f, 0.f, 0.f, 0.f);
            unsigned eidx_n = 0;
            if (lane < n_entry)
            {
                eidx_n          = s_rec[warp][j_n].x;
                e0_n            = head[2 * (size_t)eidx_n];  // u v ps conf
            }
            for (int e0 = 0; e0 < n_entry; e0 += 32)
            {
                const int seg = seg_n, j = j_n;
                const float4 e0v = e0_n;  // u v ps conf
                const float conf = e0v.w;
                const unsigned eidx = eidx_n;
                const bool valid = e0 + lane < n_entry;
                if (e0 + 32 < n_entry)
                {
                    locate(e0 + 32 + lane, seg_n, j_n);
                    if (e0 + 32 + lane < n_entry)
                    {
                        eidx_n          = s_rec[warp][j_n].x;
                        e0_n            = head[2 * (size_t)eidx_n];
                    }
                }
                const int layer_s = layer;  // a tile lies on one layer
                const int gx_s = gx0 + (seg & (kTileW - 1)), gy_s = gy0 + (seg >> 3);
                // (lanes without a fragment run through with zero weights: the exchange below needs all lanes)
                const float ga = valid ? s_d[warp][j] : 0.f;
                const float w  = valid ? __uint_as_float(s_rec[warp][j].y) : 0.f;
                // bilinear weight of this pixel and its Jacobian at uv (compute_blending_fac, PointBlending.h:216-257)
                const float fac = __int_as_float((127 - layer_s) << 23);
                const float ux = e0v.x * fac, uy = e0v.y * fac;
                const float ps = e0v.z;
                const int q    = ((float)gx_s < ux ? 0 : 1) + ((float)gy_s < uy ? 0 : 2);
                const float sx = ux - floorf(ux), sy = uy - floorf(uy);
                float bf = ((q & 1) ? sx : (1.f - sx)) * ((q & 2) ? sy : (1.f - sy));
                const float J0 = (q & 1) ? ((q & 2) ? sy : (1.f - sy)) : ((q & 2) ? -sy : (sy - 1.f));
                const float J1 = (q & 2) ? ((q & 1) ? sx : (1.f - sx)) : ((q & 1) ? -sx : (sx - 1.f));
                if (fabsf(ux - (float)gx_s) > 1.f || fabsf(uy - (float)gy_s) > 1.f) bf *= 0.f;
                float lf_grad   = 0.f;
                // (without use_layer_point_size the forward pass applied no layer factor: none here, and no size gradient)
                const float lf  = pr.use_layer_point_size ? layer_factor<true>(ps, layer_s, g.L, &lf_grad) : 1.f;
                const float gbs = conf * lf * ga;  // dLoss / d(bilinear weight) (RenderBackward.cu:385)
                // image-space sums of the entry: the chain to position / size / pose is linear in them and is applied
                // once per entry by entry_grad_finish_kernel
                const float4 h0 = make_float4(J0 * gbs, J1 * gbs, bf * conf * lf_grad * ga, bf * lf * ga);
                float gt[(C + 3) & ~3];
#pragma unroll
                for (int c = 0; c < ((C + 3) & ~3); ++c) gt[c] = (c < C) ? w * s_g[warp][c < C ? c : 0][seg] : 0.f;
                if constexpr (((C + 3) & ~3) == 4)
                {
                    // The row of an entry is 32 bytes: two 16-byte atomics.  Lanes work in pairs: the even lane adds the
                    // first half and the odd lane the second half of the SAME row (first the even lane's fragment, then
                    // the odd lane's), so an atomic instruction touches 16 rows instead of 32.  The load/store unit
                    // handles one 128-byte line per cycle, and that, not DRAM or the L2 atomic rate, bounds this kernel.
                    const bool odd       = lane & 1;
                    const unsigned mine  = valid ? eidx : 0xffffffffu;
                    const unsigned other = __shfl_xor_sync(kFull, mine, 1);
                    float4 x;  // even lane receives the partner's first half, odd lane the partner's second half
                    x.x = __shfl_xor_sync(kFull, odd ? h0.x : gt[0], 1);
                    x.y = __shfl_xor_sync(kFull, odd ? h0.y : gt[1], 1);
                    x.z = __shfl_xor_sync(kFull, odd ? h0.z : gt[2], 1);
                    x.w = __shfl_xor_sync(kFull, odd ? h0.w : gt[3], 1);
                    const unsigned row_a = odd ? other : mine;  // the even lane's fragment
                    const unsigned row_b = odd ? mine : other;  // the odd lane's fragment
                    const float4 own     = odd ? make_float4(gt[0], gt[1], gt[2], gt[3]) : h0;
                    if (row_a != 0xffffffffu) atomicAdd(reinterpret_cast<float4*>(egrad + (size_t)row_a * GS + (odd ? 4 : 0)), odd ? x : own);
                    if (row_b != 0xffffffffu) atomicAdd(reinterpret_cast<float4*>(egrad + (size_t)row_b * GS + (odd ? 4 : 0)), odd ? own : x);
                }
                else if (valid)
                {
                    float* eg = egrad + (size_t)eidx * GS;
                    atomicAdd(reinterpret_cast<float4*>(eg), h0);
                    atomic_add_row<((C + 3) & ~3)>(eg + 4, gt);
                }
            }
        }
        __syncwarp();
    }
    // view-level gradients: warp shuffle reduction, then one double atomic per warp
#pragma unroll
    for (int c = 0; c < C; ++c)
    {
        double v = warp_sum_d(acc_bg[c]);
        if (lane == 0 && v != 0.0) atomicAdd(bb.g_bg + c, v);
    }
}

// The gradient rows of the entries the forward pass wrote start from zero.  Their number is known on the device only
// (entry_base[B]): the host does not wait for the forward pass's counts.
__global__ __launch_bounds__(256) void zero_entry_rows_kernel(float4* __restrict__ egrad, const unsigned long long* __restrict__ entry_base, int B,
                                                              int row_f4)
{
    const unsigned long long n = entry_base[B] * (unsigned long long)row_f4;
    const float4 z             = make_float4(0.f, 0.f, 0.f, 0.f);
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (unsigned long long)gridDim.x * blockDim.x)
        egrad[i] = z;
}

cudaError_t launch_zero_entry_rows(int C, int B, const FwdBuffers& fb, const BwdBuffers& bb, int sm_count, cudaStream_t st)
{
    zero_entry_rows_kernel<<<sm_count * 8, 256, 0, st>>>(reinterpret_cast<float4*>(bb.egrad), fb.entry_base, B, egrad_stride(C) / 4);
    return cudaGetLastError();
}

cudaError_t launch_blend_backward(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr,
                                  int B, const FwdBuffers& fb, const BwdBuffers& bb, const ConstLayerPtrs& grad_in,
                                  bool want_cam_grads, int sm_count, cudaStream_t st)
{
    cudaError_t e = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) return e;
    const int grid = (int)max(1u, min((unsigned)(sm_count * kBwdBlocksPerSM), ((unsigned)g.n_tiles * (unsigned)B + kBwdWarps - 1) / kBwdWarps));
#define TRIPS_BWD_CASE(CC)                                                                                         \
    case CC:                                                                                                       \
        if (pr.saturated_alpha_accumulation)                                                                       \
            blend_backward_kernel<CC, true><<<grid, kBwdThreads, 0, st>>>(sc, cams, g, pr, B, fb, bb, grad_in);   \
        else                                                                                                       \
            blend_backward_kernel<CC, false><<<grid, kBwdThreads, 0, st>>>(sc, cams, g, pr, B, fb, bb, grad_in);  \
        break;
    switch (sc.C)
    {
        TRIPS_BWD_CASE(3)
        TRIPS_BWD_CASE(4)
        TRIPS_BWD_CASE(6)
        TRIPS_BWD_CASE(8)
        TRIPS_BWD_CASE(16)
        default: return cudaErrorInvalidValue;
    }
#undef TRIPS_BWD_CASE
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// per-entry gradient rows -> per-point sums (one set of atomics per visible point and view instead of one per
// fragment), then the reference's output layouts (PointRenderer.cu:1423-1426)
// ------------------------------------------------------------------------------------------------------------
// Applies, once per entry, the chain from the accumulated image-space sums to the point: crop rotation, crop
// transform, pinhole, division by z and the rotation (ProjectPointPinholeBackward, PointRendererHelper.h:434-494,
// zero distortion), the softplus derivative for the size, and adds the entry's gradients to its point
// (one set of atomics per visible point and view instead of one per fragment).  Pose and intrinsics gradients
// are summed per view in double (RenderBackward.cu:453-466,587-611).
// DIST: lens distortion between the division by z and the pinhole matrix (TripsRenderParams.distortion): the
// view-space position then comes from the entry's world position (the stored projection cannot be undistorted in
// closed form), the chain goes through J_p_dis^T and the eight coefficients receive J_dis_dis^T
// (PointRendererHelper.h:468-491).  A separate instantiation: the plain pinhole carries none of it.
template <int C, bool CAM_GRADS, bool DIST>
__global__ __launch_bounds__(256) void entry_grad_finish_kernel(FwdBuffers fb, BwdBuffers bb, const CamConst* __restrict__ cams, int B)
{
    constexpr int GS = egrad_stride(C);
    constexpr int PS = egrad_stride(C);  // per-point row: xyz + size | descriptor row
    constexpr int NA = CAM_GRADS ? (DIST ? 19 : 11) : 1;  // 6 pose + 5 pinhole (+ 8 distortion) sums per view
    __shared__ CamConst cam;
    __shared__ double s_acc[8][NA];
    const int b = blockIdx.y;
    if (threadIdx.x < sizeof(CamConst) / 4) ((int*)&cam)[threadIdx.x] = ((const int*)&cams[b])[threadIdx.x];
    __syncthreads();
    const float fxc = cam.fx * cam.cfx;
    const unsigned long long first = fb.entry_base[b], n = fb.entry_base[b + 1] - first;
    const float4* head   = fb.ent_head + first * 2;
    const float* egrad   = bb.egrad + first * GS;
    double acc[NA];
#pragma unroll
    for (int k = 0; k < NA; ++k) acc[k] = 0.0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (unsigned long long)gridDim.x * blockDim.x)
    {
        const float* eg = egrad + i * GS;
        const float4 s4 = *reinterpret_cast<const float4*>(eg);      // sum J0 gbs, sum J1 gbs, sum bf conf lf' ga, sum bf lf ga
        const float4 e1 = head[2 * i + 1];  // pid z raw nl|rank
        const float4 e0 = head[2 * i];      // u v ps conf
        const int pid   = __float_as_int(e1.x);
        // row of the point: by spatial rank when the forward pass stored one (rows of a screen bin then share L2 lines)
        const size_t row = fb.point_rank ? (size_t)(__float_as_uint(e1.w) >> kRankShift) : (size_t)pid;
        // View-space position from the stored projection: (u, v) back through crop rotation, crop transform and the
        // pinhole matrix gives the normalised coordinates, the stored depth scales them.  This spares the read of the
        // entry's world position (a third of the kernel's DRAM traffic); the round trip costs a few 1e-7 relative,
        // far inside the gradient tolerance.
        float vz = e1.y;
        float vx, vy;
        if constexpr (DIST)
        {
            const float4 wp = *reinterpret_cast<const float4*>(fb.ent_tail + (first + i) * tail_stride(C));  // world xyz | texture index
            transform_point(cam, wp.x, wp.y, wp.z, vx, vy, vz);
        }
        else
        {
            const float du = e0.x - cam.cenx, dv = e0.y - cam.ceny;
            const float idet = 1.f / (cam.r00 * cam.r11 - cam.r01 * cam.r10);
            const float jx = (cam.r11 * du - cam.r01 * dv) * idet + cam.cenx;
            const float jy = (cam.r00 * dv - cam.r10 * du) * idet + cam.ceny;
            const float iy = (jy - cam.ccy) / cam.cfy;
            const float ix = (jx - cam.ccx - cam.cs * iy) / cam.cfx;
            const float ny = (iy - cam.cy) / cam.fy;
            const float nx = (ix - cam.cx - cam.s * ny) / cam.fx;
            vx = nx * vz;
            vy = ny * vz;
        }
        if (vz > 0.f && (s4.x != 0.f || s4.y != 0.f || s4.z != 0.f))
        {
            const float iz  = 1.f / vz;
            const float gr0 = cam.r00 * s4.x + cam.r10 * s4.y;
            const float gr1 = cam.r01 * s4.x + cam.r11 * s4.y;
            const float gk0 = cam.cfx * gr0;
            const float gk1 = cam.cs * gr0 + cam.cfy * gr1;
            float gn0 = cam.fx * gk0;
            float gn1 = cam.s * gk0 + cam.fy * gk1;
            float kx = vx * iz, ky = vy * iz;  // the normalised coordinates the pinhole matrix sees
            if constexpr (DIST)
            {
                float xd, yd, Jd[4], Jk[16];
                distort_point(cam, kx, ky, xd, yd, Jd, CAM_GRADS ? Jk : nullptr);
                if constexpr (CAM_GRADS)
                {
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[11 + k] += (double)(Jk[k] * gn0 + Jk[8 + k] * gn1);
                }
                const float g0 = Jd[0] * gn0 + Jd[2] * gn1;
                const float g1 = Jd[1] * gn0 + Jd[3] * gn1;
                gn0 = g0, gn1 = g1;
                kx = xd, ky = yd;
            }
            const float gv0 = iz * gn0;
            const float gv1 = iz * gn1;
            const float gv2 = (-vx * iz * iz) * gn0 + (-vy * iz * iz) * gn1;
            const float gp0 = cam.R[0] * gv0 + cam.R[3] * gv1 + cam.R[6] * gv2;
            const float gp1 = cam.R[1] * gv0 + cam.R[4] * gv1 + cam.R[7] * gv2;
            const float gp2 = cam.R[2] * gv0 + cam.R[5] * gv1 + cam.R[8] * gv2;
            const float gl  = tm_softplus_grad(e1.z) * (fxc / vz) * s4.z;
            atomicAdd(reinterpret_cast<float4*>(bb.g_point + row * PS), make_float4(gp0, gp1, gp2, gl));
            if constexpr (CAM_GRADS)
            {
                const float nx = kx, ny = ky;
                acc[0] += (double)gv0;
                acc[1] += (double)gv1;
                acc[2] += (double)gv2;
                acc[3] += (double)(vy * gv2 - vz * gv1);
                acc[4] += (double)(vz * gv0 - vx * gv2);
                acc[5] += (double)(vx * gv1 - vy * gv0);
                acc[6] += (double)(nx * gk0);
                acc[7] += (double)(ny * gk1);
                acc[8] += (double)gk0;
                acc[9] += (double)gk1;
                acc[10] += (double)(ny * gk0);
            }
        }
        // (an entry whose texture index is out of range was drawn with alpha 0: its sums are zero, and the unpack pass
        // skips its column anyway)
        if (s4.w != 0.f) atomicAdd(bb.g_conf_pt + row, s4.w);
        float gt[(C + 3) & ~3];
        bool any = false;
#pragma unroll
        for (int c = 0; c < ((C + 3) & ~3); c += 4)
        {
            const float4 v4 = *reinterpret_cast<const float4*>(eg + 4 + c);
            gt[c] = v4.x, gt[c + 1] = v4.y, gt[c + 2] = v4.z, gt[c + 3] = v4.w;
            any |= (v4.x != 0.f || v4.y != 0.f || v4.z != 0.f || v4.w != 0.f);
        }
        // descriptor gradients share the point's row with the position gradient: both atomics hit one 32-byte sector
        if (any) atomic_add_row<((C + 3) & ~3)>(bb.g_point + row * PS + 4, gt);
    }
    if constexpr (CAM_GRADS)
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int k = 0; k < NA; ++k)
        {
            const double v = warp_sum_d(acc[k]);
            if (lane == 0) s_acc[warp][k] = v;
        }
        __syncthreads();
        if (threadIdx.x < NA)
        {
            double v = 0.0;
            for (int w = 0; w < 8; ++w) v += s_acc[w][threadIdx.x];
            if (v != 0.0)
            {
                if (threadIdx.x < 6)
                    atomicAdd(bb.g_pose + (size_t)b * 6 + threadIdx.x, v);
                else if (threadIdx.x < 11)
                    atomicAdd(bb.g_k + (size_t)b * 5 + (threadIdx.x - 6), v);
                else
                    atomicAdd(bb.g_dis + (size_t)b * 8 + (threadIdx.x - 11), v);
            }
        }
    }
}

// per-point rows (keyed by point id) -> the reference's output layouts (PointRenderer.cu:1423-1426).  With a
// texture index the descriptor / confidence gradients of all points sharing a column are added (atomics into
// zeroed outputs); with the identity index they are plain stores.
template <int C>
__global__ __launch_bounds__(256) void unpack_point_kernel(const float* __restrict__ g_point, const float* __restrict__ g_conf_pt,
                                                           const uint32_t* __restrict__ rank, const int32_t* __restrict__ index, int N, int n_tex,
                                                           float4* __restrict__ g_points, float* __restrict__ g_size,
                                                           float* __restrict__ g_texture, float* __restrict__ g_confidence,
                                                           const float* __restrict__ raw_texture, const float* __restrict__ raw_confidence,
                                                           float confidence_scale)
{
    constexpr int PS = egrad_stride(C);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)N; i += (size_t)gridDim.x * blockDim.x)
    {
        const size_t r = rank ? (size_t)rank[i] : i;  // where the point's row lives
        const float4 v = *reinterpret_cast<const float4*>(g_point + r * PS);
        if (g_points) g_points[i] = make_float4(v.x, v.y, v.z, 0.f);
        if (g_size) g_size[i] = v.w;
        float gt[(C + 3) & ~3];
#pragma unroll
        for (int c = 0; c < ((C + 3) & ~3); c += 4)
        {
            const float4 t4 = *reinterpret_cast<const float4*>(g_point + r * PS + 4 + c);
            gt[c] = t4.x, gt[c + 1] = t4.y, gt[c + 2] = t4.z, gt[c + 3] = t4.w;
        }
        float gc = g_conf_pt[r];
        // fused texture preparation: chain through sigmoid(scale * raw) and |raw| (raw_* are null when the caller passes
        // activated tensors)
        const int col = index ? index[i] : (int)i;
        if ((unsigned)col < (unsigned)n_tex)
        {
            if (raw_confidence)
            {
                const float sg = tm_sigmoid(confidence_scale * raw_confidence[col]);
                gc             = gc * (confidence_scale * (sg * (1.f - sg)));
            }
            if (raw_texture)
            {
#pragma unroll
                for (int c = 0; c < C; ++c)
                {
                    const float w = raw_texture[(size_t)c * n_tex + col];
                    gt[c]         = w > 0.f ? gt[c] : (w < 0.f ? -gt[c] : 0.f);
                }
            }
        }
        if (!index)
        {
            if (g_texture)
            {
#pragma unroll
                for (int c = 0; c < C; ++c) g_texture[(size_t)c * n_tex + i] = gt[c];
            }
            if (g_confidence) g_confidence[i] = gc;
        }
        else
        {
            const int tex = index[i];
            if ((unsigned)tex >= (unsigned)n_tex) continue;
            if (g_texture)
            {
#pragma unroll
                for (int c = 0; c < C; ++c)
                    if (gt[c] != 0.f) atomicAdd(g_texture + (size_t)c * n_tex + tex, gt[c]);
            }
            if (g_confidence && gc != 0.f) atomicAdd(g_confidence + tex, gc);
        }
    }
}

__global__ void unpack_small_kernel(int C, int B, const CamConst* __restrict__ cams, const double* g_bg, const double* g_pose,
                                    const double* g_k, const double* g_dis, float* out_bg, double* out_pose, float* out_intr)
{
    // launched with one thread: B and C are tiny, and several views may share an image / camera index
    if (out_bg)
        for (int c = 0; c < C; ++c) out_bg[c] = (float)g_bg[c];
    for (int b = 0; b < B; ++b)
    {
        if (out_pose)
            for (int k = 0; k < 6; ++k) out_pose[(size_t)cams[b].image_index * 6 + k] += g_pose[b * 6 + k];
        if (out_intr)
        {
            for (int k = 0; k < 5; ++k) out_intr[(size_t)cams[b].camera_index * 13 + k] += (float)g_k[b * 5 + k];
            for (int k = 0; k < 8; ++k) out_intr[(size_t)cams[b].camera_index * 13 + 5 + k] += (float)g_dis[b * 8 + k];  // zero without distortion
        }
    }
}

cudaError_t launch_unpack_grads(const ScenePtrs& sc, const CamConst* cams, int B, const FwdBuffers& fb, const BwdBuffers& bb,
                                const TripsGrads& out, const TripsRenderParams& pr, int sm_count, cudaStream_t st)
{
    // the entry counts live on the device: the grid covers a fixed share of the worst case and threads stride
    {
        const bool cam_grads = out.pose_tangent || out.intrinsics;
        int bx = max(1, min(sm_count * 8 / max(1, min(B, 8)) + 1, (sc.N + 255) / 256));
        dim3 grid(bx, B);
#define TRIPS_FIN_CASE(CC)                                                                                      \
    case CC:                                                                                                    \
        if (cam_grads && pr.distortion)                                                                         \
            entry_grad_finish_kernel<CC, true, true><<<grid, 256, 0, st>>>(fb, bb, cams, B);                    \
        else if (cam_grads)                                                                                     \
            entry_grad_finish_kernel<CC, true, false><<<grid, 256, 0, st>>>(fb, bb, cams, B);                   \
        else if (pr.distortion)                                                                                 \
            entry_grad_finish_kernel<CC, false, true><<<grid, 256, 0, st>>>(fb, bb, cams, B);                   \
        else                                                                                                    \
            entry_grad_finish_kernel<CC, false, false><<<grid, 256, 0, st>>>(fb, bb, cams, B);                  \
        break;
        if (sc.N > 0)
        {
            switch (sc.C)
            {
                TRIPS_FIN_CASE(3)
                TRIPS_FIN_CASE(4)
                TRIPS_FIN_CASE(6)
                TRIPS_FIN_CASE(8)
                TRIPS_FIN_CASE(16)
                default: return cudaErrorInvalidValue;
            }
        }
#undef TRIPS_FIN_CASE
    }
    if (sc.N > 0 && (out.texture || out.confidence || out.points || out.point_size))
    {
        if (sc.index || sc.n_tex != sc.N)
        {
            // columns are accumulated (or not covered by the identity mapping): start from zero
            if (out.texture)
            {
                cudaError_t e = cudaMemsetAsync(out.texture, 0, sizeof(float) * (size_t)sc.C * sc.n_tex, st);
                if (e != cudaSuccess) return e;
            }
            if (out.confidence)
            {
                cudaError_t e = cudaMemsetAsync(out.confidence, 0, sizeof(float) * (size_t)sc.n_tex, st);
                if (e != cudaSuccess) return e;
            }
        }
        int blocks = max(1, (int)min((size_t)sm_count * 16, ((size_t)sc.N + 255) / 256));
#define TRIPS_UNPACK_CASE(CC)                                                                                           \
    case CC:                                                                                                            \
        unpack_point_kernel<CC><<<blocks, 256, 0, st>>>(bb.g_point, bb.g_conf_pt, fb.point_rank, sc.index, sc.N, sc.n_tex,   \
                                                        (float4*)out.points, out.point_size, out.texture, out.confidence, \
                                                        pr.texture_abs ? sc.texture : nullptr,                          \
                                                        pr.confidence_is_raw ? sc.confidence : nullptr, pr.confidence_scale); \
        break;
        switch (sc.C)
        {
            TRIPS_UNPACK_CASE(3)
            TRIPS_UNPACK_CASE(4)
            TRIPS_UNPACK_CASE(6)
            TRIPS_UNPACK_CASE(8)
            TRIPS_UNPACK_CASE(16)
            default: return cudaErrorInvalidValue;
        }
#undef TRIPS_UNPACK_CASE
    }
    unpack_small_kernel<<<1, 1, 0, st>>>(sc.C, B, cams, bb.g_bg, bb.g_pose, bb.g_k, bb.g_dis, out.background, out.pose_tangent,
                                         out.intrinsics);
    return cudaGetLastError();
}
}  // namespace trips
