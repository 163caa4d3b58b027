// Backward rasterizer: replays the kept fragments of every pixel and scatters gradients to descriptors,
// confidences, positions, point sizes, the background colour, the camera pose and the pinhole coefficients.
//
// Replaces BlendBackwardsBilinearTiled (src/lib/rendering/RenderBackward.cu:90-618).  Differences in structure:
//   * half-warp per pixel, lane j = j-th kept fragment; the reference's O(K^2) inner loop
//     (RenderBackward.cu:284-301) becomes a suffix sum over lanes;
//   * gradients are accumulated in row-packed buffers ([n_tex,C] and [N,4] = xyz + size) with vector atomics,
//     and transposed to the reference's layouts once per call (unpack_grads_kernel);
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
constexpr int kBwdThreads = 128;  // 4 warps: 3 x 4 x 32 x 17 floats of per-entry scratch stay below 48 KB of static shared memory
constexpr int kBwdWarps   = kBwdThreads / 32;

// One warp differentiates an 8x4 pixel tile of one view (blockIdx.y = view).
//   phase 0 (lane = kept fragment, lanes densely packed over the tile's fragments): gather the descriptor row of
//     the fragment's entry, G_j = <col_j, g> and alpha_j go to shared memory.
//   phase 1 (lane = pixel, shared memory only): the sequential recurrences over the pixel's kept fragments:
//     transmittance T_j, w_j = T_j alpha_j, and d_j = dLoss/dalpha_j = T_j G_j - (W_bg + sum_{i>j} W_i) / (1 - alpha_j + 1e-9)
//     with W_i = G_i T_i alpha_i (RenderBackward.cu:262-303; the reference's O(K^2) inner loop becomes a reverse
//     running sum).
//   phase 2 (lane = kept fragment): the per-fragment chain to descriptors, confidence, position and size
//     (RenderBackward.cu:335-466), accumulated with vector atomics into the per-entry gradient rows, which are in
//     screen-bin order like the entries and therefore stay hot in L2 while a region of the image is processed.
template <int C, bool CAM_GRADS>
__global__ __launch_bounds__(kBwdThreads) void blend_backward_kernel(ScenePtrs sc, const CamConst* __restrict__ cams,
                                                                     const __grid_constant__ Geom g, TripsRenderParams pr, int B,
                                                                     FwdBuffers fb, BwdBuffers bb,
                                                                     const __grid_constant__ ConstLayerPtrs grad_in)
{
    constexpr int ES = entry_stride(C);
    constexpr int GS = egrad_stride(C);
    __shared__ float s_g[kBwdWarps][C][32];
    __shared__ float s_d[kBwdWarps][32 * kPad];   // G_j, then dA_j = G_j T_j, finally d_j
    __shared__ float s_W[kBwdWarps][32 * kPad];   // alpha_j
    __shared__ float s_w[kBwdWarps][32 * kPad];   // w_j = T_j * alpha_j
    __shared__ CamConst s_cam;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);

    const int b = blockIdx.y;
    if (threadIdx.x < sizeof(CamConst) / 4) ((int*)&s_cam)[threadIdx.x] = ((const int*)&cams[b])[threadIdx.x];
    __syncthreads();
    const CamConst& cam  = s_cam;
    const float fxc      = cam.fx * cam.cfx;
    const size_t bP      = (size_t)b * g.P;
    const float* entries = fb.entries + fb.entry_base[b] * ES;
    float* egrad         = bb.egrad + fb.entry_base[b] * GS;
    float* my_d          = s_d[warp] + lane * kPad;
    float* my_W          = s_W[warp] + lane * kPad;
    float* my_w          = s_w[warp] + lane * kPad;

    double acc_bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) acc_bg[c] = 0.0;
    double acc_cam[CAM_GRADS ? 11 : 1];
#pragma unroll
    for (int k = 0; k < (CAM_GRADS ? 11 : 1); ++k) acc_cam[k] = 0.0;

    for (;;)
    {
        unsigned tile = 0;
        if (lane == 0) tile = atomicAdd(fb.ticket + b, 1u);
        tile = __shfl_sync(kFull, tile, 0);
        if (tile >= (unsigned)g.n_tiles) break;
        int layer, gx, gy, p;
        tile_pixel(g, (int)tile, lane, layer, gx, gy, p);
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
        __syncwarp();

        // ---- phase 0 (lane = kept fragment) ----
        for (int e0 = 0; e0 < n_entry; e0 += 32)
        {
            const int e = e0 + lane;
            int seg     = 0;
#pragma unroll
            for (int step = 16; step > 0; step >>= 1)
            {
                const int probe  = seg + step;
                const int pstart = __shfl_sync(kFull, rel, probe & 31);
                if (probe < 32 && pstart <= e) seg = probe;
            }
            const int j     = e - __shfl_sync(kFull, rel, seg);
            const int seg_p = __shfl_sync(kFull, p, seg);
            if (e < n_entry)
            {
                const uint2 rc   = fb.records[(bP + seg_p) * 16 + j];
                const float* row = entries + (size_t)rc.x * ES + 12;
                float G          = 0.f;
#pragma unroll
                for (int c = 0; c < C; c += 4)
                {
                    const float4 v4 = *reinterpret_cast<const float4*>(row + c);
                    G += v4.x * s_g[warp][c][seg];
                    if (c + 1 < C) G += v4.y * s_g[warp][c + 1][seg];
                    if (c + 2 < C) G += v4.z * s_g[warp][c + 2][seg];
                    if (c + 3 < C) G += v4.w * s_g[warp][c + 3][seg];
                }
                s_d[warp][seg * kPad + j] = G;
                s_W[warp][seg * kPad + j] = __uint_as_float(rc.y);
            }
        }
        __syncwarp();

        // ---- phase 1 (lane = pixel), forward: T_j, dA_j = G_j T_j, w_j = T_j a_j ----
        float run = 1.f;
        for (int j = 0; j < m_max; ++j)
        {
            if (j < m)
            {
                const float a = my_W[j];
                my_d[j]       = my_d[j] * run;
                my_w[j]       = run * a;
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
        for (int j = m_max - 1; j >= 0; --j)
        {
            if (j < m)
            {
                const float a   = my_W[j];
                const float dA  = my_d[j];
                const float dem = 1.f / (1.f - a + 1e-9f);
                my_d[j]         = dA - R * dem;
                R += dA * a;
            }
        }
        __syncwarp();

        // ---- phase 2 (lane = kept fragment) ----
        for (int e0 = 0; e0 < n_entry; e0 += 32)
        {
            const int e      = e0 + lane;
            const bool valid = e < n_entry;
            int seg          = 0;
#pragma unroll
            for (int step = 16; step > 0; step >>= 1)
            {
                const int probe  = seg + step;
                const int pstart = __shfl_sync(kFull, rel, probe & 31);
                if (probe < 32 && pstart <= e) seg = probe;
            }
            const int j       = e - __shfl_sync(kFull, rel, seg);
            const int seg_p   = __shfl_sync(kFull, p, seg);
            const int layer_s = __shfl_sync(kFull, layer, seg);
            const int gx_s    = __shfl_sync(kFull, gx, seg);
            const int gy_s    = __shfl_sync(kFull, gy, seg);
            if (!valid) continue;
            const uint2 rc  = fb.records[(bP + seg_p) * 16 + j];
            const float* en = entries + (size_t)rc.x * ES;
            float* eg       = egrad + (size_t)rc.x * GS;
            const float ga  = s_d[warp][seg * kPad + j];
            const float w   = s_w[warp][seg * kPad + j];
            const float4 e0v = *reinterpret_cast<const float4*>(en);      // u v ps z
            const float4 e1v = *reinterpret_cast<const float4*>(en + 4);  // pid conf raw nl
            const float4 e2v = *reinterpret_cast<const float4*>(en + 8);  // x y z tex
            if (__float_as_int(e2v.w) < 0) continue;  // invalid texture index: flagged in the forward pass, alpha was 0
            // descriptor gradient: T_j alpha_j g
            {
                float gt[(C + 3) & ~3];
#pragma unroll
                for (int c = 0; c < ((C + 3) & ~3); ++c) gt[c] = (c < C) ? w * s_g[warp][c < C ? c : 0][seg] : 0.f;
                atomic_add_row<((C + 3) & ~3)>(eg + 8, gt);
            }
            // bilinear weights and their Jacobian at uv (compute_blending_fac, PointBlending.h:216-257)
            const float fac = __int_as_float((127 - layer_s) << 23);
            const float ux = e0v.x * fac, uy = e0v.y * fac;
            const float ps = e0v.z;
            const int q    = ((float)gx_s < ux ? 0 : 1) + ((float)gy_s < uy ? 0 : 2);
            const float sx = ux - floorf(ux), sy = uy - floorf(uy);
            float bf = ((q & 1) ? sx : (1.f - sx)) * ((q & 2) ? sy : (1.f - sy));
            const float J0 = (q & 1) ? ((q & 2) ? sy : (1.f - sy)) : ((q & 2) ? -sy : (sy - 1.f));
            const float J1 = (q & 2) ? ((q & 1) ? sx : (1.f - sx)) : ((q & 1) ? -sx : (sx - 1.f));
            if (fabsf(ux - (float)gx_s) > 1.f || fabsf(uy - (float)gy_s) > 1.f) bf *= 0.f;
            const float conf = e1v.y;
            float lf_grad    = 0.f;
            const float lf   = layer_factor(ps, layer_s, g.L, &lf_grad);
            atomicAdd(eg + 4, bf * lf * ga);
            const float gbs   = conf * lf * ga;
            const float grad0 = J0 * gbs, grad1 = J1 * gbs;
            // ProjectPointPinholeBackward (PointRendererHelper.h:434-494), zero distortion
            float vx, vy, vz;
            transform_point(cam, e2v.x, e2v.y, e2v.z, vx, vy, vz);
            if (vz > 0.f)
            {
                const float g_layer_proj = fxc / vz;
                const float iz = 1.f / vz;
                const float nx = vx * iz, ny = vy * iz;
                const float gr0 = cam.r00 * grad0 + cam.r10 * grad1;
                const float gr1 = cam.r01 * grad0 + cam.r11 * grad1;
                const float gk0 = cam.cfx * gr0;
                const float gk1 = cam.cs * gr0 + cam.cfy * gr1;
                const float gn0 = cam.fx * gk0;
                const float gn1 = cam.s * gk0 + cam.fy * gk1;
                const float gv0 = iz * gn0;
                const float gv1 = iz * gn1;
                const float gv2 = (-vx * iz * iz) * gn0 + (-vy * iz * iz) * gn1;
                const float gp0 = cam.R[0] * gv0 + cam.R[3] * gv1 + cam.R[6] * gv2;
                const float gp1 = cam.R[1] * gv0 + cam.R[4] * gv1 + cam.R[7] * gv2;
                const float gp2 = cam.R[2] * gv0 + cam.R[5] * gv1 + cam.R[8] * gv2;
                const float J_sp = tm_softplus_grad(e1v.z);
                const float glp  = J_sp * g_layer_proj * lf_grad * ga;
                const float gl   = bf * conf * glp;
                atomicAdd(reinterpret_cast<float4*>(eg), make_float4(gp0, gp1, gp2, gl));
                if constexpr (CAM_GRADS)
                {
                    acc_cam[0] += (double)gv0;
                    acc_cam[1] += (double)gv1;
                    acc_cam[2] += (double)gv2;
                    acc_cam[3] += (double)(vy * gv2 - vz * gv1);
                    acc_cam[4] += (double)(vz * gv0 - vx * gv2);
                    acc_cam[5] += (double)(vx * gv1 - vy * gv0);
                    acc_cam[6] += (double)(nx * gk0);
                    acc_cam[7] += (double)(ny * gk1);
                    acc_cam[8] += (double)gk0;
                    acc_cam[9] += (double)gk1;
                    acc_cam[10] += (double)(ny * gk0);
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
    if constexpr (CAM_GRADS)
    {
#pragma unroll
        for (int k = 0; k < 11; ++k)
        {
            double v = warp_sum_d(acc_cam[k]);
            if (lane == 0 && v != 0.0)
            {
                if (k < 6)
                    atomicAdd(bb.g_pose + (size_t)b * 6 + k, v);
                else
                    atomicAdd(bb.g_k + (size_t)b * 5 + (k - 6), v);
            }
        }
    }
}

cudaError_t launch_blend_backward(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr,
                                  int B, const FwdBuffers& fb, const BwdBuffers& bb, const ConstLayerPtrs& grad_in,
                                  bool want_cam_grads, int sm_count, cudaStream_t st)
{
    cudaError_t e = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned) * B, st);
    if (e != cudaSuccess) return e;
    int bx = max(1, min((sm_count * 12 + B - 1) / B, (g.n_tiles + kBwdWarps - 1) / kBwdWarps));
    dim3 grid(bx, B);
#define TRIPS_BWD_CASE(CC)                                                                                         \
    case CC:                                                                                                       \
        if (want_cam_grads)                                                                                        \
            blend_backward_kernel<CC, true><<<grid, kBwdThreads, 0, st>>>(sc, cams, g, pr, B, fb, bb, grad_in);    \
        else                                                                                                       \
            blend_backward_kernel<CC, false><<<grid, kBwdThreads, 0, st>>>(sc, cams, g, pr, B, fb, bb, grad_in);   \
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
template <int C>
__global__ __launch_bounds__(256) void entry_grad_scatter_indirect(FwdBuffers fb, BwdBuffers bb, int B)
{
    constexpr int ES = entry_stride(C);
    constexpr int GS = egrad_stride(C);
    const unsigned long long n_total = fb.entry_base[B];
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_total;
         i += (unsigned long long)gridDim.x * blockDim.x)
    {
        const float* en = fb.entries + i * ES;
        const float* eg = bb.egrad + i * GS;
        const int pid   = __float_as_int(en[4]);
        const int tex   = __float_as_int(en[11]);
        const float4 gp = *reinterpret_cast<const float4*>(eg);
        if (gp.x != 0.f || gp.y != 0.f || gp.z != 0.f || gp.w != 0.f) atomicAdd(bb.g_pos_size + pid, gp);
        if (tex < 0) continue;
        const float gc = eg[4];
        if (gc != 0.f) atomicAdd(bb.g_conf + tex, gc);
        float gt[(C + 3) & ~3];
        bool any = false;
#pragma unroll
        for (int c = 0; c < ((C + 3) & ~3); c += 4)
        {
            const float4 v4 = *reinterpret_cast<const float4*>(eg + 8 + c);
            gt[c] = v4.x, gt[c + 1] = v4.y, gt[c + 2] = v4.z, gt[c + 3] = v4.w;
            any |= (v4.x != 0.f || v4.y != 0.f || v4.z != 0.f || v4.w != 0.f);
        }
        if (any)
        {
            float gtc[C];
#pragma unroll
            for (int c = 0; c < C; ++c) gtc[c] = gt[c];
            atomic_add_row<C>(bb.g_tex_packed + (size_t)tex * C, gtc);
        }
    }
}

template <int C>
__global__ void unpack_tex_kernel(const float* __restrict__ g_packed, int n_tex, float* __restrict__ g_texture)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n_tex; i += (size_t)gridDim.x * blockDim.x)
    {
        float v[C];
#pragma unroll
        for (int c = 0; c < C; ++c) v[c] = g_packed[i * C + c];
#pragma unroll
        for (int c = 0; c < C; ++c) g_texture[(size_t)c * n_tex + i] = v[c];
    }
}

__global__ void unpack_pos_kernel(const float4* __restrict__ g_pos_size, int N, float4* __restrict__ g_points,
                                  float* __restrict__ g_size)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)N; i += (size_t)gridDim.x * blockDim.x)
    {
        float4 v = g_pos_size[i];
        if (g_points) g_points[i] = make_float4(v.x, v.y, v.z, 0.f);
        if (g_size) g_size[i] = v.w;
    }
}

__global__ void unpack_small_kernel(int C, int B, const CamConst* __restrict__ cams, const double* g_bg, const double* g_pose,
                                    const double* g_k, float* out_bg, double* out_pose, float* out_intr)
{
    // launched with one thread: B and C are tiny, and several views may share an image / camera index
    if (out_bg)
        for (int c = 0; c < C; ++c) out_bg[c] = (float)g_bg[c];
    for (int b = 0; b < B; ++b)
    {
        if (out_pose)
            for (int k = 0; k < 6; ++k) out_pose[(size_t)cams[b].image_index * 6 + k] += g_pose[b * 6 + k];
        if (out_intr)
            for (int k = 0; k < 5; ++k) out_intr[(size_t)cams[b].camera_index * 13 + k] += (float)g_k[b * 5 + k];
    }
}

cudaError_t launch_unpack_grads(const ScenePtrs& sc, const CamConst* cams, int B, const FwdBuffers& fb, const BwdBuffers& bb,
                                const TripsGrads& out, int sm_count, cudaStream_t st)
{
    // fb.entry_base lives on the device; the launch covers the worst case and threads stop at the real count
    {
        const unsigned long long cap = (unsigned long long)B * (unsigned long long)sc.N;
        int blocks = (int)min((unsigned long long)sm_count * 16, (cap + 255) / 256);
        if (blocks > 0)
        {
            switch (sc.C)
            {
                case 3: entry_grad_scatter_indirect<3><<<blocks, 256, 0, st>>>(fb, bb, B); break;
                case 4: entry_grad_scatter_indirect<4><<<blocks, 256, 0, st>>>(fb, bb, B); break;
                case 6: entry_grad_scatter_indirect<6><<<blocks, 256, 0, st>>>(fb, bb, B); break;
                case 8: entry_grad_scatter_indirect<8><<<blocks, 256, 0, st>>>(fb, bb, B); break;
                case 16: entry_grad_scatter_indirect<16><<<blocks, 256, 0, st>>>(fb, bb, B); break;
                default: return cudaErrorInvalidValue;
            }
        }
    }
    if (out.texture)
    {
        int blocks = max(1, (int)min((size_t)148 * 16, ((size_t)sc.n_tex + 255) / 256));
        switch (sc.C)
        {
            case 3: unpack_tex_kernel<3><<<blocks, 256, 0, st>>>(bb.g_tex_packed, sc.n_tex, out.texture); break;
            case 4: unpack_tex_kernel<4><<<blocks, 256, 0, st>>>(bb.g_tex_packed, sc.n_tex, out.texture); break;
            case 6: unpack_tex_kernel<6><<<blocks, 256, 0, st>>>(bb.g_tex_packed, sc.n_tex, out.texture); break;
            case 8: unpack_tex_kernel<8><<<blocks, 256, 0, st>>>(bb.g_tex_packed, sc.n_tex, out.texture); break;
            case 16: unpack_tex_kernel<16><<<blocks, 256, 0, st>>>(bb.g_tex_packed, sc.n_tex, out.texture); break;
            default: return cudaErrorInvalidValue;
        }
    }
    if (out.confidence)
    {
        cudaError_t e = cudaMemcpyAsync(out.confidence, bb.g_conf, sizeof(float) * sc.n_tex, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return e;
    }
    if (out.points || out.point_size)
    {
        int blocks = max(1, (int)min((size_t)148 * 16, ((size_t)sc.N + 255) / 256));
        unpack_pos_kernel<<<blocks, 256, 0, st>>>(bb.g_pos_size, sc.N, (float4*)out.points, out.point_size);
    }
    unpack_small_kernel<<<1, 1, 0, st>>>(sc.C, B, cams, bb.g_bg, bb.g_pose, bb.g_k, out.background, out.pose_tangent,
                                         out.intrinsics);
    return cudaGetLastError();
}
}  // namespace trips
