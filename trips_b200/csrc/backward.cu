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

template <int C, bool CAM_GRADS>
__global__ __launch_bounds__(256) void blend_backward_kernel(ScenePtrs sc, const CamConst* __restrict__ cams, const __grid_constant__ Geom g,
                                                             TripsRenderParams pr, int B, FwdBuffers fb, BwdBuffers bb,
                                                             const __grid_constant__ ConstLayerPtrs grad_in, unsigned n_tiles,
                                                             unsigned tiles_per_view)
{
    __shared__ float s_g[8][C][32];
    __shared__ CamConst s_cam;
    __shared__ int s_cam_view;
    const int lane  = threadIdx.x & 31;
    const int warp  = threadIdx.x >> 5;
    const int j     = lane & 15;
    const int hbase = lane & 16;
    const int K     = pr.k_keep;
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);

    // Every block works on the tiles of one view at a time (blockIdx.y = view), so the camera lives in shared
    // memory and the per-view camera / background gradients are reduced once per block.
    const int b = blockIdx.y;
    if (threadIdx.x < sizeof(CamConst) / 4) ((int*)&s_cam)[threadIdx.x] = ((const int*)&cams[b])[threadIdx.x];
    if (threadIdx.x == 0) s_cam_view = b;
    __syncthreads();
    const CamConst& cam = s_cam;
    const float fxc     = cam.fx * cam.cfx;
    const size_t bP     = (size_t)b * g.P;
    const size_t bN     = (size_t)b * sc.N;

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
        if (tile >= tiles_per_view) break;
        const int p0     = tile * 32;
        const int p_mine = p0 + lane;
        int m_mine = 0, layer_mine = 0, gx_mine = 0, gy_mine = 0;
        if (p_mine < g.P)
        {
            m_mine = fb.rec_n[bP + p_mine];
            pixel_to_layer(g, p_mine, layer_mine, gx_mine, gy_mine);
            const int Wl = g.W[layer_mine], Hl = g.H[layer_mine];
            const float* gi = grad_in.p[layer_mine] + ((size_t)b * C * Hl + gy_mine) * Wl + gx_mine;
#pragma unroll
            for (int c = 0; c < C; ++c) s_g[warp][c][lane] = __ldg(gi + (size_t)c * Hl * Wl);
        }
        __syncwarp();
        for (int it = 0; it < 16; ++it)
        {
            const int src   = it * 2 + (hbase >> 4);
            const int m     = __shfl_sync(kFull, m_mine, src);
            const int layer = __shfl_sync(kFull, layer_mine, src);
            const int gx    = __shfl_sync(kFull, gx_mine, src);
            const int gy    = __shfl_sync(kFull, gy_mine, src);
            const int p     = p0 + src;
            const int m_o   = __shfl_xor_sync(kFull, m, 16);
            if (p0 + it * 2 >= g.P) break;
            const bool pix_ok = p < g.P;
            const bool active = pix_ok && j < m;
            float gin[C];
#pragma unroll
            for (int c = 0; c < C; ++c) gin[c] = s_g[warp][c][src];

            float a = 0.f;
            int pid = 0, tex = 0;
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
            float col[C];
#pragma unroll
            for (int c = 0; c < C; ++c) col[c] = 0.f;
            if (active)
            {
                uint2 rc = fb.records[(bP + p) * 16 + j];
                pid      = (int)rc.x;
                a        = __uint_as_float(rc.y);
                r        = fb.rec[bN + pid];
                tex      = __float_as_int(r.w);
                const float* row = fb.tex_packed + (size_t)tex * C;
#pragma unroll
                for (int c = 0; c < C; ++c) col[c] = __ldg(row + c);
            }
            // transmittance before my fragment, and after the last kept fragment (run)
            const int m_max = max(m, m_o);
            float run = 1.f, T = 1.f;
            for (int s = 1; s <= m_max; ++s)
            {
                float am = __shfl_sync(kFull, a, hbase | ((s - 1) & 15));
                run      = (1.f - am) * run;
                if (j == s) T = run;
            }
            // after the loop `run` includes the other half's extra (1 - 0) factors only: it equals T_m of my pixel
            float G = 0.f, Wj = 0.f;
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                G += col[c] * gin[c];
                Wj += gin[c] * col[c] * T * a;
            }
            if (!active) Wj = 0.f;
            const bool has_bg = pix_ok && run >= kAlphaCut;  // background step with alpha = 1 (RenderBackward.cu:205-210)
            float Wbg = 0.f;
            if (has_bg)
            {
#pragma unroll
                for (int c = 0; c < C; ++c) Wbg += gin[c] * bg[c] * run * 1.f;
                if (j == 0)
                {
#pragma unroll
                    for (int c = 0; c < C; ++c) acc_bg[c] += (double)(run * 1.f * gin[c]);
                }
            }
            // suffix sum over later fragments: R_j = sum_{i>j} W_i + W_bg
            float S = Wj;
#pragma unroll
            for (int o = 1; o < 16; o <<= 1)
            {
                float t = __shfl_down_sync(kFull, S, o, 16);
                if (j + o < 16) S += t;
            }
            float R = __shfl_down_sync(kFull, S, 1, 16);
            if (j == 15) R = 0.f;
            R += Wbg;
            if (active)
            {
                const float dem = 1.f / (1.f - a + 1e-9f);
                const float ga  = G * T - R * dem;  // d loss / d alpha_j
                // descriptor gradient
                {
                    float gt[C];
                    const float w = T * a;
#pragma unroll
                    for (int c = 0; c < C; ++c) gt[c] = w * gin[c];
                    atomic_add_row<C>(bb.g_tex_packed + (size_t)tex * C, gt);
                }
                // bilinear weights and their Jacobian at uv (compute_blending_fac, PointBlending.h:216-257)
                const float fac = __int_as_float((127 - layer) << 23);
                const float ux = r.x * fac, uy = r.y * fac;
                const float ps = r.z;
                const int q    = ((float)gx < ux ? 0 : 1) + ((float)gy < uy ? 0 : 2);
                const float sx = ux - floorf(ux), sy = uy - floorf(uy);
                float bf = ((q & 1) ? sx : (1.f - sx)) * ((q & 2) ? sy : (1.f - sy));
                float J0 = (q & 1) ? ((q & 2) ? sy : (1.f - sy)) : ((q & 2) ? -sy : (sy - 1.f));
                float J1 = (q & 2) ? ((q & 1) ? sx : (1.f - sx)) : ((q & 1) ? -sx : (sx - 1.f));
                if (fabsf(ux - (float)gx) > 1.f || fabsf(uy - (float)gy) > 1.f) bf *= 0.f;
                const float conf = __ldg(sc.confidence + tex);
                float lf_grad    = 0.f;
                const float lf   = layer_factor(ps, layer, g.L, &lf_grad);
                atomicAdd(bb.g_conf + tex, bf * lf * ga);
                const float gbs   = conf * lf * ga;
                const float grad0 = J0 * gbs, grad1 = J1 * gbs;
                // ProjectPointPinholeBackward (PointRendererHelper.h:434-494), zero distortion
                const float4 pos = __ldg(sc.position + pid);
                float vx, vy, vz;
                transform_point(cam, pos.x, pos.y, pos.z, vx, vy, vz);
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
                    const float J_sp = tm_softplus_grad(__ldg(sc.point_size + pid));
                    const float glp  = J_sp * g_layer_proj * lf_grad * ga;
                    const float gl   = bf * conf * glp;
                    atomicAdd(bb.g_pos_size + pid, make_float4(gp0, gp1, gp2, gl));
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
        }
        __syncwarp();
    }
    // per-block reduction of the view-level gradients: warp shuffle, then one double atomic per warp
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
    (void)K;
    (void)s_cam_view;
}

cudaError_t launch_blend_backward(const ScenePtrs& sc, const CamConst* cams, const Geom& g, const TripsRenderParams& pr,
                                  int B, const FwdBuffers& fb, const BwdBuffers& bb, const ConstLayerPtrs& grad_in,
                                  bool want_cam_grads, int sm_count, cudaStream_t st)
{
    unsigned tiles_per_view = (unsigned)((g.P + 31) / 32);
    unsigned n_tiles        = tiles_per_view * (unsigned)B;
    cudaError_t e           = cudaMemsetAsync(fb.ticket, 0, sizeof(unsigned) * B, st);
    if (e != cudaSuccess) return e;
    int bx = max(1, min((sm_count * 8 + B - 1) / B, (int)((tiles_per_view + 7) / 8)));
    dim3 grid(bx, B);
#define TRIPS_BWD_CASE(CC)                                                                                                \
    case CC:                                                                                                              \
        if (want_cam_grads)                                                                                               \
            blend_backward_kernel<CC, true><<<grid, 256, 0, st>>>(sc, cams, g, pr, B, fb, bb, grad_in, n_tiles, tiles_per_view); \
        else                                                                                                              \
            blend_backward_kernel<CC, false><<<grid, 256, 0, st>>>(sc, cams, g, pr, B, fb, bb, grad_in, n_tiles, tiles_per_view); \
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
// packed gradient buffers -> the reference's output layouts (PointRenderer.cu:1423-1426)
// ------------------------------------------------------------------------------------------------------------
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

cudaError_t launch_unpack_grads(const ScenePtrs& sc, const CamConst* cams, int B, const BwdBuffers& bb,
                                const TripsGrads& out, cudaStream_t st)
{
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
