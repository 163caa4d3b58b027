// Top-K selection and blend by the rules of the reference's SECOND forward pipeline
// (FastSortAndBlendWPrep2WarpSharedWork, src/lib/rendering/RenderForward.cu:3080-3674), which the reference runs when
// use_layer_point_size, render_points_in_all_lower_resolutions or combine_lists differ from their defaults
// (PointRenderer.cu:730-731).  It differs from the first pipeline's blend in four places:
//   * combine_lists: a pixel of layer l draws its 16 nearest fragments from its own list and from the lists of the
//     pixels above it, (gx >> k, gy >> k) on layer l + k (RenderForward.cu:3232-3242); every fragment is weighted as if
//     it lay on layer l, and fragments more than a pixel away get alpha 0 but keep their place in the list;
//   * the bilinear weight is the corner weight picked by blend_fac_index from the sub-pixel position
//     (RenderForward.cu:3493-3496, PointBlending.h:216-263), which is 0 on both pixels for an integer coordinate;
//   * saturated_alpha_accumulation (RenderForward.cu:3524-3548): weights 1 until the alphas sum to 1, the crossing
//     fragment gets saturate(1) / (alpha + 1e-9) as the reference computes it, 0 below the cut-off;
//   * without use_layer_point_size the alpha carries no layer factor.
// The lists themselves come from the same binning / count / collect passes as in the first pipeline (with the strict
// two-layer write where asked); the alpha stored in the fragments is not used here because it belongs to the
// fragment's own layer and pixel.  These flags are off in every shipped configuration of the reference, so this kernel
// is written for clarity: one thread per pixel, insertion into a sorted array of at most 16 keys.
#include "common.cuh"

namespace trips
{
namespace
{
template <int C>
__global__ __launch_bounds__(128) void second_blend_kernel(ScenePtrs sc, const __grid_constant__ Geom g, TripsRenderParams pr, int B, FwdBuffers fb,
                                                           const __grid_constant__ LayerPtrs out)
{
    constexpr int ES = tail_stride(C);
    const int K      = pr.k_keep;
    const size_t total = (size_t)B * (size_t)g.P;
    float bg[C];
#pragma unroll
    for (int c = 0; c < C; ++c) bg[c] = __ldg(sc.background + c);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    {
        const int b = (int)(idx / (size_t)g.P);
        const int p = (int)(idx - (size_t)b * g.P);
        int layer   = 0;
        while (layer + 1 < g.L && p >= g.base[layer + 1]) ++layer;
        const int t  = p - g.base[layer];
        const int gy = t / g.W[layer], gx = t - gy * g.W[layer];
        const size_t bP        = (size_t)b * g.P;
        const uint4* frags     = fb.frags + fb.view_base[b];
        const float4* head     = fb.ent_head + fb.entry_base[b] * 2;
        const float* tail      = fb.ent_tail + fb.entry_base[b] * ES;
        const uint32_t n_entry = (uint32_t)(fb.entry_base[b + 1] - fb.entry_base[b]);

        // ---- the K nearest fragments by (depth bits, point id) ----
        unsigned long long key[TRIPS_MAX_KEEP];
        uint32_t ent[TRIPS_MAX_KEEP];
        int n = 0;
        if (fb.view_base[b + 1] != fb.view_base[b])  // (a view that did not fit the list buffer renders as background)
        {
            int x = gx, y = gy;
            for (int l2 = layer; l2 < g.L; ++l2, x >>= 1, y >>= 1)
            {
                const int q          = g.base[l2] + y * g.W[l2] + x;
                const uint32_t cnt   = fb.counts[bP + q];
                const uint32_t start = fb.offsets[bP + q] - cnt;  // offsets hold list ends after the collect pass
                for (uint32_t f = 0; f < cnt; ++f)
                {
                    const uint4 fr             = frags[start + f];
                    const unsigned long long k = ((unsigned long long)fr.y << 32) | fr.x;
                    if (n == K && k >= key[n - 1]) continue;
                    int j = (n < K) ? n : K - 1;
                    while (j > 0 && key[j - 1] > k)
                    {
                        key[j] = key[j - 1];
                        ent[j] = ent[j - 1];
                        --j;
                    }
                    key[j] = k;
                    ent[j] = fr.w;
                    if (n < K) ++n;
                }
                if (!pr.combine_lists) break;
            }
        }

        // ---- alpha of every kept fragment on THIS pixel's layer ----
        float al[TRIPS_MAX_KEEP], w[TRIPS_MAX_KEEP];
        const float fac = __int_as_float((127 - layer) << 23);
        for (int j = 0; j < n; ++j)
        {
            if (ent[j] >= n_entry)
            {
                atomicOr(&fb.stats->status, TRIPS_DEV_BAD_FRAGMENT);  // corrupted list: contributes nothing
                ent[j] = 0;
                al[j]  = 0.f;
                continue;
            }
            const float4 e0 = head[2 * (size_t)ent[j]];  // u v ps conf
            const float ux = e0.x * fac, uy = e0.y * fac;
            const float sx = ux - floorf(ux), sy = uy - floorf(uy);
            const int q    = ((float)gx < ux ? 0 : 1) + ((float)gy < uy ? 0 : 2);
            float bf       = ((q & 1) ? sx : (1.f - sx)) * ((q & 2) ? sy : (1.f - sy));
            if (fabsf(ux - (float)gx) > 1.f || fabsf(uy - (float)gy) > 1.f) bf = 0.f;
            float a = bf * e0.w;
            if (pr.use_layer_point_size) a *= layer_factor(e0.z, layer, g.L, nullptr);
            al[j] = a;
        }

        // ---- weights ----
        float run = 1.f;
        if (pr.saturated_alpha_accumulation)
        {
            for (int j = 0; j < n; ++j)
            {
                if (j > 0) run = run - al[j - 1];
                if (j == 0)
                    w[j] = 1.f;
                else if (run >= kAlphaCut)
                    w[j] = (run - al[j] > 0.f) ? 1.f : (float)(1.0 / ((double)al[j] + 1e-9));
                else
                    w[j] = 0.f;
            }
        }
        else
        {
            for (int j = 0; j < n; ++j)
            {
                if (j > 0) run = run * (1.f - al[j - 1]);
                w[j] = (j == 0 || run >= kAlphaCut) ? run : 0.f;
            }
        }

        // ---- colour: pairwise tree over the 16 slots (the reference's xor-shuffle sum, RenderForward.cu:3608-3620), then
        //      the background weighted like the LAST kept fragment (RenderForward.cu:3630-3647) ----
        const float wb = (n == 0) ? 1.f : w[n - 1];
        const int Wl = g.W[layer], Hl = g.H[layer];
        float* o = out.p[layer] + ((size_t)b * C * Hl + gy) * Wl + gx;
#pragma unroll
        for (int c = 0; c < C; ++c)
        {
            float leaf[TRIPS_MAX_KEEP];
#pragma unroll
            for (int j = 0; j < TRIPS_MAX_KEEP; ++j) leaf[j] = (j < n) ? w[j] * al[j] * tail[(size_t)ent[j] * ES + 4 + c] : 0.f;
#pragma unroll
            for (int off = 1; off < TRIPS_MAX_KEEP; off *= 2)
#pragma unroll
                for (int j = 0; j < TRIPS_MAX_KEEP; j += 2 * off) leaf[j] = leaf[j] + leaf[j + off];
            float v = leaf[0];
            if (wb >= kAlphaCut) v += bg[c] * (wb * 1.f);
            o[(size_t)c * Hl * Wl] = v;
        }

        // ---- records for the backward pass: the leading fragments whose weight is above the cut-off ----
        if (pr.train)
        {
            int m = 0;
            while (m < n && w[m] >= kAlphaCut)
            {
                fb.records[(bP + p) * 16 + m] = make_uint2(ent[m], __float_as_uint(al[m]));
                ++m;
            }
            fb.rec_n[bP + p] = (uint8_t)m;
        }
    }
}
}  // namespace

cudaError_t launch_second_blend(const ScenePtrs& sc, const Geom& g, const TripsRenderParams& pr, int B, const FwdBuffers& fb,
                                const LayerPtrs& out, int sm_count, cudaStream_t st)
{
    const size_t total = (size_t)B * (size_t)g.P;
    const int blocks   = (int)std::max<size_t>(1, std::min<size_t>((size_t)sm_count * 16, (total + 127) / 128));
    switch (sc.C)
    {
        case 3: second_blend_kernel<3><<<blocks, 128, 0, st>>>(sc, g, pr, B, fb, out); break;
        case 4: second_blend_kernel<4><<<blocks, 128, 0, st>>>(sc, g, pr, B, fb, out); break;
        case 6: second_blend_kernel<6><<<blocks, 128, 0, st>>>(sc, g, pr, B, fb, out); break;
        case 8: second_blend_kernel<8><<<blocks, 128, 0, st>>>(sc, g, pr, B, fb, out); break;
        case 16: second_blend_kernel<16><<<blocks, 128, 0, st>>>(sc, g, pr, B, fb, out); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
}  // namespace trips
