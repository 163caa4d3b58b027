// Fused Adam over all point-parameter tensors in one launch.
//
// Per-element update of adam_step (src/lib/models/MyAdam.cu:41-88): elements whose gradient is exactly zero are
// left untouched (no moment decay, no step increment), every element has its own step counter for the bias
// correction, AdaBound clamps and relative / absolute weight decay are applied as in the reference.
// The reference launches one kernel per tensor with an int64 counter; here a block table spans all tensors and
// the counter is int32.
#include "common.cuh"

namespace trips
{
// Bias-corrected learning rate of the last step count seen by this thread: neighbouring elements (the coordinates of a
// point, the channels of a descriptor) almost always share their step count, and the two powf dominate the update.
struct LrCache
{
    int step = -1;
    float lr = 0.f;
};

__device__ __forceinline__ void adam_element(const TripsAdamTensor& t, float& w, float g, float& m, float& v, int& step, LrCache& cache)
{
    if (g == 0.f) return;
    const float gsq = g * g;
    m               = t.beta1 * m + (1.f - t.beta1) * g;
    v               = t.beta2 * v + (1.f - t.beta2) * gsq;
    step            = step + 1;
    if (step != cache.step)
    {
        const float fs = (float)(unsigned)step;
        cache.step     = step;
        cache.lr       = t.lr * (sqrtf(1.f - powf(t.beta2, fs)) / (1.f - powf(t.beta1, fs)));
    }
    const float lr  = cache.lr;
    const float eff = fminf(fmaxf(lr / (sqrtf(v) + t.eps), t.lower_lr_bound), t.upper_lr_bound);
    const float dec = (1.f - t.relative_weight_decay * lr) * w - copysignf(t.absolute_weight_decay * lr, w);
    float nw        = dec - eff * m;
    const float c   = t.weight_clipping_magnitude;
    if (c != 0.f) nw = nw < -c ? -c : (c < nw ? c : nw);
    w = nw;
}

__global__ __launch_bounds__(256) void adam_kernel(const TripsAdamTensor* __restrict__ tensors,
                                                   const int64_t* __restrict__ block_start, int n_tensors)
{
    __shared__ TripsAdamTensor t;
    __shared__ int64_t first_block;
    if (threadIdx.x == 0)
    {
        int k = 0;
        while (k + 1 < n_tensors && (int64_t)blockIdx.x >= block_start[k + 1]) ++k;
        t           = tensors[k];
        first_block = block_start[k];
    }
    __syncthreads();
    const int64_t base = ((int64_t)blockIdx.x - first_block) * kAdamPerBlock;
    const int64_t end  = min(base + (int64_t)kAdamPerBlock, t.n);
    LrCache cache;
    const bool aligned = ((((uintptr_t)t.weights) | ((uintptr_t)t.gradients) | ((uintptr_t)t.first_moments) |
                           ((uintptr_t)t.second_moments) | ((uintptr_t)t.steps)) & 15) == 0;
    if (aligned)
    {
        const int64_t end4 = base + ((end - base) & ~(int64_t)3);
        for (int64_t i = base + threadIdx.x * 4; i < end4; i += 256 * 4)
        {
            float4 g = *reinterpret_cast<const float4*>(t.gradients + i);
            if (g.x == 0.f && g.y == 0.f && g.z == 0.f && g.w == 0.f) continue;
            float4 w = *reinterpret_cast<float4*>(t.weights + i);
            float4 m = *reinterpret_cast<float4*>(t.first_moments + i);
            float4 v = *reinterpret_cast<float4*>(t.second_moments + i);
            int4 s   = *reinterpret_cast<int4*>(t.steps + i);
            adam_element(t, w.x, g.x, m.x, v.x, s.x, cache);
            adam_element(t, w.y, g.y, m.y, v.y, s.y, cache);
            adam_element(t, w.z, g.z, m.z, v.z, s.z, cache);
            adam_element(t, w.w, g.w, m.w, v.w, s.w, cache);
            *reinterpret_cast<float4*>(t.weights + i)        = w;
            *reinterpret_cast<float4*>(t.first_moments + i)  = m;
            *reinterpret_cast<float4*>(t.second_moments + i) = v;
            *reinterpret_cast<int4*>(t.steps + i)            = s;
        }
        for (int64_t i = end4 + threadIdx.x; i < end; i += 256)
        {
            float w = t.weights[i], m = t.first_moments[i], v = t.second_moments[i];
            int s   = t.steps[i];
            float g = t.gradients[i];
            if (g == 0.f) continue;
            adam_element(t, w, g, m, v, s, cache);
            t.weights[i] = w, t.first_moments[i] = m, t.second_moments[i] = v, t.steps[i] = s;
        }
    }
    else
    {
        for (int64_t i = base + threadIdx.x; i < end; i += 256)
        {
            float g = t.gradients[i];
            if (g == 0.f) continue;
            float w = t.weights[i], m = t.first_moments[i], v = t.second_moments[i];
            int s   = t.steps[i];
            adam_element(t, w, g, m, v, s, cache);
            t.weights[i] = w, t.first_moments[i] = m, t.second_moments[i] = v, t.steps[i] = s;
        }
    }
}

cudaError_t launch_adam(const TripsAdamTensor* d_tensors, const int64_t* d_block_start, int n_tensors, int64_t total_blocks,
                        cudaStream_t st)
{
    if (total_blocks <= 0) return cudaSuccess;
    adam_kernel<<<(unsigned)total_blocks, 256, 0, st>>>(d_tensors, d_block_start, n_tensors);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// Gradient sum over ranks + Adam + parameter broadcast in ONE kernel over peer memory (NVLink / NVSwitch).
//
// Every rank owns the slice [lo, hi) of the flat parameter space (and only that slice of the Adam state).  For its
// slice it reads the gradient of every rank through peer pointers (plain P2P loads, summed in rank order, so that
// all replicas see bit-identical sums), applies the reference update (adam_step, MyAdam.cu:41-88; elements whose
// summed gradient is zero stay untouched) and stores the new weight into the parameter buffer of every rank (P2P
// stores).  This is reduce-scatter + sharded Adam + all-gather with the wire traffic of one all-reduce and 1/G of
// the optimizer traffic per GPU.  The kernel never waits on another GPU: the caller orders it after every rank's
// backward pass and orders the next forward pass after it on every rank (a barrier on both sides).
// ------------------------------------------------------------------------------------------------------------
struct FusedArgs
{
    const float* grad[TRIPS_MAX_RANKS];
    float* param[TRIPS_MAX_RANKS];
    TripsAdamSegment seg[TRIPS_MAX_SEGMENTS];
    int world, rank, n_seg;
    int64_t lo, hi;
};

__device__ __forceinline__ void fused_element(const TripsAdamSegment& sg, float& w, float g, float& m, float& v, int& step, LrCache& cache)
{
    TripsAdamTensor t;
    t.lr = sg.lr, t.beta1 = sg.beta1, t.beta2 = sg.beta2, t.eps = sg.eps;
    t.relative_weight_decay = sg.relative_weight_decay, t.absolute_weight_decay = sg.absolute_weight_decay;
    t.weight_clipping_magnitude = sg.weight_clipping_magnitude;
    t.lower_lr_bound = sg.lower_lr_bound, t.upper_lr_bound = sg.upper_lr_bound;
    adam_element(t, w, g, m, v, step, cache);
}

// W: compile-time bound of the number of ranks (2, 4, 8 or 16), so that the gradient loads of all ranks are issued
// before the first one is used (one round trip over NVLink per vector instead of `world` in a row).
template <int W>
__global__ __launch_bounds__(256) void fused_reduce_adam_kernel(const __grid_constant__ FusedArgs a, float* __restrict__ m_state,
                                                                float* __restrict__ v_state, int32_t* __restrict__ steps)
{
    // 16-byte vectors over the aligned interior of [lo, hi), scalars at the ragged ends
    const int64_t lo4 = min(a.hi, (a.lo + 3) & ~(int64_t)3), hi4 = max(lo4, a.hi & ~(int64_t)3);
    const int64_t n_vec = (hi4 - lo4) >> 2;
    auto segment_of = [&](int64_t i) {
        int k = 0;
        for (int s = 1; s < a.n_seg; ++s)
            if (i >= a.seg[s].offset) k = s;
        return k;
    };
    LrCache cache;
    int cache_seg = -1;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n_vec; q += (int64_t)gridDim.x * blockDim.x)
    {
        const int64_t i = lo4 + 4 * q;
        float4 part[W];
#pragma unroll
        for (int r = 0; r < W; ++r)
            part[r] = r < a.world ? *reinterpret_cast<const float4*>(a.grad[r] + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 g = part[0];  // summed in rank order on every rank: all replicas see the same bits
#pragma unroll
        for (int r = 1; r < W; ++r)
            if (r < a.world) g.x += part[r].x, g.y += part[r].y, g.z += part[r].z, g.w += part[r].w;
        if (g.x == 0.f && g.y == 0.f && g.z == 0.f && g.w == 0.f) continue;  // unseen on every rank: nothing moves anywhere
        const int64_t j = i - a.lo;  // the optimizer state is stored for the owned slice only
        float4 w = *reinterpret_cast<const float4*>(a.param[a.rank] + i);
        float mm[4], vv[4];
        int ss[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) mm[k] = m_state[j + k], vv[k] = v_state[j + k], ss[k] = steps[j + k];
        const int s0 = segment_of(i), s3 = segment_of(i + 3);
        if (s0 != s3 || s0 != cache_seg) cache.step = -1;  // the cached learning rate belongs to one segment
        cache_seg = s3;
        fused_element(a.seg[s0], w.x, g.x, mm[0], vv[0], ss[0], cache);
        if (s0 != s3) cache.step = -1;
        fused_element(a.seg[s0 == s3 ? s0 : segment_of(i + 1)], w.y, g.y, mm[1], vv[1], ss[1], cache);
        if (s0 != s3) cache.step = -1;
        fused_element(a.seg[s0 == s3 ? s0 : segment_of(i + 2)], w.z, g.z, mm[2], vv[2], ss[2], cache);
        if (s0 != s3) cache.step = -1;
        fused_element(a.seg[s3], w.w, g.w, mm[3], vv[3], ss[3], cache);
#pragma unroll
        for (int k = 0; k < 4; ++k) m_state[j + k] = mm[k], v_state[j + k] = vv[k], steps[j + k] = ss[k];
        for (int r = 0; r < a.world; ++r) *reinterpret_cast<float4*>(a.param[r] + i) = w;
    }
    // ragged ends (at most 3 + 3 elements)
    const int64_t n_edge = (lo4 - a.lo) + (a.hi - hi4);
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n_edge; q += (int64_t)gridDim.x * blockDim.x)
    {
        const int64_t i = q < (lo4 - a.lo) ? a.lo + q : hi4 + (q - (lo4 - a.lo));
        float g = a.grad[0][i];
        for (int r = 1; r < a.world; ++r) g += a.grad[r][i];
        if (g == 0.f) continue;
        const int64_t j = i - a.lo;
        float w = a.param[a.rank][i], mm = m_state[j], vv = v_state[j];
        int ss = steps[j];
        LrCache one;
        fused_element(a.seg[segment_of(i)], w, g, mm, vv, ss, one);
        m_state[j] = mm, v_state[j] = vv, steps[j] = ss;
        for (int r = 0; r < a.world; ++r) a.param[r][i] = w;
    }
}

cudaError_t launch_fused_reduce_adam(const float* const* grad_ptrs, float* const* param_ptrs, int world, int rank,
                                     const TripsAdamSegment* segs, int n_seg, int64_t lo, int64_t hi, float* m_state,
                                     float* v_state, int32_t* steps, int sm_count, cudaStream_t st)
{
    if (hi <= lo) return cudaSuccess;
    FusedArgs a{};
    for (int r = 0; r < world; ++r) a.grad[r] = grad_ptrs[r], a.param[r] = param_ptrs[r];
    for (int s = 0; s < n_seg; ++s) a.seg[s] = segs[s];
    a.world = world, a.rank = rank, a.n_seg = n_seg, a.lo = lo, a.hi = hi;
    const int64_t n_vec = (hi - lo + 3) / 4;
    const int blocks    = (int)max((int64_t)1, min((int64_t)sm_count * 8, (n_vec + 255) / 256));
    if (world <= 2)
        fused_reduce_adam_kernel<2><<<blocks, 256, 0, st>>>(a, m_state, v_state, steps);
    else if (world <= 4)
        fused_reduce_adam_kernel<4><<<blocks, 256, 0, st>>>(a, m_state, v_state, steps);
    else if (world <= 8)
        fused_reduce_adam_kernel<8><<<blocks, 256, 0, st>>>(a, m_state, v_state, steps);
    else
        fused_reduce_adam_kernel<16><<<blocks, 256, 0, st>>>(a, m_state, v_state, steps);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// The same step through NVSwitch multicast addresses (multimem): the gradient buffers of all ranks are bound to one
// multicast object and so are the parameter replicas.  A rank fetches its slice of the gradient with
// multimem.ld_reduce (the switch reads the 16 bytes from every GPU and returns their sum) and writes the new weights
// with multimem.st (one store, delivered to every replica).  Per GPU and direction the links then carry the slice
// once per peer for the reduction plus once for the broadcast, half of what the peer-pointer kernel above moves
// (which also sends every new weight to each peer separately and receives each peer's partial gradients separately);
// with 8 ranks that kernel sits at the link bandwidth.  The switch adds in an order of its own, so weights equal the
// peer-pointer kernel's bit for bit only with two ranks; every replica receives the owner's bits, so replicas stay
// identical with any number of ranks.  Ordering is the caller's, as above; the kernel waits on nothing.
// ------------------------------------------------------------------------------------------------------------
struct McArgs
{
    const float* grad_mc;   // multicast address of the flat gradient buffers
    float* param_mc;        // multicast address of the flat parameter replicas
    const float* param;     // this rank's replica
    TripsAdamSegment seg[TRIPS_MAX_SEGMENTS];
    int n_seg;
    int64_t lo, hi;
};

__device__ __forceinline__ float4 multimem_sum4(const float* mc)
{
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
__device__ __forceinline__ void multimem_store4(float* mc, const float4& v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__global__ __launch_bounds__(256) void fused_multicast_adam_kernel(const __grid_constant__ McArgs a, float* __restrict__ m_state,
                                                                   float* __restrict__ v_state, int32_t* __restrict__ steps)
{
    // [lo, hi) is a whole number of 16-byte vectors (checked by the host)
    const int64_t n_vec = (a.hi - a.lo) >> 2;
    auto segment_of = [&](int64_t i) {
        int k = 0;
        for (int s = 1; s < a.n_seg; ++s)
            if (i >= a.seg[s].offset) k = s;
        return k;
    };
    LrCache cache;
    int cache_seg = -1;
    // kMcUnroll reductions per thread are in flight before the first is used: a multimem.ld_reduce is a round trip through
    // the switch to every GPU, several times the latency of a peer load
    constexpr int kMcUnroll = 4;
    const int64_t stride    = (int64_t)gridDim.x * blockDim.x;
    for (int64_t q0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q0 < n_vec; q0 += stride * kMcUnroll)
    {
        float4 gs[kMcUnroll];
#pragma unroll
        for (int u = 0; u < kMcUnroll; ++u)
            gs[u] = (q0 + u * stride < n_vec) ? multimem_sum4(a.grad_mc + a.lo + 4 * (q0 + u * stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < kMcUnroll; ++u)
        {
            const int64_t q = q0 + u * stride;
            if (q >= n_vec) break;
            const int64_t i = a.lo + 4 * q;
            const float4 g  = gs[u];
            if (g.x == 0.f && g.y == 0.f && g.z == 0.f && g.w == 0.f) continue;  // unseen on every rank: nothing moves anywhere
            const int64_t j = i - a.lo;
            const float4 w  = *reinterpret_cast<const float4*>(a.param + i);
            float gg[4]     = {g.x, g.y, g.z, g.w};
            float ww[4]     = {w.x, w.y, w.z, w.w};
            float mm[4], vv[4];
            int ss[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) mm[k] = m_state[j + k], vv[k] = v_state[j + k], ss[k] = steps[j + k];
            const int s0 = segment_of(i), s3 = segment_of(i + 3);
            if (s0 != s3 || s0 != cache_seg) cache.step = -1;  // the cached learning rate belongs to one segment
            cache_seg = s3;
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                if (k > 0 && s0 != s3) cache.step = -1;
                fused_element(a.seg[s0 == s3 ? s0 : segment_of(i + k)], ww[k], gg[k], mm[k], vv[k], ss[k], cache);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) m_state[j + k] = mm[k], v_state[j + k] = vv[k], steps[j + k] = ss[k];
            multimem_store4(a.param_mc + i, make_float4(ww[0], ww[1], ww[2], ww[3]));
        }
    }
}

cudaError_t launch_fused_multicast_adam(const float* grad_mc, float* param_mc, const float* param, const TripsAdamSegment* segs, int n_seg,
                                        int64_t lo, int64_t hi, float* m_state, float* v_state, int32_t* steps, int sm_count, cudaStream_t st)
{
    if (hi <= lo) return cudaSuccess;
    McArgs a{};
    a.grad_mc = grad_mc, a.param_mc = param_mc, a.param = param;
    for (int s = 0; s < n_seg; ++s) a.seg[s] = segs[s];
    a.n_seg = n_seg, a.lo = lo, a.hi = hi;
    const int64_t n_vec = (hi - lo) / 4;
    const int blocks    = (int)max((int64_t)1, min((int64_t)sm_count * 8, (n_vec + 255) / 256));
    fused_multicast_adam_kernel<<<blocks, 256, 0, st>>>(a, m_state, v_state, steps);
    return cudaGetLastError();
}

// L1 loss against a target pyramid and its gradient, all layers in one launch (benchmark helper).
__global__ __launch_bounds__(256) void l1_loss_kernel(const __grid_constant__ L1Args a, int64_t total, float inv_total,
                                                      double* __restrict__ loss_out)
{
    double acc = 0.0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    {
        int l = 0;
#pragma unroll
        for (int k = 1; k < TRIPS_MAX_LAYERS; ++k)
            if (k < a.L && i >= a.start[k]) l = k;
        const int64_t j = i - a.start[l];
        const float d   = a.out[l][j] - a.target[l][j];
        a.grad[l][j]    = d > 0.f ? inv_total : (d < 0.f ? -inv_total : 0.f);
        acc += (double)fabsf(d);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
    __shared__ double s[8];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += s[w];
        atomicAdd(loss_out, t * (double)inv_total);
    }
}

cudaError_t launch_l1_loss(const L1Args& a, int64_t total, double* loss_out, int sm_count, cudaStream_t st)
{
    if (total <= 0) return cudaSuccess;
    int blocks = (int)min((int64_t)sm_count * 8, (total + 255) / 256);
    l1_loss_kernel<<<blocks, 256, 0, st>>>(a, total, 1.0f / (float)total, loss_out);
    return cudaGetLastError();
}
}  // namespace trips
