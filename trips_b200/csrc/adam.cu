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
__device__ __forceinline__ void adam_element(const TripsAdamTensor& t, float& w, float g, float& m, float& v, int& step)
{
    if (g == 0.f) return;
    const float gsq = g * g;
    m               = t.beta1 * m + (1.f - t.beta1) * g;
    v               = t.beta2 * v + (1.f - t.beta2) * gsq;
    step            = step + 1;
    const float fs  = (float)(unsigned)step;
    const float lr  = t.lr * (sqrtf(1.f - powf(t.beta2, fs)) / (1.f - powf(t.beta1, fs)));
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
            adam_element(t, w.x, g.x, m.x, v.x, s.x);
            adam_element(t, w.y, g.y, m.y, v.y, s.y);
            adam_element(t, w.z, g.z, m.z, v.z, s.z);
            adam_element(t, w.w, g.w, m.w, v.w, s.w);
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
            adam_element(t, w, g, m, v, s);
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
            adam_element(t, w, g, m, v, s);
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
