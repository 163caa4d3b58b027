// Spatial rank of every point: its position in Morton order of the world-space positions.
//
// The backward pass sums the gradients of a point over views and fragments into a per-point row.  The entries that
// feed those rows are in screen-bin order, the rows would be in point-id order, and a point cloud comes in arbitrary
// order: every row update would be a read-modify-write of a random DRAM sector.  Rows are therefore stored by
// spatial rank: the points of a screen bin come from a few compact patches of the surface, i.e. from a few short rank
// ranges, and their rows stay in L2 while the bin is processed.  The rank only decides where a row lives, never a
// result, so a rank computed from positions of some steps ago is as good as a fresh one; the context refreshes it
// when the number of points changes and every few hundred forward passes.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace trips
{
// order-preserving float <-> uint encoding for atomicMin / atomicMax
__device__ __forceinline__ unsigned enc(float f)
{
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float dec(unsigned u) { return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u); }

__global__ void bbox_init_kernel(unsigned* bbox)
{
    if (threadIdx.x < 3) bbox[threadIdx.x] = 0xffffffffu;
    else if (threadIdx.x < 6) bbox[threadIdx.x] = 0u;
}

__global__ __launch_bounds__(256) void bbox_kernel(const float4* __restrict__ pos, int N, unsigned* __restrict__ bbox)
{
    unsigned lo[3] = {0xffffffffu, 0xffffffffu, 0xffffffffu}, hi[3] = {0u, 0u, 0u};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)N; i += (size_t)gridDim.x * blockDim.x)
    {
        const float4 p = pos[i];
        const float v[3] = {p.x, p.y, p.z};
#pragma unroll
        for (int k = 0; k < 3; ++k)
            if (v[k] == v[k] && fabsf(v[k]) < 3.0e38f)  // NaN / inf positions do not stretch the box
            {
                lo[k] = min(lo[k], enc(v[k]));
                hi[k] = max(hi[k], enc(v[k]));
            }
    }
#pragma unroll
    for (int k = 0; k < 3; ++k)
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            lo[k] = min(lo[k], __shfl_xor_sync(kFull, lo[k], o));
            hi[k] = max(hi[k], __shfl_xor_sync(kFull, hi[k], o));
        }
        if ((threadIdx.x & 31) == 0)
        {
            atomicMin(bbox + k, lo[k]);
            atomicMax(bbox + 3 + k, hi[k]);
        }
    }
}

__device__ __forceinline__ unsigned spread10(unsigned v)  // 10 bits -> every third bit
{
    v = (v | (v << 16)) & 0x030000ffu;
    v = (v | (v << 8)) & 0x0300f00fu;
    v = (v | (v << 4)) & 0x030c30c3u;
    v = (v | (v << 2)) & 0x09249249u;
    return v;
}

__global__ __launch_bounds__(256) void morton_kernel(const float4* __restrict__ pos, int N, const unsigned* __restrict__ bbox,
                                                     unsigned* __restrict__ keys, unsigned* __restrict__ ids)
{
    float lo[3], inv[3];
#pragma unroll
    for (int k = 0; k < 3; ++k)
    {
        lo[k]         = bbox[k] == 0xffffffffu ? 0.f : dec(bbox[k]);
        const float h = bbox[3 + k] == 0u ? 0.f : dec(bbox[3 + k]);
        const float e = h - lo[k];
        inv[k]        = e > 0.f ? 1023.f / e : 0.f;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)N; i += (size_t)gridDim.x * blockDim.x)
    {
        const float4 p = pos[i];
        const float v[3] = {p.x, p.y, p.z};
        unsigned q[3];
#pragma unroll
        for (int k = 0; k < 3; ++k)
        {
            float t = (v[k] - lo[k]) * inv[k];
            t       = (t == t) ? fminf(fmaxf(t, 0.f), 1023.f) : 0.f;
            q[k]    = (unsigned)t;
        }
        keys[i] = spread10(q[0]) | (spread10(q[1]) << 1) | (spread10(q[2]) << 2);
        ids[i]  = (unsigned)i;
    }
}

__global__ __launch_bounds__(256) void rank_scatter_kernel(const unsigned* __restrict__ sorted_ids, int N, unsigned* __restrict__ rank)
{
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < (size_t)N; j += (size_t)gridDim.x * blockDim.x) rank[sorted_ids[j]] = (unsigned)j;
}

size_t rank_temp_bytes(int N)
{
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const unsigned*)nullptr, (unsigned*)nullptr, (const unsigned*)nullptr, (unsigned*)nullptr, N, 0, 30);
    return bytes;
}

// scratch: 4 arrays of N unsigned (keys in / out, ids in / out) + 6 unsigned (bounding box); temp: rank_temp_bytes(N)
cudaError_t launch_point_rank(const float4* position, int N, unsigned* scratch, void* temp, size_t temp_bytes, unsigned* rank,
                              int sm_count, cudaStream_t st)
{
    if (N <= 0) return cudaSuccess;
    unsigned* keys_in  = scratch;
    unsigned* keys_out = scratch + (size_t)N;
    unsigned* ids_in   = scratch + 2 * (size_t)N;
    unsigned* ids_out  = scratch + 3 * (size_t)N;
    unsigned* bbox     = scratch + 4 * (size_t)N;
    const int blocks   = (int)min((size_t)sm_count * 8, ((size_t)N + 255) / 256);
    bbox_init_kernel<<<1, 32, 0, st>>>(bbox);
    bbox_kernel<<<blocks, 256, 0, st>>>(position, N, bbox);
    morton_kernel<<<blocks, 256, 0, st>>>(position, N, bbox, keys_in, ids_in);
    cudaError_t e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys_in, keys_out, ids_in, ids_out, N, 0, 30, st);
    if (e != cudaSuccess) return e;
    rank_scatter_kernel<<<blocks, 256, 0, st>>>(ids_out, N, rank);
    return cudaGetLastError();
}
}  // namespace trips
