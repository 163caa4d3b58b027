// Point removal / growth for all per-point tensors of a scene and their optimizer state in one pass on the device.
//
// The reference removes points by sorting the indices on the host, erasing mesh vertices on the CPU, rebuilding the
// point cloud, and running one index_select (plus allocation) per tensor: texture, confidence, point size and the
// three Adam state tensors of every texture parameter (NeuralScene.cpp:1375-1431, NeuralTexture.cpp:195-208,
// MyAdam.cu:346-373); growth appends columns filled with a constant (NeuralTexture.cpp:153-193, MyAdam.cu:376-415).
// Here: mark the removed points, scan the keep flags, and gather every tensor (parameters and optimizer state,
// point-major [N, rows] or planar [rows, N]) into caller-provided destinations with one launch; columns beyond the
// kept points are filled with the tensor's constant.  Order of the kept points is preserved, as index_select with an
// ascending index list does.
#include "common.cuh"

namespace trips
{
constexpr int kResizeItems = 4096;  // flags per block in the scan passes

__global__ __launch_bounds__(256) void mark_removed_kernel(const int64_t* __restrict__ remove, int64_t n_remove, int64_t n_points,
                                                           uint8_t* __restrict__ keep, DevStats* stats)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_remove; i += (int64_t)gridDim.x * blockDim.x)
    {
        const int64_t r = remove[i];
        if (r < 0 || r >= n_points)
            atomicOr(&stats->status, TRIPS_DEV_BAD_POINT_INDEX);
        else
            keep[r] = 0;
    }
}

__global__ __launch_bounds__(256) void keep_count_kernel(const uint8_t* __restrict__ keep, int64_t n, uint32_t* __restrict__ block_sum)
{
    const int64_t base = (int64_t)blockIdx.x * kResizeItems;
    uint32_t c = 0;
    for (int k = threadIdx.x; k < kResizeItems; k += 256)
        if (base + k < n) c += keep[base + k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(kFull, c, o);
    __shared__ uint32_t s[8];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        uint32_t t = 0;
        for (int w = 0; w < 8; ++w) t += s[w];
        block_sum[blockIdx.x] = t;
    }
}

// one block: exclusive scan of the block sums in place; total -> *n_keep
__global__ __launch_bounds__(1024) void keep_scan_kernel(uint32_t* __restrict__ block_sum, int n_blocks, uint32_t* __restrict__ n_keep,
                                                         uint32_t expected, DevStats* stats)
{
    __shared__ uint32_t sm[32];
    __shared__ uint32_t carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int s0 = 0; s0 < n_blocks; s0 += 1024)
    {
        const int i      = s0 + threadIdx.x;
        const uint32_t v = i < n_blocks ? block_sum[i] : 0u;
        uint32_t inc     = v;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1)
        {
            const uint32_t t = __shfl_up_sync(kFull, inc, k);
            if (lane >= k) inc += t;
        }
        if (lane == 31) sm[warp] = inc;
        __syncthreads();
        const uint32_t wsum = sm[lane];
        uint32_t winc       = wsum;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1)
        {
            const uint32_t t = __shfl_up_sync(kFull, winc, k);
            if (lane >= k) winc += t;
        }
        const uint32_t tot   = __shfl_sync(kFull, winc, 31);
        const uint32_t woff  = __shfl_sync(kFull, winc - wsum, warp);
        const uint32_t carry = carry_s;
        if (i < n_blocks) block_sum[i] = carry + woff + inc - v;
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + tot;
        __syncthreads();
    }
    if (threadIdx.x == 0)
    {
        *n_keep = carry_s;
        if (carry_s != expected) atomicOr(&stats->status, TRIPS_DEV_BAD_POINT_INDEX);  // duplicate indices in the removal list
    }
}

// kept[j] = old index of the j-th kept point
__global__ __launch_bounds__(256) void keep_list_kernel(const uint8_t* __restrict__ keep, int64_t n, const uint32_t* __restrict__ block_base,
                                                        uint32_t* __restrict__ kept)
{
    __shared__ uint32_t s_warp[8];
    const int64_t base = (int64_t)blockIdx.x * kResizeItems;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t run = block_base[blockIdx.x];
    for (int k0 = 0; k0 < kResizeItems; k0 += 256)
    {
        const int64_t i  = base + k0 + threadIdx.x;
        const uint32_t f = (i < n) ? keep[i] : 0u;
        const uint32_t ballot = __ballot_sync(kFull, f != 0);
        if (lane == 0) s_warp[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w)
        {
            const uint32_t c = s_warp[w];
            if (w < warp) before += c;
            total += c;
        }
        if (f) kept[run + before + __popc(ballot & ((1u << lane) - 1u))] = (uint32_t)i;
        run += total;
        __syncthreads();
    }
}

struct ResizeArgs
{
    TripsPointTensor t[TRIPS_MAX_POINT_TENSORS];
    int n;
};

template <typename T>
__device__ __forceinline__ void resize_one(const TripsPointTensor& t, int64_t j, bool live, int64_t src_i, int64_t n_old, int64_t n_new)
{
    const T* src = static_cast<const T*>(t.src);
    T* dst       = static_cast<T*>(t.dst);
    T fill;
    if (sizeof(T) == 4)
        fill = *reinterpret_cast<const T*>(&t.fill_bits);
    else
    {
        const unsigned long long wide = t.fill_bits;  // 8-byte elements are filled with the zero-extended bits (0 for counters)
        fill = *reinterpret_cast<const T*>(&wide);
    }
    for (int r = 0; r < t.rows; ++r)
    {
        const T v = live ? (t.point_major ? src[src_i * t.rows + r] : src[(int64_t)r * n_old + src_i]) : fill;
        if (t.point_major)
            dst[j * t.rows + r] = v;
        else
            dst[(int64_t)r * n_new + j] = v;
    }
}

__global__ __launch_bounds__(256) void resize_gather_kernel(const __grid_constant__ ResizeArgs a, const uint32_t* __restrict__ kept,
                                                            const uint32_t* __restrict__ n_keep_p, int64_t n_old, int64_t n_new)
{
    const int64_t n_keep = *n_keep_p;
    const TripsPointTensor& t = a.t[blockIdx.y];
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_new; j += (int64_t)gridDim.x * blockDim.x)
    {
        const bool live     = j < n_keep;
        const int64_t src_i = live ? (int64_t)kept[j] : 0;
        if (t.elem_bytes == 4 && t.point_major && t.rows == 4 && (((uintptr_t)t.src | (uintptr_t)t.dst) & 15) == 0)
        {
            // [N,4] float tensors (positions and their Adam state): one 16-byte load and store per point
            const uint32_t f = t.fill_bits;
            static_cast<uint4*>(t.dst)[j] = live ? static_cast<const uint4*>(t.src)[src_i] : make_uint4(f, f, f, f);
        }
        else if (t.elem_bytes == 4)
            resize_one<uint32_t>(t, j, live, src_i, n_old, n_new);
        else
            resize_one<unsigned long long>(t, j, live, src_i, n_old, n_new);
    }
}

// scratch: keep flags [n_points] bytes | block sums [n_blocks + 1] u32 | kept list [n_points] u32
size_t resize_scratch_bytes(int64_t n_points)
{
    const int64_t nb = (n_points + kResizeItems - 1) / kResizeItems;
    return (size_t)((n_points + 15) / 16 * 16) + sizeof(uint32_t) * (size_t)(nb + 4) + sizeof(uint32_t) * (size_t)(n_points + 4);
}

cudaError_t launch_resize_points(const int64_t* remove, int64_t n_remove, int64_t n_points, int64_t n_new, const TripsPointTensor* tensors,
                                 int n_tensors, void* scratch, DevStats* stats, int sm_count, cudaStream_t st)
{
    const int64_t nb   = (n_points + kResizeItems - 1) / kResizeItems;
    uint8_t* keep      = static_cast<uint8_t*>(scratch);
    uint32_t* block    = reinterpret_cast<uint32_t*>(keep + (n_points + 15) / 16 * 16);
    uint32_t* n_keep   = block + nb;
    uint32_t* kept     = block + nb + 4;
    cudaError_t e;
    if ((e = cudaMemsetAsync(keep, 1, (size_t)n_points, st)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(n_keep, 0, sizeof(uint32_t), st)) != cudaSuccess) return e;
    if (n_remove > 0)
        mark_removed_kernel<<<(int)min((int64_t)sm_count * 8, (n_remove + 255) / 256), 256, 0, st>>>(remove, n_remove, n_points, keep, stats);
    if (n_points > 0)
    {
        keep_count_kernel<<<(unsigned)nb, 256, 0, st>>>(keep, n_points, block);
        keep_scan_kernel<<<1, 1024, 0, st>>>(block, (int)nb, n_keep, (uint32_t)(n_points - n_remove), stats);
        keep_list_kernel<<<(unsigned)nb, 256, 0, st>>>(keep, n_points, block, kept);
    }
    if (n_new > 0 && n_tensors > 0)
    {
        ResizeArgs a{};
        a.n = n_tensors;
        for (int i = 0; i < n_tensors; ++i) a.t[i] = tensors[i];
        dim3 grid((unsigned)min((int64_t)sm_count * 8, (n_new + 255) / 256), (unsigned)n_tensors);
        resize_gather_kernel<<<grid, 256, 0, st>>>(a, kept, n_keep, n_points, n_new);
    }
    return cudaGetLastError();
}
}  // namespace trips
