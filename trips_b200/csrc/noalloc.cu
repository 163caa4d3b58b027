// trips_adam_step_static: the fused Adam step for callers that must not allocate device memory.
//
// trips_adam_step keeps the table that tells the kernel where every parameter tensor lives (pointers, sizes,
// hyper-parameters, and the first thread block of each tensor) in context scratch that it cudaMallocs on first use
// and regrows when more tensors arrive.  Some callers cannot tolerate that: an optimizer step issued while the
// framework above holds every free byte in its own caching pool, or a plugin whose host rules forbid cudaMalloc
// after start-up.  This variant places the same table in a fixed device array that is part of the loaded library
// image, so that a call does no cudaMalloc, no cudaFree and no allocating library call; it needs no TripsContext
// either.  The table is uploaded from this function's stack frame with every call, so the call belongs on a stream
// that executes it now: a stream that is being captured is refused (TRIPS_ERR_UNSUPPORTED) before anything is
// enqueued, because a recorded copy would read the dead stack frame when the graph is replayed.
#include <mutex>

#include "common.cuh"

namespace
{
constexpr int kStaticAdamMaxTensors = TRIPS_ADAM_STATIC_MAX_TENSORS;
constexpr int kMaxDevices           = 64;

struct StaticAdamTable
{
    TripsAdamTensor tensors[kStaticAdamMaxTensors];
    int64_t block_start[kStaticAdamMaxTensors + 1];
};

// The scratch itself: one copy per GPU that loads the library, held until the process exits (about 6 KB).
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_adam_table[sizeof(StaticAdamTable)];

std::mutex g_mutex;
void* g_table_ptr[kMaxDevices] = {};  // device address of g_static_adam_table, per device, resolved on first use
}  // namespace

extern "C" int trips_adam_step_static(const TripsAdamTensor* tensors, int n_tensors, void* stream)
{
    if (!tensors || n_tensors < 1) return TRIPS_ERR_INVALID_ARG;
    if (n_tensors > kStaticAdamMaxTensors) return TRIPS_ERR_TOO_LARGE;  // the fixed table holds at most 64 tensors
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    {
        (void)cudaGetLastError();
        return TRIPS_ERR_CUDA;
    }
    cudaStream_t st = (cudaStream_t)stream;
    {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) != cudaSuccess)
        {
            (void)cudaGetLastError();
            return TRIPS_ERR_CUDA;
        }
        if (cap != cudaStreamCaptureStatusNone) return TRIPS_ERR_UNSUPPORTED;  // host-only check, nothing was enqueued
    }
    // Set-up, once per device and with that device current: ask the runtime where this device's copy of the
    // array lives.  The first call on a device should therefore come before any stream capture.
    void* table = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_table_ptr[device])
        {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_adam_table) != cudaSuccess || !p)
            {
                (void)cudaGetLastError();
                return TRIPS_ERR_CUDA;
            }
            g_table_ptr[device] = p;
        }
        table = g_table_ptr[device];
    }
    StaticAdamTable host;  // on the stack: no host heap either
    host.block_start[0] = 0;
    for (int i = 0; i < n_tensors; ++i)
    {
        const TripsAdamTensor& t = tensors[i];
        if (t.n < 0 || (t.n > 0 && (!t.weights || !t.gradients || !t.first_moments || !t.second_moments || !t.steps)))
            return TRIPS_ERR_INVALID_ARG;
        host.tensors[i]         = t;
        host.block_start[i + 1] = host.block_start[i] + (t.n + trips::kAdamPerBlock - 1) / trips::kAdamPerBlock;
    }
    const int64_t total_blocks = host.block_start[n_tensors];
    if (total_blocks >= (1ll << 31)) return TRIPS_ERR_TOO_LARGE;
    // The whole table is rewritten by every call, so nothing of the previous call's contents is ever read.  The
    // source is pageable stack memory: the runtime stages it before cudaMemcpyAsync returns.
    unsigned char* dev = static_cast<unsigned char*>(table);
    if (cudaMemcpyAsync(dev + offsetof(StaticAdamTable, tensors), host.tensors, sizeof(TripsAdamTensor) * n_tensors,
                        cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaMemcpyAsync(dev + offsetof(StaticAdamTable, block_start), host.block_start, sizeof(int64_t) * (n_tensors + 1),
                        cudaMemcpyHostToDevice, st) != cudaSuccess)
    {
        (void)cudaGetLastError();
        return TRIPS_ERR_CUDA;
    }
    const cudaError_t e = trips::launch_adam(reinterpret_cast<const TripsAdamTensor*>(dev + offsetof(StaticAdamTable, tensors)),
                                             reinterpret_cast<const int64_t*>(dev + offsetof(StaticAdamTable, block_start)),
                                             n_tensors, total_blocks, st);
    if (e != cudaSuccess)
    {
        (void)cudaGetLastError();
        return TRIPS_ERR_CUDA;
    }
    return TRIPS_OK;
}
