// Prioritised-replay weights from the per-segment |advantage| sums (sm_100a).
//
// Replaces the eager torch sequence of the reference trainer
// (pufferlib/pufferl.py:359-361):
//     adv = advantages.abs().sum(axis=1)          <- fused into the advantage kernel
//     w   = nan_to_num(adv ** prio_alpha, 0, 0, 0)
//     p   = (w + 1e-6) / (w.sum() + 1e-6)
// Two entry points so that a caller whose segments are sharded over several
// GPUs can all-reduce the scalar sum between them.  The sum is accumulated in
// fp64 by a fixed two-level tree (per-CTA partials in caller-owned scratch,
// then one CTA), so it does not depend on scheduling.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/puff_advantage.h"

namespace puff {
void count_launch();

constexpr int kPrioThreads = 256;
constexpr int kPrioMaxBlocks = 1024;

__device__ __forceinline__ double block_sum(double x, double* s_part)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) s_part[warp] = x;
    __syncthreads();
    double tot = 0.0;
    if (threadIdx.x == 0)
        for (int i = 0; i < (blockDim.x >> 5); ++i) tot += s_part[i];
    return tot;   // valid in thread 0
}

// weights[s] = finite(pow(abs_sum[s], alpha)) else 0; partial[b] = sum over the CTA's slab
__global__ void __launch_bounds__(kPrioThreads)
puff_prio_weights_kernel(const float* __restrict__ seg_abs_sum, float* __restrict__ weights,
                         double* __restrict__ partial, float alpha, long long num_segments)
{
    __shared__ double s_part[kPrioThreads / 32];
    // contiguous slab per CTA, so the partial does not depend on the grid-stride order
    const long long per = (num_segments + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x;
    const long long hi = lo + per < num_segments ? lo + per : num_segments;
    double acc = 0.0;
    for (long long s = lo + threadIdx.x; s < hi; s += blockDim.x) {
        float w = powf(seg_abs_sum[s], alpha);
        if (!isfinite(w)) w = 0.0f;
        weights[s] = w;
        acc += static_cast<double>(w);
    }
    const double tot = block_sum(acc, s_part);
    if (threadIdx.x == 0) partial[blockIdx.x] = tot;
}

__global__ void __launch_bounds__(kPrioThreads)
puff_prio_total_kernel(const double* __restrict__ partial, int n, double* __restrict__ total_w)
{
    __shared__ double s_part[kPrioThreads / 32];
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
    const double tot = block_sum(acc, s_part);
    if (threadIdx.x == 0) *total_w = tot;
}

__global__ void __launch_bounds__(kPrioThreads)
puff_prio_probs_kernel(const float* __restrict__ weights, const double* __restrict__ total_w,
                       float* __restrict__ probs, long long num_segments)
{
    // pufferl.py:361 evaluates in fp32: (w + 1e-6) / (sum + 1e-6)
    const float denom = static_cast<float>(*total_w) + 1e-6f;
    for (long long s = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; s < num_segments;
         s += static_cast<long long>(gridDim.x) * blockDim.x)
        probs[s] = (weights[s] + 1e-6f) / denom;
}

static int prio_blocks(long long num_segments)
{
    long long b = (num_segments + kPrioThreads * 4 - 1) / (kPrioThreads * 4);
    if (b < 1) b = 1;
    if (b > kPrioMaxBlocks) b = kPrioMaxBlocks;
    return static_cast<int>(b);
}
}  // namespace puff

using namespace puff;

extern "C" size_t puff_priorities_sm100_scratch_bytes(long long num_segments)
{
    if (num_segments <= 0) return 8;
    return static_cast<size_t>(prio_blocks(num_segments)) * sizeof(double);
}

extern "C" int puff_priorities_sm100_weights(const float* seg_abs_sum, float* weights, double* total_w,
                                             float alpha, long long num_segments, void* scratch,
                                             size_t scratch_bytes, void* cuda_stream)
{
    if (num_segments < 0) return PUFF_ERR_SHAPE;
    if (total_w == nullptr) return PUFF_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (num_segments == 0) {
        cudaError_t e = cudaMemsetAsync(total_w, 0, sizeof(double), st);
        return static_cast<int>(e);
    }
    if (seg_abs_sum == nullptr || weights == nullptr) return PUFF_ERR_NULL;
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 7u) ||
        scratch_bytes < puff_priorities_sm100_scratch_bytes(num_segments))
        return PUFF_ERR_WORKSPACE;
    const int blocks = prio_blocks(num_segments);
    double* partial = static_cast<double*>(scratch);
    puff_prio_weights_kernel<<<blocks, kPrioThreads, 0, st>>>(seg_abs_sum, weights, partial, alpha, num_segments);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    puff_prio_total_kernel<<<1, kPrioThreads, 0, st>>>(partial, blocks, total_w);
    count_launch();
    return static_cast<int>(cudaGetLastError());
}

extern "C" int puff_priorities_sm100_probs(const float* weights, const double* total_w, float* probs,
                                           long long num_segments, void* cuda_stream)
{
    if (num_segments < 0) return PUFF_ERR_SHAPE;
    if (num_segments == 0) return PUFF_OK;
    if (weights == nullptr || total_w == nullptr || probs == nullptr) return PUFF_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    long long blocks = (num_segments + kPrioThreads - 1) / kPrioThreads;
    if (blocks > 148 * 8) blocks = 148 * 8;
    puff_prio_probs_kernel<<<static_cast<int>(blocks), kPrioThreads, 0, st>>>(weights, total_w, probs, num_segments);
    count_launch();
    return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// priority weights without any allocation
// ---------------------------------------------------------------------------
// puff_priorities_sm100_weights needs a few KB of scratch for its per-CTA
// partial sums and expects the caller to own it.  A caller that sits behind a
// plain C FFI inside a trainer whose device memory is already carved up -- the
// policy, the experience buffers and the framework's caching allocator hold
// all of it, or the host wrapper simply has no allocator handle to pass down --
// cannot produce that buffer: cudaMalloc there may fail outright, and where it
// succeeds it stalls the device in the middle of the minibatch loop.  For such
// callers the scratch lives in the library image instead: one fixed array per
// GPU that loads this library, held until the process exits.
//
// The array is sized for kNoAllocMaxBlocks partial sums (4 KB), which covers
// PUFF_NOALLOC_MAX_SEGMENTS segments; larger requests are refused, not
// truncated.  `g_noalloc_partials` below is the device symbol; in host code
// that name is only a stand-in, so the real device address is looked up with
// cudaGetSymbolAddress once per device (with that device current) and that
// pointer is what the kernels receive.
constexpr int kNoAllocMaxBlocks = 512;
static_assert(static_cast<long long>(kNoAllocMaxBlocks) * kPrioThreads * 4 == PUFF_NOALLOC_MAX_SEGMENTS,
              "header limit and scratch size disagree");
static __device__ __align__(256) double g_noalloc_partials[kNoAllocMaxBlocks];

namespace puff {
constexpr int kNoAllocMaxDevices = 64;
static std::mutex g_noalloc_mutex;
static double* g_noalloc_ptr[kNoAllocMaxDevices] = {};

// Device address of the scratch array on the current device; looked up on the
// first call per device and cached.
static int noalloc_scratch(double** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kNoAllocMaxDevices) return PUFF_ERR_ARCH;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_partials);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (p == nullptr) return PUFF_ERR_WORKSPACE;
        g_noalloc_ptr[dev] = static_cast<double*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return PUFF_OK;
}
}  // namespace puff

extern "C" int puff_priorities_sm100_weights_noalloc(const float* seg_abs_sum, float* weights, double* total_w,
                                                     float alpha, long long num_segments, void* cuda_stream)
{
    if (num_segments < 0) return PUFF_ERR_SHAPE;
    if (num_segments > PUFF_NOALLOC_MAX_SEGMENTS) return PUFF_ERR_SIZE;
    if (total_w == nullptr) return PUFF_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (num_segments == 0) return static_cast<int>(cudaMemsetAsync(total_w, 0, sizeof(double), st));
    if (seg_abs_sum == nullptr || weights == nullptr) return PUFF_ERR_NULL;
    double* partial = nullptr;
    const int rc = noalloc_scratch(&partial);
    if (rc != PUFF_OK) return rc;
    // Nothing in the scratch has to start at zero: the first kernel overwrites
    // partial[0 .. blocks) and the second reads exactly those entries, so
    // whatever an earlier (possibly larger) call left behind is never read.
    const int blocks = prio_blocks(num_segments);
    puff_prio_weights_kernel<<<blocks, kPrioThreads, 0, st>>>(seg_abs_sum, weights, partial, alpha, num_segments);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    puff_prio_total_kernel<<<1, kPrioThreads, 0, st>>>(partial, blocks, total_w);
    count_launch();
    return static_cast<int>(cudaGetLastError());
}
