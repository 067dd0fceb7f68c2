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
#include <new>

#include "../../include/puff_advantage.h"
#include "puff_launch.cuh"

namespace puff {
void count_launch();
int* device_status_ptr();   // puff_advantage_sm100.cu: device address of the status word, current device

constexpr int kPrioThreads = 256;
constexpr int kPrioMaxBlocks = 1024;
// The priority kernels usually run on a side stream under a persistent advantage kernel whose
// two CTAs per SM leave 8192 registers and a few KB of shared memory free.  Asking for eight
// resident CTAs per SM caps them at 32 registers per thread, so one 256-thread CTA always fits
// beside the advantage grid instead of waiting for it to retire.
#define PUFF_PRIO_BOUNDS __launch_bounds__(kPrioThreads, 8)

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
__global__ void PUFF_PRIO_BOUNDS
puff_prio_weights_kernel(const float* __restrict__ seg_abs_sum, float* __restrict__ weights,
                         double* __restrict__ partial, float alpha, long long num_segments)
{
    __shared__ double s_part[kPrioThreads / 32];
    pdl_wait();
    pdl_launch_dependents();
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

__global__ void PUFF_PRIO_BOUNDS
puff_prio_total_kernel(const double* __restrict__ partial, int n, double* __restrict__ total_w)
{
    __shared__ double s_part[kPrioThreads / 32];
    pdl_wait();
    pdl_launch_dependents();
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
    const double tot = block_sum(acc, s_part);
    if (threadIdx.x == 0) *total_w = tot;
}

__global__ void PUFF_PRIO_BOUNDS
puff_prio_probs_kernel(const float* __restrict__ weights, const double* __restrict__ total_w,
                       float* __restrict__ probs, long long num_segments)
{
    pdl_wait();
    pdl_launch_dependents();
    // pufferl.py:361 evaluates in fp32: (w + 1e-6) / (sum + 1e-6)
    const float denom = static_cast<float>(*total_w) + 1e-6f;
    for (long long s = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; s < num_segments;
         s += static_cast<long long>(gridDim.x) * blockDim.x)
        probs[s] = (weights[s] + 1e-6f) / denom;
}

// ---------------------------------------------------------------------------
// cross-GPU exchange of the weight total (segments sharded over several GPUs)
// ---------------------------------------------------------------------------
// Every rank owns a small mailbox in its own HBM: kExRing x world slots of (value, seq).
// After summing its local weights a rank stores the total into slot [seq % kExRing][rank] of
// EVERY rank's mailbox (its own included) with plain stores through peer-mapped pointers, a
// system-scope fence, then the sequence number as the flag.  The probabilities kernel polls its
// OWN mailbox -- local memory -- until all `world` slots carry the current sequence number, adds
// them in rank order (so every rank forms the identical fp64 sum) and normalises.  No remote
// loads, no multicast, no library collective; 16 bytes cross NVLink per peer and step.
//
// The wait is bounded: after `wait_ns` nanoseconds a CTA that still misses a slot records
// PUFF_ERR_DEVICE_WAIT in the device status word and returns without writing its probabilities.
//
// Ordering: consecutive exchanges reuse slot seq % kExRing.  A rank can run at most one exchange
// ahead of the slowest reader of its previous one (its next push is stream-ordered behind its own
// gather, which needs everybody's push of the current round), so a ring of four is ample as long
// as each rank issues its exchanges on one stream (or otherwise in order).
constexpr int kExRing = 4;
struct ExSlot {
    double value;
    unsigned long long seq;
};
struct ExControl {              // device memory of the owning rank, not shared
    unsigned long long seq;     // number of pushes so far
    unsigned int arrived;       // CTAs of the current weights + push launch that have stored their partial
};
constexpr int kExMaxWorld = 32;
constexpr unsigned kExMaxPolls = 1u << 24;
struct ExPeers {                // passed by value to the push kernel
    ExSlot* slots[kExMaxWorld];
};

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_f64(double* p, double v)
{
    asm volatile("st.relaxed.sys.global.f64 [%0], %1;" ::"l"(p), "d"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p)
{
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ex_global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// one CTA: local total from the per-CTA partials, then the push to every rank's mailbox
__global__ void PUFF_PRIO_BOUNDS
puff_prio_total_push_kernel(const double* __restrict__ partial, int n, ExControl* ctl, ExPeers peers,
                            int rank, int world)
{
    __shared__ double s_part[kPrioThreads / 32];
    __shared__ double s_total;
    pdl_wait();
    pdl_launch_dependents();
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
    const double tot = block_sum(acc, s_part);
    if (threadIdx.x == 0) s_total = tot;
    __syncthreads();
    const unsigned long long seq = ctl->seq + 1ull;
    if (static_cast<int>(threadIdx.x) < world) {
        ExSlot* dst = peers.slots[threadIdx.x] + (seq % kExRing) * world + rank;
        st_relaxed_sys_f64(&dst->value, s_total);
        __threadfence_system();                 // the value is visible before the flag
        st_relaxed_sys_u64(&dst->seq, seq);
    }
    __syncthreads();
    if (threadIdx.x == 0) ctl->seq = seq;
}

// Weights, local total and push in ONE launch: every CTA writes its slab's weights and partial
// sum and takes a ticket; the CTA that draws the last ticket (no CTA waits for another) adds the
// partials in index order -- so the total does not depend on which CTA came last -- and pushes.
__global__ void PUFF_PRIO_BOUNDS
puff_prio_weights_push_kernel(const float* __restrict__ seg_abs_sum, float* __restrict__ weights, double* partial,
                              float alpha, long long num_segments, ExControl* ctl, ExPeers peers, int rank, int world)
{
    __shared__ double s_part[kPrioThreads / 32];
    __shared__ double s_total;
    __shared__ bool s_last;
    pdl_wait();
    pdl_launch_dependents();
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
    const double mine = block_sum(acc, s_part);
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = mine;
        __threadfence();                                   // the partial is visible before the ticket
        s_last = atomicAdd(&ctl->arrived, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();                                       // the other CTAs' partials, behind their tickets
    double tot_acc = 0.0;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) tot_acc += __ldcg(partial + i);
    __syncthreads();                                       // s_part is reused
    const double tot = block_sum(tot_acc, s_part);
    if (threadIdx.x == 0) s_total = tot;
    __syncthreads();
    const unsigned long long seq = ctl->seq + 1ull;
    if (static_cast<int>(threadIdx.x) < world) {
        ExSlot* dst = peers.slots[threadIdx.x] + (seq % kExRing) * world + rank;
        st_relaxed_sys_f64(&dst->value, s_total);
        __threadfence_system();                 // the value is visible before the flag
        st_relaxed_sys_u64(&dst->seq, seq);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        ctl->seq = seq;
        ctl->arrived = 0u;                      // for the next launch, which is stream-ordered behind this one
    }
}

// probabilities from the gathered totals; every CTA waits on this rank's own mailbox
__global__ void PUFF_PRIO_BOUNDS
puff_prio_probs_gathered_kernel(const float* __restrict__ weights, const ExSlot* mailbox, const ExControl* ctl,
                                double* __restrict__ total_w, float* __restrict__ probs, long long num_segments,
                                int world, unsigned long long wait_ns, int* status)
{
    __shared__ double s_total;
    __shared__ int s_ok;
    pdl_wait();   // the push of this exchange, the previous kernel of the stream, has completed
    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const unsigned long long seq = ctl->seq;    // the push of this exchange precedes this kernel in its stream
        const int lane = threadIdx.x;
        const ExSlot* slot = mailbox + (seq % kExRing) * world + (lane < world ? lane : 0);
        bool here = lane >= world || ld_acquire_sys_u64(&slot->seq) == seq;
        bool ok = __all_sync(0xffffffffu, here);
        if (!ok) {
            // bounded: lane 0's clock (and a poll count) decides for the whole warp
            const unsigned long long t0 = ex_global_ns();
            for (unsigned polls = 0; polls < kExMaxPolls; ++polls) {
                if (!here) here = ld_acquire_sys_u64(&slot->seq) == seq;
                ok = __all_sync(0xffffffffu, here);
                const int expired = __shfl_sync(0xffffffffu, static_cast<int>(ex_global_ns() - t0 > wait_ns), 0);
                if (ok || expired) break;
                __nanosleep(200);
            }
        }
        const double mine = (ok && lane < world) ? slot->value : 0.0;
        double tot = 0.0;
        for (int r = 0; r < world; ++r) tot += __shfl_sync(0xffffffffu, mine, r);   // rank order on every GPU
        if (lane == 0) {
            s_total = tot;
            s_ok = ok ? 1 : 0;
            if (!ok) atomicExch(status, PUFF_ERR_DEVICE_WAIT);
            if (ok && blockIdx.x == 0 && total_w != nullptr) *total_w = tot;
        }
    }
    __syncthreads();
    if (!s_ok) return;
    const float denom = static_cast<float>(s_total) + 1e-6f;
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
    // The first kernel of the call is launched plainly: what precedes it is not this library's to
    // know, and behind an advantage kernel of ANOTHER stream a programmatic launch was measured to
    // cost the pipelined step 3 us (131072 x 256: 106.5 against 103.6 us; bare kernel 103.5).
    puff_prio_weights_kernel<<<blocks, kPrioThreads, 0, st>>>(seg_abs_sum, weights, partial, alpha, num_segments);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    e = launch_neighbour(puff_prio_total_kernel, 1, kPrioThreads, 0, st, partial, blocks, total_w);
    count_launch();
    return static_cast<int>(e);
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
    const cudaError_t e = launch_neighbour(puff_prio_probs_kernel, static_cast<int>(blocks), kPrioThreads, 0, st, weights,
                                        total_w, probs, num_segments);
    count_launch();
    return static_cast<int>(e);
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


// ---------------------------------------------------------------------------
// host side of the exchange
// ---------------------------------------------------------------------------
struct puff_exchange {
    int rank = 0, world = 1, device = 0;
    bool connected = false;
    puff::ExSlot* mailbox = nullptr;          // this rank's, cudaMalloc'd (shareable by CUDA IPC)
    puff::ExControl* control = nullptr;
    puff::ExSlot* peer[puff::kExMaxWorld] = {};   // every rank's mailbox as seen from this device
    bool opened[puff::kExMaxWorld] = {};           // mapped with cudaIpcOpenMemHandle
    unsigned long long wait_ns = 2000000000ull;
    int* status = nullptr;
};

static_assert(sizeof(cudaIpcMemHandle_t) == PUFF_EXCHANGE_HANDLE_BYTES, "handle size");

extern "C" int puff_exchange_sm100_create(int rank, int world, void* handle_out, puff_exchange** out)
{
    if (out == nullptr) return PUFF_ERR_NULL;
    *out = nullptr;
    if (world < 1 || world > kExMaxWorld || rank < 0 || rank >= world) return PUFF_ERR_SHAPE;
    puff_exchange* x = new (std::nothrow) puff_exchange();
    if (x == nullptr) return PUFF_ERR_WORKSPACE;
    x->rank = rank;
    x->world = world;
    cudaError_t e = cudaGetDevice(&x->device);
    const size_t bytes = sizeof(ExSlot) * kExRing * world;
    if (e == cudaSuccess) e = cudaMalloc(&x->mailbox, bytes);
    if (e == cudaSuccess) e = cudaMemset(x->mailbox, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&x->control, sizeof(ExControl));
    if (e == cudaSuccess) e = cudaMemset(x->control, 0, sizeof(ExControl));
    if (e == cudaSuccess && handle_out != nullptr)
        e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out), x->mailbox);
    if (e == cudaSuccess) {
        x->status = device_status_ptr();
        if (x->status == nullptr) e = cudaErrorInvalidSymbol;
    }
    if (e != cudaSuccess) {
        if (x->mailbox != nullptr) cudaFree(x->mailbox);
        if (x->control != nullptr) cudaFree(x->control);
        delete x;
        return static_cast<int>(e);
    }
    x->peer[rank] = x->mailbox;
    if (world == 1) x->connected = true;
    *out = x;
    return PUFF_OK;
}

extern "C" int puff_exchange_sm100_connect(puff_exchange* x, const void* all_handles)
{
    if (x == nullptr || all_handles == nullptr) return PUFF_ERR_NULL;
    const cudaIpcMemHandle_t* h = static_cast<const cudaIpcMemHandle_t*>(all_handles);
    for (int r = 0; r < x->world; ++r) {
        if (r == x->rank || x->peer[r] != nullptr) continue;
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return static_cast<int>(e);
        x->peer[r] = static_cast<ExSlot*>(p);
        x->opened[r] = true;
    }
    x->connected = true;
    return PUFF_OK;
}

extern "C" int puff_exchange_sm100_connect_pointers(puff_exchange* x, void* const* mailboxes)
{
    if (x == nullptr || mailboxes == nullptr) return PUFF_ERR_NULL;
    for (int r = 0; r < x->world; ++r) {
        if (r == x->rank) continue;
        if (mailboxes[r] == nullptr) return PUFF_ERR_NULL;
        x->peer[r] = static_cast<ExSlot*>(mailboxes[r]);
    }
    x->connected = true;
    return PUFF_OK;
}

extern "C" void* puff_exchange_sm100_mailbox(puff_exchange* x) { return x == nullptr ? nullptr : x->mailbox; }

extern "C" int puff_exchange_sm100_set_wait_ns(puff_exchange* x, unsigned long long wait_ns)
{
    if (x == nullptr) return PUFF_ERR_NULL;
    x->wait_ns = wait_ns;
    return PUFF_OK;
}

extern "C" int puff_exchange_sm100_destroy(puff_exchange* x)
{
    if (x == nullptr) return PUFF_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(x->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < x->world; ++r)
        if (x->opened[r]) cudaIpcCloseMemHandle(x->peer[r]);
    cudaFree(x->mailbox);
    cudaFree(x->control);
    cudaSetDevice(prev);
    delete x;
    return PUFF_OK;
}

extern "C" int puff_priorities_sm100_weights_push(const float* seg_abs_sum, float* weights, float alpha,
                                                  long long num_segments, void* scratch, size_t scratch_bytes,
                                                  puff_exchange* x, void* cuda_stream)
{
    if (num_segments < 0) return PUFF_ERR_SHAPE;
    if (x == nullptr) return PUFF_ERR_NULL;
    if (!x->connected) return PUFF_ERR_WORKSPACE;
    if (num_segments > 0 && (seg_abs_sum == nullptr || weights == nullptr)) return PUFF_ERR_NULL;
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 7u) ||
        scratch_bytes < puff_priorities_sm100_scratch_bytes(num_segments))
        return PUFF_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    double* partial = static_cast<double*>(scratch);
    ExPeers peers;
    for (int r = 0; r < kExMaxWorld; ++r) peers.slots[r] = r < x->world ? x->peer[r] : nullptr;
    // A plain launch, not a programmatic dependent one: this kernel usually follows an advantage
    // kernel of another stream, and CTAs that become resident early sit on registers and thread
    // slots which the next persistent advantage grid needs (two CTAs on every SM).  Measured at
    // two GPUs, 131072 x 256 per GPU: step 104.1 us with a plain launch here, 114.7 with a
    // programmatic one (bare kernel 103.1-104.3).  The gather behind it is launched
    // programmatically, with at most 128 CTAs: fewer than one per SM, so it never takes the slot
    // of an advantage CTA.
    if (num_segments > 0)
        puff_prio_weights_push_kernel<<<prio_blocks(num_segments), kPrioThreads, 0, st>>>(
            seg_abs_sum, weights, partial, alpha, num_segments, x->control, peers, x->rank, x->world);
    else   // a rank without rows still takes part with a total of zero
        puff_prio_total_push_kernel<<<1, kPrioThreads, 0, st>>>(partial, 0, x->control, peers, x->rank, x->world);
    count_launch();
    return static_cast<int>(cudaGetLastError());
}

extern "C" int puff_priorities_sm100_probs_gathered(const float* weights, double* total_w, float* probs,
                                                    long long num_segments, puff_exchange* x, void* cuda_stream)
{
    if (num_segments < 0) return PUFF_ERR_SHAPE;
    if (x == nullptr) return PUFF_ERR_NULL;
    if (!x->connected) return PUFF_ERR_WORKSPACE;
    if (num_segments > 0 && (weights == nullptr || probs == nullptr)) return PUFF_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    long long blocks = (num_segments + kPrioThreads - 1) / kPrioThreads;
    if (blocks > 128) blocks = 128;   // fewer than one CTA per SM: see the note in puff_priorities_sm100_weights_push
    if (blocks < 1) blocks = 1;       // the total is still gathered (and written) for a rank without rows
    const cudaError_t e = launch_neighbour(puff_prio_probs_gathered_kernel, static_cast<int>(blocks), kPrioThreads, 0, st,
                                        weights, x->mailbox, x->control, total_w, probs, num_segments, x->world,
                                        x->wait_ns, x->status);
    count_launch();
    return static_cast<int>(e);
}
