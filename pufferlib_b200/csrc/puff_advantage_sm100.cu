// V-trace-clipped GAE advantage op for sm_100a: kernel selection, launch and the C ABI.
//
// Torch-free on purpose: a standalone nvcc harness can #include this file, and
// the torch operator binding only sees the extern "C" entry points declared in
// include/puff_advantage.h.
//
// Replaces pufferlib/extensions/cuda/pufferlib.cu:7-82 of the reference (one
// thread per segment walking global memory at a stride of `horizon` floats).
// The op is a memory-bound linear recurrence: 20 algorithmic bytes and about
// ten flops per element, so the design goal is HBM bandwidth, not flops.
//
// Kernels (puff_kernels_*.cuh; shared device code in puff_device.cuh)
//   tma2d   serial, bit-exact, H % 4 == 0 and 16-byte aligned bases.  Tiles of 32
//           segments, the horizon walked backwards in chunks of 32 columns; each
//           chunk of the four inputs arrives as a 32x32 TMA box in 128B-swizzled
//           shared memory behind an mbarrier ring, and the advantages leave through
//           a TMA store.  Two forms: a warp-specialised CTA of a producer warp,
//           four warps that compute what does not depend on the running advantage,
//           and one warp that runs the recurrence (the default), and one warp per
//           CTA doing everything (on request).  TMA clips a store at
//           the tensor edge in whole 16-byte units only, so column H-1 cannot be
//           masked out of the box: each lane reads its row's advantages[H-1] once
//           per tile and the store writes that same value back.
//   bulk1d  serial, bit-exact, for H % 4 != 0 (row pitch not a multiple of
//           16 bytes, so no 2-D tensor map exists): tiles of 4..32 whole rows
//           are contiguous spans, fetched with 1-D bulk copies and written back
//           with one 1-D bulk store per tile.  One-stage and warp-specialised forms.
//   scan    T threads per row, 4 steps per thread: local affine composition,
//           warp-shuffle + shared-memory scan of the (k, d) pairs, serial
//           replay of the 4 steps from the scanned carry-in.  For long rows
//           with few segments, where one thread per row cannot fill the GPU.
//   generic serial, bit-exact, plain global loads.  Any alignment, any H.
//
// Every wait on an mbarrier is bounded: when the limit is hit the warp records
// PUFF_ERR_DEVICE_WAIT in a status word, drains its own stores and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "../../include/puff_advantage.h"
#include "puff_device.cuh"
#include "puff_kernels_bulk1d.cuh"
#include "puff_kernels_scan.cuh"
#include "puff_kernels_tma2d.cuh"

namespace puff {

// ---------------------------------------------------------------------------
// launch counter and per-thread record of the kernel last used
// ---------------------------------------------------------------------------
static std::atomic<long long> g_launch_count{0};
static thread_local int t_last_kernel = PUFF_KERNEL_NONE;

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    int max_smem_optin = 0;
    cudaError_t err = cudaSuccess;
    std::atomic<bool> ready{false};   // set last, with release order, under g_dev_mutex
};
static DeviceInfo g_dev[64];
static std::mutex g_dev_mutex;

template <int NST>
static void set_tma2d_attrs()
{
    cudaFuncSetAttribute(puff_adv_tma2d_kernel<NST, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma2d_smem_bytes<NST>());
    cudaFuncSetAttribute(puff_adv_tma2d_kernel<NST, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma2d_smem_bytes<NST>());
}

template <int NST, int NT>
static void set_tma2d_ws_attrs()
{
    cudaFuncSetAttribute(puff_adv_tma2d_ws_kernel<NST, NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma2d_ws_smem_bytes<NST, NT>());
    cudaFuncSetAttribute(puff_adv_tma2d_ws_kernel<NST, NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tma2d_ws_smem_bytes<NST, NT>());
}

static const DeviceInfo* device_info(int* code)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *code = static_cast<int>(e);
        return nullptr;
    }
    if (dev < 0 || dev >= 64) {
        *code = PUFF_ERR_ARCH;
        return nullptr;
    }
    DeviceInfo& d = g_dev[dev];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!d.ready.load(std::memory_order_relaxed)) {
            cudaError_t e1 = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
            cudaError_t e2 = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
            cudaError_t e3 = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
            d.err = e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3);
            if (d.err == cudaSuccess && d.cc_major == 10) {
                // opt in to large dynamic shared memory once per device
                set_tma2d_attrs<2>();
                set_tma2d_attrs<3>();
                set_tma2d_attrs<4>();
                set_tma2d_ws_attrs<2, 2>();
                set_tma2d_ws_attrs<3, 2>();
                set_tma2d_ws_attrs<4, 2>();
                set_tma2d_ws_attrs<6, 2>();
                cudaFuncSetAttribute(puff_adv_bulk1d_kernel<kB1Threads>, cudaFuncAttributeMaxDynamicSharedMemorySize, d.max_smem_optin);
                cudaFuncSetAttribute(puff_adv_bulk1d_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, d.max_smem_optin);
                cudaFuncSetAttribute(puff_adv_bulk1d_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, d.max_smem_optin);
                d.err = cudaGetLastError();
            }
            // a failed query is retried on the next call; the error is reported from a local
            // copy so that no other thread reads d.err while it may still change
            const cudaError_t err = d.err;
            if (err != cudaSuccess) {
                *code = static_cast<int>(err);
                return nullptr;
            }
            d.ready.store(true, std::memory_order_release);
        }
    }
    if (d.cc_major != 10) {
        *code = PUFF_ERR_ARCH;
        return nullptr;
    }
    return &d;
}

// cuTensorMapEncodeTiled through the runtime, so the library has no link-time
// dependency on libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// [rows, width] fp32 view with a row pitch of `pitch_elems` floats, 32x32 boxes, 128B swizzle
static bool make_map(CUtensorMap* tm, const float* base, long long rows, long long width, long long pitch_elems)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * 4u};
    const cuuint32_t box[2] = {kChunkCols, kTileRows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapSet {
    const float* ptr[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    CUtensorMap tm[5];
};

// Per-thread cache of encoded tensor maps, one entry per (base, rows, horizon).  A map
// holds nothing but the address and the shape, so an entry stays valid however often the
// memory behind it is freed and reallocated.  The trainer passes the same four input
// buffers on every call and a fresh advantages tensor that the caching allocator usually
// places at the same address: all five lookups hit.
struct MapEntry {
    const float* ptr = nullptr;
    long long rows = -1, horizon = -1;
    unsigned long long stamp = 0;
    CUtensorMap tm;
};
constexpr int kMapCacheEntries = 16;
struct MapCache {
    MapEntry e[kMapCacheEntries];
    unsigned long long clock = 0;
};

static const CUtensorMap* cached_map(MapCache& c, const float* base, long long rows, long long horizon)
{
    int victim = 0;
    for (int i = 0; i < kMapCacheEntries; ++i) {
        MapEntry& m = c.e[i];
        if (m.ptr == base && m.rows == rows && m.horizon == horizon) {
            m.stamp = ++c.clock;
            return &m.tm;
        }
        if (m.stamp < c.e[victim].stamp) victim = i;
    }
    MapEntry& m = c.e[victim];
    m.ptr = nullptr;   // not valid while it is being rewritten
    if (!make_map(&m.tm, base, rows, horizon, horizon)) return nullptr;
    m.ptr = base;
    m.rows = rows;
    m.horizon = horizon;
    m.stamp = ++c.clock;
    return &m.tm;
}

// Tuning knobs (tests, sweeps): process-wide, -1 = automatic.  Initialised once from the
// environment (PUFF_ADV_FORCE_KERNEL, PUFF_ADV_STAGES, PUFF_ADV_WS, PUFF_ADV_CTAS_PER_SM,
// PUFF_ADV_GROUP) and changed at run time through puff_advantage_sm100_set_tuning, so the
// launch path itself never touches the environment.
static std::atomic<int> g_tune[PUFF_TUNE_COUNT];
static std::once_flag g_tune_once;

static void tune_init()
{
    std::call_once(g_tune_once, [] {
        static const char* const names[PUFF_TUNE_COUNT] = {"PUFF_ADV_FORCE_KERNEL", "PUFF_ADV_STAGES", "PUFF_ADV_WS",
                                                           "PUFF_ADV_CTAS_PER_SM", "PUFF_ADV_GROUP",
                                                           "PUFF_ADV_SCAN_THREADS", "PUFF_ADV_RESERVE_SMS",
                                                           "PUFF_ADV_TILE_ROWS", "PUFF_ADV_PDL", "PUFF_ADV_SCAN_WIDE",
                                                           "PUFF_ADV_B1_WARP_TEAMS"};
        for (int i = 0; i < PUFF_TUNE_COUNT; ++i) {
            const char* v = getenv(names[i]);
            g_tune[i].store((v != nullptr && *v != '\0') ? atoi(v) : -1, std::memory_order_relaxed);
        }
    });
}

static int tune(int knob, int fallback)
{
    tune_init();
    const int v = g_tune[knob].load(std::memory_order_relaxed);
    return v < 0 ? fallback : v;
}

// SMs a persistent (warp-specialised) grid is sized for: all of them, minus the few that
// PUFF_TUNE_RESERVE_SMS leaves free for kernels of other streams that must not wait for the
// whole persistent grid to retire (a collective's kernel, for instance)
static int persistent_sms(int sm_count)
{
    const int r = tune(PUFF_TUNE_RESERVE_SMS, 0);
    const int n = sm_count - (r < 0 ? 0 : r);
    return n < 1 ? 1 : n;
}

// Every advantage kernel is launched through launch_kernel() (puff_launch.cuh) with the
// programmatic-stream-serialization attribute (unless PUFF_TUNE_PDL is 0): its set-up may then
// overlap the tail of whatever precedes it in the stream, and it waits (pdl_wait in the kernels)
// for that predecessor to complete before it touches a tensor.
template <int NST>
static cudaError_t launch_tma2d(const MapSet& m, const float* adv_in, float* seg_abs_sum, float gamma, float lambda, float rho_clip,
                                float c_clip, long long rows, int horizon, int grid, int tiles, cudaStream_t st)
{
    if (seg_abs_sum != nullptr)
        return launch_kernel(puff_adv_tma2d_kernel<NST, true>, grid, 32, tma2d_smem_bytes<NST>(), st,
                             m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], adv_in, seg_abs_sum, gamma, lambda, rho_clip,
                             c_clip, rows, horizon, tiles);
    return launch_kernel(puff_adv_tma2d_kernel<NST, false>, grid, 32, tma2d_smem_bytes<NST>(), st,
                         m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], adv_in, static_cast<float*>(nullptr), gamma, lambda,
                         rho_clip, c_clip, rows, horizon, tiles);
}

template <int NST, int NT>
static cudaError_t launch_tma2d_ws(const MapSet& m, const float* adv_in, float* seg_abs_sum, float gamma, float lambda, float rho_clip,
                                   float c_clip, long long rows, int horizon, int grid, int tiles, cudaStream_t st)
{
    int group = tune(PUFF_TUNE_LOAD_GROUP, NST % 2 == 0 ? 2 : 1);
    if (group < 1 || NST % group != 0) group = 1;
    if (seg_abs_sum != nullptr)
        return launch_kernel(puff_adv_tma2d_ws_kernel<NST, NT, true>, grid, kWsThreads, tma2d_ws_smem_bytes<NST, NT>(), st,
                             m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], m.ptr[0], m.ptr[1], m.ptr[2], m.ptr[3], adv_in,
                             seg_abs_sum, gamma, lambda, rho_clip, c_clip, rows, horizon, tiles, group);
    return launch_kernel(puff_adv_tma2d_ws_kernel<NST, NT, false>, grid, kWsThreads, tma2d_ws_smem_bytes<NST, NT>(), st,
                         m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], m.ptr[0], m.ptr[1], m.ptr[2], m.ptr[3], adv_in,
                         static_cast<float*>(nullptr), gamma, lambda, rho_clip, c_clip, rows, horizon, tiles, group);
}

static bool ranges_overlap(const void* a, size_t na, const void* b, size_t nb)
{
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + nb && b0 < a0 + na;
}

// bulk1d tile height: the largest of 32/16/8/4 rows whose tile holds at most kB1MaxElems
// elements (72 KB of stage: three CTAs per SM, and every thread can keep the terms of its
// units in registers); 0 when even four rows do not fit
static int bulk1d_tile_rows(long long horizon, int max_smem, size_t* smem_bytes)
{
    const int cand[4] = {32, 16, 8, 4};
    const int cap = tune(PUFF_TUNE_TILE_ROWS, 32);
    for (int i = 0; i < 4; ++i) {
        if (cand[i] > cap && cand[i] > 4) continue;
        if (static_cast<long long>(cand[i]) * horizon > kB1MaxElems) continue;
        const size_t arr = (static_cast<size_t>(cand[i]) * horizon * 4 + 15) & ~static_cast<size_t>(15);
        const size_t need = 4 * arr + 16 + 128;
        if (need > static_cast<size_t>(max_smem)) continue;
        *smem_bytes = need;
        return cand[i];
    }
    *smem_bytes = 0;
    return 0;
}

// Warp-specialised bulk1d: two raw stages, two terms buffers and two output tiles, 56 bytes of
// shared memory per element of a tile; the largest of 32/16/8/4 rows that fits, 0 if none does
static int bulk1d_ws_tile_rows(long long horizon, int max_smem, size_t* smem_bytes)
{
    const int cand[4] = {32, 16, 8, 4};
    const int cap = tune(PUFF_TUNE_TILE_ROWS, 32);
    for (int i = 0; i < 4; ++i) {
        if (cand[i] > cap && cand[i] > 4) continue;
        const size_t arr = (static_cast<size_t>(cand[i]) * horizon * 4 + 15) & ~static_cast<size_t>(15);
        const size_t need = (kB1wStages * 4 + kB1wTerms * 3) * arr + 8 * (2 * kB1wStages + 2 * kB1wTerms) + 4 * kB1wTerms + 64 + 128;
        if (need > static_cast<size_t>(max_smem)) continue;
        *smem_bytes = need;
        return cand[i];
    }
    *smem_bytes = 0;
    return 0;
}

}  // namespace puff

using namespace puff;

extern "C" int puff_advantage_sm100_launch(const float* values, const float* rewards, const float* dones,
                                           const float* importance, float* advantages, float* seg_abs_sum,
                                           float gamma, float lambda, float rho_clip, float c_clip,
                                           long long num_segments, long long horizon, int variant,
                                           void* cuda_stream)
{
    return puff_advantage_sm100_launch_ex(values, rewards, dones, importance, advantages, seg_abs_sum, gamma, lambda,
                                          rho_clip, c_clip, num_segments, horizon, variant, 0u, cuda_stream);
}

namespace puff {
// NVTX range "puff_advantage" around the host side of every launch, so that a timeline shows the
// op by name (the reference trainer books it under its "train_misc" section, pufferl.py:349).
// Header-only NVTX: a no-op costing a few nanoseconds unless a profiler has injected itself.
struct LaunchRange {
    LaunchRange() { nvtxRangePushA("puff_advantage"); }
    ~LaunchRange() { nvtxRangePop(); }
};
}  // namespace puff

extern "C" int puff_advantage_sm100_launch_ex(const float* values, const float* rewards, const float* dones,
                                              const float* importance, float* advantages, float* seg_abs_sum,
                                              float gamma, float lambda, float rho_clip, float c_clip,
                                              long long num_segments, long long horizon, int variant,
                                              unsigned flags, void* cuda_stream)
{
    const LaunchRange nvtx_range;
    t_last_kernel = PUFF_KERNEL_NONE;
    if (num_segments < 0 || horizon < 0) return PUFF_ERR_SHAPE;
    if (variant < PUFF_VARIANT_AUTO || variant > PUFF_VARIANT_GENERIC) return PUFF_ERR_VARIANT;
    if (flags & ~static_cast<unsigned>(PUFF_FLAG_ZERO_LAST_COLUMN)) return PUFF_ERR_VARIANT;
    const int zero_last = (flags & PUFF_FLAG_ZERO_LAST_COLUMN) ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (num_segments == 0) return PUFF_OK;
    if (horizon < 2) {
        // no step exists: the sums are empty, and advantages is written only when the op owns column H-1
        if (seg_abs_sum != nullptr) {
            cudaError_t e = cudaMemsetAsync(seg_abs_sum, 0, static_cast<size_t>(num_segments) * 4, st);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        if (zero_last && horizon == 1) {
            if (advantages == nullptr) return PUFF_ERR_NULL;
            cudaError_t e = cudaMemsetAsync(advantages, 0, static_cast<size_t>(num_segments) * 4, st);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        return PUFF_OK;
    }
    if (values == nullptr || rewards == nullptr || dones == nullptr || importance == nullptr ||
        advantages == nullptr)
        return PUFF_ERR_NULL;
    const void* ptrs[6] = {values, rewards, dones, importance, advantages, seg_abs_sum};
    bool aligned16 = true;
    for (int i = 0; i < 6; ++i) {
        const uintptr_t p = reinterpret_cast<uintptr_t>(ptrs[i]);
        if (p & 3u) return PUFF_ERR_ALIGN;
        if (i < 5 && (p & 15u)) aligned16 = false;
    }
    const size_t bytes = static_cast<size_t>(num_segments) * static_cast<size_t>(horizon) * 4;
    for (int i = 0; i < 4; ++i) {
        if (ranges_overlap(advantages, bytes, ptrs[i], bytes)) return PUFF_ERR_ALIAS;
        if (seg_abs_sum != nullptr && ranges_overlap(seg_abs_sum, static_cast<size_t>(num_segments) * 4, ptrs[i], bytes))
            return PUFF_ERR_ALIAS;
    }
    if (seg_abs_sum != nullptr && ranges_overlap(seg_abs_sum, static_cast<size_t>(num_segments) * 4, advantages, bytes))
        return PUFF_ERR_ALIAS;

    int code = 0;
    const DeviceInfo* dev = device_info(&code);
    if (dev == nullptr) return code;

    // ---- choose the kernel -------------------------------------------------
    size_t bulk_smem = 0;
    const int bulk_rows = (aligned16 && horizon < (1 << 20)) ? bulk1d_tile_rows(horizon, dev->max_smem_optin, &bulk_smem) : 0;
    const bool can_tma2d = aligned16 && (horizon % 4 == 0) && horizon <= 0x7fffffffLL - 64;
    const bool can_bulk1d = bulk_rows > 0;
    const bool can_scan = horizon <= 0x7fffffffLL - 8;
    int kernel;
    if (variant == PUFF_VARIANT_GENERIC) {
        kernel = PUFF_KERNEL_GENERIC;
    } else if (variant == PUFF_VARIANT_SCAN) {
        kernel = can_scan ? PUFF_KERNEL_SCAN : PUFF_KERNEL_GENERIC;
    } else {
        const int serial_kernel = can_tma2d ? PUFF_KERNEL_TMA2D : (can_bulk1d ? PUFF_KERNEL_BULK1D : PUFF_KERNEL_GENERIC);
        // long rows with too few segments to give every SM a few rows: scan.  Its error bar
        // rests on a contracting recurrence, so AUTO only takes it while gamma*lambda*c_clip <= 1
        // (every gain (gamma*lambda)*min(importance, c_clip) is then at most 1); otherwise the
        // rounding of the re-associated carries could grow along the row, and the bit-exact
        // serial kernel is used instead.
        const bool few_rows = num_segments < static_cast<long long>(dev->sm_count) * 24;
        const float gain_cap = gamma * lambda * c_clip;
        const bool contracting = gain_cap >= 0.0f && gain_cap <= 1.0f;   // false for NaN
        if (variant == PUFF_VARIANT_AUTO && can_scan && few_rows && horizon >= 512 && contracting)
            kernel = PUFF_KERNEL_SCAN;
        else
            kernel = serial_kernel;
    }
    {
        const int forced = tune(PUFF_TUNE_FORCE_KERNEL, 0);   // tests: PUFF_KERNEL_*
        if (forced == PUFF_KERNEL_TMA2D && can_tma2d) kernel = forced;
        if (forced == PUFF_KERNEL_BULK1D && can_bulk1d) kernel = forced;
        if (forced == PUFF_KERNEL_SCAN && can_scan) kernel = forced;
        if (forced == PUFF_KERNEL_GENERIC) kernel = forced;
    }

    cudaError_t err = cudaSuccess;
    if (kernel == PUFF_KERNEL_TMA2D) {
        // TMA coordinates are 32-bit: process blocks of at most 2^30 rows
        const long long block_rows = 1LL << 30;
        static thread_local MapCache map_cache;
        MapSet cache;
        // measured on cfg2 (131072 x 256): two CTAs per SM with a four-stage ring each
        // beat both more, shallower CTAs and one deeper CTA
        int nst = tune(PUFF_TUNE_STAGES, 4);
        nst = nst <= 2 ? 2 : nst == 3 ? 3 : 4;
        const int stage_smem = nst * kStageBytes + 2 * kBoxBytes + nst * 8 + 1024;
        int ctas_per_sm = (dev->max_smem_optin + 1024) / (stage_smem + 1024);
        {
            const int o = tune(PUFF_TUNE_CTAS_PER_SM, nst == 4 ? 2 : 0);
            if (o > 0 && o < ctas_per_sm) ctas_per_sm = o;
        }
        if (ctas_per_sm < 1) ctas_per_sm = 1;
        for (long long r0 = 0; r0 < num_segments && err == cudaSuccess; r0 += block_rows) {
            const long long rows = num_segments - r0 < block_rows ? num_segments - r0 : block_rows;
            const long long off = r0 * horizon;
            const float* p[5] = {values + off, rewards + off, dones + off, importance + off, advantages + off};
            for (int i = 0; i < 5; ++i) {
                const CUtensorMap* tm = cached_map(map_cache, p[i], rows, horizon);
                if (tm == nullptr) return PUFF_ERR_DRIVER;
                cache.tm[i] = *tm;
                cache.ptr[i] = p[i];
            }
            const long long tiles = (rows + kTileRows - 1) / kTileRows;
            float* abs_p = seg_abs_sum != nullptr ? seg_abs_sum + r0 : nullptr;
            // The warp-specialised kernel.  Measured on 131072 x 256: four raw stages whose loads
            // are issued two chunks at a time, two terms buffers, two CTAs per SM (more CTAs per
            // SM lowered the achieved DRAM rate).  With programmatic dependent launch hiding its
            // longer set-up it is level with or ahead of the single-warp kernel at every size
            // measured (single-warp / warp-specialised, us): 1024 x 64 3.34 / 3.34, 8192 x 64
            // 4.73 / 4.67, 1024 x 256 8.92 / 6.65, 4096 x 256 9.65 / 7.78, 8192 x 128 7.73 / 6.64,
            // 32768 x 64 11.98 / 10.48, 524288 x 64 115.7 / 110.9, 1048576 x 32 131.0 / 129.1.
            // PUFF_TUNE_WS_STAGES: 0 = single-warp, N = warp-specialised with N raw stages (2, 3, 4, 6).
            const int ws = tune(PUFF_TUNE_WS_STAGES, 4);
            if (ws != 0) {
                const int wnst = ws <= 2 ? 2 : ws == 3 ? 3 : ws <= 5 ? 4 : 6;
                const int smem = wnst * kStageBytes + 2 * kTermBytes + kWsOutSlots * kBoxBytes + 2048;
                int per_sm = (dev->max_smem_optin + 1024) / (smem + 1024);
                if (per_sm > 2) per_sm = 2;
                { const int o = tune(PUFF_TUNE_CTAS_PER_SM, 0); if (o > 0) per_sm = o < 3 ? o : 3; }
                if (per_sm < 1) per_sm = 1;
                const long long mg = static_cast<long long>(persistent_sms(dev->sm_count)) * per_sm;
                const int grid = static_cast<int>(tiles < mg ? tiles : mg);
#define PUFF_WS_CASE(A, B) err = launch_tma2d_ws<A, B>(cache, zero_last ? nullptr : p[4], abs_p, gamma, lambda, rho_clip, c_clip, rows, static_cast<int>(horizon), grid, static_cast<int>(tiles), st)
                if (wnst == 2) PUFF_WS_CASE(2, 2);
                else if (wnst == 3) PUFF_WS_CASE(3, 2);
                else if (wnst == 4) PUFF_WS_CASE(4, 2);
                else PUFF_WS_CASE(6, 2);
#undef PUFF_WS_CASE
                g_launch_count.fetch_add(1, std::memory_order_relaxed);
                continue;
            }
            const long long max_grid = static_cast<long long>(dev->sm_count) * ctas_per_sm;
            const int grid = static_cast<int>(tiles < max_grid ? tiles : max_grid);
#define PUFF_TMA2D_CASE(N)                                                                               \
    err = launch_tma2d<N>(cache, zero_last ? nullptr : p[4], abs_p, gamma, lambda, rho_clip, c_clip, rows, static_cast<int>(horizon), grid, \
                          static_cast<int>(tiles), st)
            switch (nst) {
                case 2: PUFF_TMA2D_CASE(2); break;
                case 3: PUFF_TMA2D_CASE(3); break;
                default: PUFF_TMA2D_CASE(4); break;
            }
#undef PUFF_TMA2D_CASE
            g_launch_count.fetch_add(1, std::memory_order_relaxed);
        }
    } else if (kernel == PUFF_KERNEL_BULK1D) {
        // PUFF_TUNE_WS_STAGES: 0 = one-stage kernel, otherwise the warp-specialised pipeline
        size_t ws_smem = 0;
        const int ws_rows = bulk1d_ws_tile_rows(horizon, dev->max_smem_optin, &ws_smem);
        // measured at H = 127 (one-stage against pipeline): 10007 rows, two tiles per SM, 9.9 against
        // 10.2 us; 20000 rows 17.7 / 13.8; 32768 rows 25.1 / 17.4; 131072 rows 67.2 / 54.9.  The
        // pipeline takes over from three tiles per SM.
        const long long ws_tiles = ws_rows > 0 ? (num_segments + ws_rows - 1) / ws_rows : 0;
        const int use_ws = ws_rows > 0 ? tune(PUFF_TUNE_WS_STAGES, ws_tiles >= 3LL * dev->sm_count ? 1 : 0) : 0;
        if (use_ws != 0) {
            const long long tiles = (num_segments + ws_rows - 1) / ws_rows;
            const long long max_grid = persistent_sms(dev->sm_count);
            const int grid = static_cast<int>(tiles < max_grid ? tiles : max_grid);
            err = launch_kernel(puff_adv_bulk1d_ws_kernel, grid, kB1wThreads, ws_smem, st, values, rewards, dones,
                                importance, advantages, seg_abs_sum, gamma, lambda, rho_clip, c_clip, num_segments,
                                static_cast<int>(horizon), ws_rows, tiles, zero_last);
        } else if (horizon * 8 <= kB1WarpMaxElems && tune(PUFF_TUNE_B1_WARP_TEAMS, 1) != 0) {
            // four warps per CTA, each on 8-row tiles of its own
            const int teams = 4;
            const int rows = 8;
            const size_t arr = (static_cast<size_t>(rows) * horizon * 4 + 15) & ~static_cast<size_t>(15);
            const size_t smem = teams * 4 * arr + 4 * 8 + 16 + 128;
            const long long tiles = (num_segments + rows - 1) / rows;
            const long long ctas = (tiles + teams - 1) / teams;
            int per_sm = static_cast<int>(static_cast<size_t>(dev->max_smem_optin + 1024) / (smem + 1024));
            per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
            const long long max_grid = static_cast<long long>(dev->sm_count) * per_sm;
            const int grid = static_cast<int>(ctas < max_grid ? ctas : max_grid);
            err = launch_kernel(puff_adv_bulk1d_kernel<32>, grid, kB1Threads, smem, st, values, rewards, dones, importance,
                                advantages, seg_abs_sum, gamma, lambda, rho_clip, c_clip, num_segments,
                                static_cast<int>(horizon), rows, tiles, zero_last);
        } else {
        const long long tiles = (num_segments + bulk_rows - 1) / bulk_rows;
        int per_sm = static_cast<int>(static_cast<size_t>(dev->max_smem_optin + 1024) / (bulk_smem + 1024));
        per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
        const long long max_grid = static_cast<long long>(dev->sm_count) * per_sm;
        const int grid = static_cast<int>(tiles < max_grid ? tiles : max_grid);
        err = launch_kernel(puff_adv_bulk1d_kernel<kB1Threads>, grid, kB1Threads, bulk_smem, st, values, rewards, dones,
                            importance, advantages, seg_abs_sum, gamma, lambda, rho_clip, c_clip, num_segments,
                            static_cast<int>(horizon), bulk_rows, tiles, zero_last);
        }
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
    } else if (kernel == PUFF_KERNEL_SCAN) {
        // Threads per row: a power of two up to 512 (with ~60 registers per thread two such CTAs
        // share an SM, so 256 rows of 4096 columns run as one wave).  A thread takes four columns
        // per pass, or eight when the row would otherwise need a second pass: half the scans and
        // barriers, and all of a thread's loads in flight at once.
        // Threads per row.  Few rows: as many as the row has 4-column units, up to 512, so that the
        // SMs are busy at all (256 x 4096: 6.8 us with 512, 7.7 with 256, 9.7 with 128).  Many rows:
        // fewer threads per row, so that several rows are in flight per SM and one row's loads
        // overlap the others' scans -- as many as keep all rows resident at once, but no fewer than
        // one eight-column pass needs (or 128).  Measured: 2048 x 4096 34.3 us with 512 threads per
        // row, 29.4 with 128; 3000 x 1024 15.3 / 12.0; 512 x 4096 11.4 / 10.2 (256); 3500 x 512
        // 8.9 (128) / 8.1 (64).
        const long long units4 = (horizon + 3) / 4;
        int nt = 32;
        while (nt < 512 && nt < units4) nt <<= 1;
        {
            int cap = 512;
            while (cap > 32 && static_cast<long long>(cap) * num_segments > 1280LL * dev->sm_count) cap >>= 1;
            int floor_nt = 32;   // threads of one eight-column pass, at most 128
            while (floor_nt < 128 && 2LL * floor_nt < units4) floor_nt <<= 1;
            if (cap < floor_nt) cap = floor_nt;
            if (nt > cap) nt = cap;
        }
        {
            const int o = tune(PUFF_TUNE_SCAN_THREADS, 0);
            if (o >= 32 && o <= 1024 && (o & (o - 1)) == 0) nt = o;
        }
        const bool wide = units4 > nt && nt <= 512 && tune(PUFF_TUNE_SCAN_WIDE, 1) != 0;
        const long long max_grid = static_cast<long long>(dev->sm_count) * (2048 / nt) ;
        const int grid = static_cast<int>(num_segments < max_grid ? num_segments : max_grid);
        const bool vec = aligned16 && horizon % 4 == 0;
#define PUFF_SCAN_CASE(V, U)                                                                                          \
    err = launch_kernel(puff_adv_scan_kernel<V, U>, grid, nt, 0, st, values, rewards, dones, importance, advantages, \
                        seg_abs_sum, gamma, lambda, rho_clip, c_clip, num_segments, static_cast<int>(horizon), zero_last)
        if (vec && wide) PUFF_SCAN_CASE(true, 2);
        else if (vec) PUFF_SCAN_CASE(true, 1);
        else if (wide) PUFF_SCAN_CASE(false, 2);
        else PUFF_SCAN_CASE(false, 1);
#undef PUFF_SCAN_CASE
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
    } else {
        const long long blocks = (num_segments + 127) / 128;
        const long long max_grid = static_cast<long long>(dev->sm_count) * 16;
        const int grid = static_cast<int>(blocks < max_grid ? blocks : max_grid);
        err = launch_kernel(puff_adv_generic_kernel, grid, 128, 0, st, values, rewards, dones, importance, advantages,
                            seg_abs_sum, gamma, lambda, rho_clip, c_clip, num_segments, horizon, zero_last);
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
    }
    t_last_kernel = kernel;
    return static_cast<int>(err);
}

extern "C" const char* puff_advantage_sm100_strerror(int code)
{
    switch (code) {
        case PUFF_OK: return "success";
        case PUFF_ERR_NULL: return "a required pointer is NULL";
        case PUFF_ERR_SHAPE: return "num_segments and horizon must be non-negative";
        case PUFF_ERR_VARIANT: return "unknown kernel variant";
        case PUFF_ERR_ALIGN: return "pointers must be 4-byte aligned";
        case PUFF_ERR_ALIAS: return "output buffers must not overlap the inputs";
        case PUFF_ERR_ARCH: return "the current CUDA device is not compute capability 10.x (sm_100a build)";
        case PUFF_ERR_DRIVER: return "cuTensorMapEncodeTiled is unavailable or rejected the tensor map";
        case PUFF_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel gave up";
        case PUFF_ERR_WORKSPACE: return "scratch or workspace missing, misaligned or too small";
        case PUFF_ERR_SIZE: return "size beyond what this entry point supports";
        case PUFF_ERR_DEVICE_BOUNDS: return "a kernel formed an out-of-range index (debug build)";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error code";
}

extern "C" int puff_advantage_sm100_last_kernel(void) { return t_last_kernel; }

extern "C" long long puff_advantage_sm100_launch_count(void)
{
    return g_launch_count.load(std::memory_order_relaxed);
}

namespace puff {
void count_launch() { g_launch_count.fetch_add(1, std::memory_order_relaxed); }
int tune_value(int knob, int fallback) { return tune(knob, fallback); }
}

namespace puff {
// Device address of the status word on the current device (nullptr on failure), for kernels of
// other translation units that report into the same word.
int* device_status_ptr()
{
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    return static_cast<int*>(p);
}

// Reads (and, when set, clears) the status word of the current device.  The caller has already
// synchronised the streams whose kernels it asks about.
int take_device_status()
{
    int h = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&h, g_device_status, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (h != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    }
    return h;
}
}  // namespace puff

extern "C" int puff_advantage_sm100_device_status(void)
{
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    return take_device_status();
}

extern "C" int puff_advantage_sm100_inject_status(int value)
{
    return static_cast<int>(cudaMemcpyToSymbol(g_device_status, &value, sizeof(int)));
}

#ifdef PUFF_TIMELINE
// Debug builds only: copies the per-CTA phase stamps (kTimelineSlots per CTA: clock64 values or
// cycle totals, %globaltimer anchors in slots 12 and 14) of the most recent instrumented launch
// into `out`.
extern "C" int puff_advantage_sm100_timeline(unsigned long long* out, int ctas)
{
    if (ctas > kTimelineCtas) ctas = kTimelineCtas;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess)
        e = cudaMemcpyFromSymbol(out, g_timeline, sizeof(unsigned long long) * kTimelineSlots * ctas);
    return static_cast<int>(e);
}
#endif

extern "C" int puff_advantage_sm100_set_tuning(int knob, int value)
{
    if (knob < 0 || knob >= PUFF_TUNE_COUNT) return PUFF_ERR_VARIANT;
    tune_init();
    return g_tune[knob].exchange(value < 0 ? -1 : value, std::memory_order_relaxed);
}

extern "C" const char* puff_advantage_sm100_version(void) { return "0.1"; }

#ifdef PUFF_DEBUG_BOUNDS
// Debug builds only: proves that the index checks are compiled in and report.  One thread asks for
// element `index` of an array of `extent` floats; an index outside it is recorded in the status
// word and the access is skipped.
namespace puff {
__global__ void puff_bounds_selftest_kernel(float* buf, long long index, long long extent)
{
    stg_chk(buf, index, extent, 1.0f);
}
}  // namespace puff
extern "C" int puff_advantage_sm100_bounds_selftest(float* device_buf, long long index, long long extent)
{
    puff_bounds_selftest_kernel<<<1, 1>>>(device_buf, index, extent);
    return static_cast<int>(cudaGetLastError());
}
#endif
