// V-trace-clipped GAE advantage kernels for sm_100a and their C-ABI launcher.
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
// Kernels
//   tma2d   serial, bit-exact.  One warp per CTA owns a tile of 32 segments;
//           the horizon is walked backwards in chunks of 32 columns.  Each
//           chunk of the four inputs arrives as a 32x32 TMA box in
//           128B-swizzled shared memory behind an mbarrier ring, lane r runs
//           row r's recurrence out of shared memory with conflict-free 128-bit
//           reads, and the advantages leave through a TMA store.  TMA clips a
//           store at the tensor edge in whole 16-byte units only, so column
//           H-1 cannot be masked out of the box: each lane reads its row's
//           advantages[H-1] once per tile and the store writes that same value
//           back.  Needs H % 4 == 0 and 16-byte aligned base pointers.
//   bulk1d  serial, bit-exact, for H % 4 != 0 (row pitch not a multiple of
//           16 bytes, so no 2-D tensor map exists): tiles of 4..32 whole rows
//           are contiguous spans, fetched with 1-D bulk copies.
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
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "../../include/puff_advantage.h"

namespace puff {

// ---------------------------------------------------------------------------
// device-side status word and launch counter
// ---------------------------------------------------------------------------
__device__ int g_device_status = 0;
static std::atomic<long long> g_launch_count{0};
static thread_local int t_last_kernel = PUFF_KERNEL_NONE;

constexpr int kTileRows = 32;              // segments per warp tile
constexpr int kChunkCols = 32;             // columns per TMA box (128 bytes)
constexpr int kBoxBytes = kTileRows * kChunkCols * 4;   // 4096
constexpr int kStageBytes = 4 * kBoxBytes;              // v, r, d, w
constexpr uint32_t kWaitLimit = 1u << 24;             // mbarrier polls before giving up ...
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // ... or two seconds, whichever comes first

// ---------------------------------------------------------------------------
// the recurrence step, in the reference's operation order
// (pufferlib/extensions/pufferlib.cpp:34-38).  Explicit round-to-nearest
// intrinsics are never contracted into FMAs, which is what keeps the serial
// kernels bit-identical to the CPU build of the reference.  `1.0 - dones` is a
// double subtraction there; for fp32 operands the fp32 subtraction rounds to
// the same value (53 >= 2*24 + 2).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float adv_step(float v_t, float w_t, float v_n, float r_n,
                                          float d_n, float a_next, float gamma, float gl,
                                          float rho_clip, float c_clip)
{
    const float nn = __fsub_rn(1.0f, d_n);
    const float rho = fminf(w_t, rho_clip);
    const float c = fminf(w_t, c_clip);
    const float td = __fsub_rn(__fadd_rn(r_n, __fmul_rn(__fmul_rn(gamma, v_n), nn)), v_t);
    const float delta = __fmul_rn(rho, td);
    const float carry = __fmul_rn(__fmul_rn(__fmul_rn(gl, c), a_next), nn);
    return __fadd_rn(delta, carry);
}

// The part of a step that does not depend on the running advantage:
//   delta = rho * ((r' + (gamma*v')*nn) - v),  gc = (gamma*lambda)*c,  nn = 1 - d'
// so that A = delta + (gc * A_next) * nn reproduces adv_step() bit for bit.
__device__ __forceinline__ void adv_terms(float v_t, float w_t, float v_n, float r_n, float d_n,
                                          float gamma, float gl, float rho_clip, float c_clip,
                                          float& delta, float& gc, float& nn)
{
    nn = __fsub_rn(1.0f, d_n);
    const float rho = fminf(w_t, rho_clip);
    const float c = fminf(w_t, c_clip);
    const float td = __fsub_rn(__fadd_rn(r_n, __fmul_rn(__fmul_rn(gamma, v_n), nn)), v_t);
    delta = __fmul_rn(rho, td);
    gc = __fmul_rn(gl, c);
}

// ---------------------------------------------------------------------------
// PTX wrappers: mbarrier, TMA (non-multicast), bulk groups
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// One try_wait.  The suspend-time hint lets the hardware park the thread until the phase
// completes (or the hint runs out) instead of spinning through the loop below: most warps
// of the warp-specialised kernel spend most of their time waiting, and a spinning warp
// costs issue slots and power that the memory-bound kernel pays for in clock speed.
constexpr uint32_t kWaitHintNs = 200000u;
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait; returns true when every lane of the warp saw the phase flip.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity)
{
    uint32_t ok = mbar_try_wait(bar, parity);
    if (!ok) {
        const unsigned long long t0 = global_ns();
        uint32_t polls = 0;
        while (!ok && polls < kWaitLimit) {
            ok = mbar_try_wait(bar, parity);
            if (!ok && ((++polls & 15u) == 0u) && global_ns() - t0 > kWaitLimitNs) break;
        }
    }
    return __all_sync(0xffffffffu, ok != 0);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tm), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, int x, int y, uint32_t src)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm),
                 "r"(x), "r"(y), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tm)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}
__device__ __forceinline__ float4 lds128(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, float4 v)
{
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
                 "f"(v.w)
                 : "memory");
}


// ---------------------------------------------------------------------------
// one 32-column chunk of one row, out of a 128B-swizzled stage
// ---------------------------------------------------------------------------
// sum of |x[j]| in a fixed pairwise order
__device__ __forceinline__ float abs_tree32(const float (&x)[32])
{
    float t[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) t[j] = __fadd_rn(fabsf(x[2 * j + 1]), fabsf(x[2 * j]));
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = __fadd_rn(t[2 * j + 1], t[2 * j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) t[j] = __fadd_rn(t[2 * j + 1], t[2 * j]);
    return __fadd_rn(__fadd_rn(t[3], t[2]), __fadd_rn(t[1], t[0]));
}

// Literal path: the reference's operation order step by step, any H % 4 == 0,
// columns at or beyond H-1 skipped (the advantage stays what it was).
__device__ __forceinline__ void chunk_literal(uint32_t st, uint32_t row_off, uint32_t sw, int cbase, int horizon,
                                              float gamma, float gl, float rho_clip, float c_clip,
                                              float& a_run, float& nv, float& nr, float& nd, float (&out)[32])
{
#pragma unroll
    for (int q = 7; q >= 0; --q) {
        const int col0 = cbase + 4 * q;
        out[4 * q] = out[4 * q + 1] = out[4 * q + 2] = out[4 * q + 3] = 0.0f;
        if (col0 < horizon) {   // warp-uniform
            const uint32_t off = row_off + ((static_cast<uint32_t>(q) ^ sw) << 4);
            const float4 v4 = lds128(st + 0 * kBoxBytes + off);
            const float4 r4 = lds128(st + 1 * kBoxBytes + off);
            const float4 d4 = lds128(st + 2 * kBoxBytes + off);
            const float4 w4 = lds128(st + 3 * kBoxBytes + off);
            if (col0 + 4 < horizon) {   // column col0+3 is H-1 in the last unit of a row: no step
                a_run = adv_step(v4.w, w4.w, nv, nr, nd, a_run, gamma, gl, rho_clip, c_clip);
                out[4 * q + 3] = a_run;
            }
            a_run = adv_step(v4.z, w4.z, v4.w, r4.w, d4.w, a_run, gamma, gl, rho_clip, c_clip);
            out[4 * q + 2] = a_run;
            a_run = adv_step(v4.y, w4.y, v4.z, r4.z, d4.z, a_run, gamma, gl, rho_clip, c_clip);
            out[4 * q + 1] = a_run;
            a_run = adv_step(v4.x, w4.x, v4.y, r4.y, d4.y, a_run, gamma, gl, rho_clip, c_clip);
            out[4 * q] = a_run;
            nv = v4.x;
            nr = r4.x;
            nd = d4.x;
        }
    }
}

// Packed path for a chunk whose 32 columns all lie inside the row.  Everything
// that does not depend on the running advantage is computed first, two steps
// per instruction with the f32x2 forms of the same IEEE operations (so every
// intermediate equals the scalar one bit for bit):
//     nn = 1 - d'          as fma(d', -1, 1)       (the product is exact)
//     delta = rho * ((r' + (gamma*v')*nn) - v),    k = ((gamma*lambda)*c) * nn
// and the serial part is A = delta + k*A.  The reference evaluates
// ((gamma*lambda*c)*A)*nn; for nn in {0, 1} that is the same fp32 value as
// (gamma*lambda*c*nn)*A unless the inner product overflows.  Returns false --
// and the caller redoes the chunk literally -- when any lane saw d'*nn != 0
// (nn is not exactly 0 or 1) or advantages beyond 1e30.
// `row_end`: column cbase+31 is H-1, which has no step.
__device__ __forceinline__ bool chunk_packed(uint32_t st, uint32_t row_off, uint32_t sw, bool row_end,
                                             float gamma, float gl, float rho_clip, float c_clip,
                                             float& a_run, float& nv, float& nr, float& nd, float (&out)[32])
{
    float vc[33], rc[33], dc[33], wc[32];   // index j <-> column cbase + j; 32 = carried from the later chunk
    vc[32] = nv;
    rc[32] = nr;
    dc[32] = nd;
#pragma unroll
    for (int u = 7; u >= 0; --u) {
        const uint32_t off = row_off + ((static_cast<uint32_t>(u) ^ sw) << 4);
        const float4 v4 = lds128(st + 0 * kBoxBytes + off);
        const float4 r4 = lds128(st + 1 * kBoxBytes + off);
        const float4 d4 = lds128(st + 2 * kBoxBytes + off);
        const float4 w4 = lds128(st + 3 * kBoxBytes + off);
        vc[4 * u] = v4.x; vc[4 * u + 1] = v4.y; vc[4 * u + 2] = v4.z; vc[4 * u + 3] = v4.w;
        rc[4 * u] = r4.x; rc[4 * u + 1] = r4.y; rc[4 * u + 2] = r4.z; rc[4 * u + 3] = r4.w;
        dc[4 * u] = d4.x; dc[4 * u + 1] = d4.y; dc[4 * u + 2] = d4.z; dc[4 * u + 3] = d4.w;
        wc[4 * u] = w4.x; wc[4 * u + 1] = w4.y; wc[4 * u + 2] = w4.z; wc[4 * u + 3] = w4.w;
    }
    nv = vc[0];
    nr = rc[0];
    nd = dc[0];

    float dl[32], kk[32];
    uint32_t nonbin = 0u;
    const float a_in = a_run;
    // step 31 alone (its t+1 operands are the carried ones); masked at the end of a row
    {
        float d, g, n;
        adv_terms(vc[31], wc[31], vc[32], rc[32], dc[32], gamma, gl, rho_clip, c_clip, d, g, n);
        nonbin |= __float_as_uint(__fmul_rn(dc[32], n));
        dl[31] = row_end ? 0.0f : d;
        kk[31] = row_end ? 0.0f : __fmul_rn(g, n);
    }
    // steps (j, j+1) for odd j: their t+1 operands (j+1, j+2) are aligned register pairs
    const float2 neg1 = make_float2(-1.0f, -1.0f), one2 = make_float2(1.0f, 1.0f);
    const float2 gamma2 = make_float2(gamma, gamma), gl2 = make_float2(gl, gl);
#pragma unroll
    for (int j = 29; j >= 1; j -= 2) {
        const float2 dn = make_float2(dc[j + 1], dc[j + 2]);
        const float2 vn = make_float2(vc[j + 1], vc[j + 2]);
        const float2 rn = make_float2(rc[j + 1], rc[j + 2]);
        const float2 nn2 = __ffma2_rn(dn, neg1, one2);
        const float2 t2 = __fadd2_rn(rn, __fmul2_rn(__fmul2_rn(gamma2, vn), nn2));
        const float2 td2 = make_float2(__fsub_rn(t2.x, vc[j]), __fsub_rn(t2.y, vc[j + 1]));
        const float2 rho2 = make_float2(fminf(wc[j], rho_clip), fminf(wc[j + 1], rho_clip));
        const float2 c2 = make_float2(fminf(wc[j], c_clip), fminf(wc[j + 1], c_clip));
        const float2 d2 = __fmul2_rn(rho2, td2);
        const float2 k2 = __fmul2_rn(__fmul2_rn(gl2, c2), nn2);
        const float2 q2 = __fmul2_rn(dn, nn2);
        nonbin |= __float_as_uint(q2.x) | __float_as_uint(q2.y);
        dl[j] = d2.x;
        dl[j + 1] = d2.y;
        kk[j] = k2.x;
        kk[j + 1] = k2.y;
    }
    {
        float d, g, n;
        adv_terms(vc[0], wc[0], vc[1], rc[1], dc[1], gamma, gl, rho_clip, c_clip, d, g, n);
        nonbin |= __float_as_uint(__fmul_rn(dc[1], n));
        dl[0] = d;
        kk[0] = __fmul_rn(g, n);
    }
    // the serial part
    float a = a_in;
#pragma unroll
    for (int j = 31; j >= 0; --j) {
        a = __fadd_rn(dl[j], __fmul_rn(kk[j], a));
        out[j] = a;
    }
    a_run = a;
    const float big = __fadd_rn(fabsf(a_in), abs_tree32(out));
    const bool ok = ((nonbin << 1) == 0u) && (big <= 1e30f);
    return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------
// tma2d: serial, one warp per CTA, 32-row x 32-column TMA boxes
// ---------------------------------------------------------------------------
// Shared memory (offsets from a 1024-byte aligned base, which the 128B swizzle
// pattern is anchored to):
//   [0, NST*16K)            NST stages, each v | r | d | w boxes of 4 KB
//   [NST*16K, NST*16K+8K)   two output boxes (ring for the TMA stores)
//   then NST mbarriers
// In a 128B-swizzled box the 16-byte unit q of row r sits at
// r*128 + ((q ^ (r & 7)) << 4): lane r reading unit q of its own row touches
// eight different units per quarter-warp, i.e. no bank conflicts.
template <int NST>
constexpr int tma2d_smem_bytes()
{
    return NST * kStageBytes + 2 * kBoxBytes + NST * 8 + 1024;
}

template <int NST, bool EPI>
__global__ void __launch_bounds__(32)
puff_adv_tma2d_kernel(const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_r,
                      const __grid_constant__ CUtensorMap tm_d,
                      const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_a,
                      const float* adv_in, float* __restrict__ seg_abs_sum, float gamma, float lambda,
                      float rho_clip, float c_clip, long long num_segments, int horizon, int num_tiles)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t out_base = base + NST * kStageBytes;
    const uint32_t bar_base = out_base + 2 * kBoxBytes;
    const int lane = threadIdx.x;

    if (static_cast<int>(blockIdx.x) >= num_tiles) return;
    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                         static_cast<int>(gridDim.x);
    const int nchunks = (horizon + kChunkCols - 1) / kChunkCols;
    const int total = my_tiles * nchunks;

    if (lane == 0) {
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_r);
        prefetch_tensormap(&tm_d);
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_a);
        for (int s = 0; s < NST; ++s) mbar_init(bar_base + 8 * s, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncwarp();

    // work item i -> (tile, chunk); chunks of a tile run from the last column block down
    auto issue = [&](int i) {
        const int k = i / nchunks;
        const int c = nchunks - 1 - (i - k * nchunks);
        const int tile = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
        const int s = i % NST;
        const uint32_t st = base + s * kStageBytes;
        const uint32_t bar = bar_base + 8 * s;
        const int x = c * kChunkCols;
        const int y = tile * kTileRows;
        mbar_expect_tx(bar, kStageBytes);
        tma_load_2d(st + 0 * kBoxBytes, &tm_v, x, y, bar);
        tma_load_2d(st + 1 * kBoxBytes, &tm_r, x, y, bar);
        tma_load_2d(st + 2 * kBoxBytes, &tm_d, x, y, bar);
        tma_load_2d(st + 3 * kBoxBytes, &tm_w, x, y, bar);
    };

    if (lane == 0) {
        const int pre = total < NST ? total : NST;
        for (int i = 0; i < pre; ++i) issue(i);
    }

    const float gl = __fmul_rn(gamma, lambda);
    const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
    const uint32_t sw = static_cast<uint32_t>(lane) & 7u;

    float a_run = 0.0f, abs_run = 0.0f;
    float nv = 0.0f, nr = 0.0f, nd = 0.0f;   // values/rewards/dones at column t+1 across units
    float keep_last = 0.0f;                  // the caller's advantages[row, H-1]
    int k = 0, c = nchunks - 1, s = 0;
    uint32_t parity = 0;
    bool failed = false;

    for (int i = 0; i < total; ++i) {
        if (c == nchunks - 1) {   // new tile
            const long long row = (static_cast<long long>(blockIdx.x) + static_cast<long long>(k) * gridDim.x) * kTileRows + lane;
            keep_last = (adv_in != nullptr && row < num_segments) ? adv_in[row * horizon + horizon - 1] : 0.0f;
            a_run = 0.0f;
            abs_run = 0.0f;
        }
        // the output box i&1 was last read by the store of item i-2
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        if (!mbar_wait_warp(bar_base + 8 * s, parity)) {
            failed = true;
            break;
        }
        const uint32_t st = base + s * kStageBytes;
        const uint32_t ob = out_base + (i & 1) * kBoxBytes;
        const int cbase = c * kChunkCols;
        float out[32];   // advantages of columns cbase .. cbase+31 of this lane's row
        const float a_in = a_run, nv_in = nv, nr_in = nr, nd_in = nd;
        // Full chunks take the packed path; a last chunk that ends inside the box
        // (H % 32 != 0) and chunks that fail the checks below take the literal one.
        bool literal = (cbase + kChunkCols > horizon);
        if (!literal) {
            literal = !chunk_packed(st, row_off, sw, cbase + kChunkCols == horizon, gamma, gl, rho_clip, c_clip,
                                    a_run, nv, nr, nd, out);
        }
        if (literal) {
            a_run = a_in;
            nv = nv_in;
            nr = nr_in;
            nd = nd_in;
            chunk_literal(st, row_off, sw, cbase, horizon, gamma, gl, rho_clip, c_clip, a_run, nv, nr, nd, out);
        }
        if (EPI) abs_run = __fadd_rn(abs_run, abs_tree32(out));
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t off = row_off + ((static_cast<uint32_t>(u) ^ sw) << 4);
            float4 a4 = make_float4(out[4 * u], out[4 * u + 1], out[4 * u + 2], out[4 * u + 3]);
            // column H-1 (last of its unit, H % 4 == 0) goes back unchanged
            if (cbase + 4 * u + 3 == horizon - 1) a4.w = keep_last;
            sts128(ob + off, a4);
        }
        const int tile = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
        if (EPI && c == 0) {
            const long long row = static_cast<long long>(tile) * kTileRows + lane;
            if (row < num_segments) seg_abs_sum[row] = abs_run;
        }
        // generic-proxy reads of the stage and writes of the output box are
        // ordered before the async-proxy operations issued below
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(&tm_a, cbase, tile * kTileRows, ob);
            bulk_commit();
            if (i + NST < total) issue(i + NST);
        }
        if (--c < 0) {
            c = nchunks - 1;
            ++k;
        }
        if (++s == NST) {
            s = 0;
            parity ^= 1u;
        }
    }
    if (lane == 0) {
        // the stores only have to be done reading shared memory before the CTA exits;
        // their global writes complete with the grid
        bulk_wait_read<0>();
        if (failed) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    }
}


// ---------------------------------------------------------------------------
// tma2d, warp-specialised: one CTA per tile stream, six warps with three roles
// ---------------------------------------------------------------------------
// A lone warp per tile cannot issue instructions fast enough to keep up with
// HBM once the pipeline is deep (measured: one such warp per SM is compute
// bound at about a third of the bandwidth).  Here the work of a 32x32 chunk is
// split by dependency instead:
//   warp 0      producer: waits for a free stage, issues the four TMA loads
//   warps 2..5  terms:    128 threads, 8 columns of one row each, read the raw
//                         boxes and write delta and k = (gamma*lambda*c)*nn of
//                         every step into a terms buffer (same swizzled layout);
//                         columns without a step get delta = k = 0
//   warp 1      chain:    lane r walks row r's 32 steps from the terms buffer,
//                         A = delta + k*A, stores the advantages by TMA.  When the
//                         terms warps flagged a non-binary nn, or A nears the
//                         overflow range, it redoes the chunk in the reference's
//                         literal order straight from global memory (rare, slow)
// Rings: NST raw stages (full: TMA -> terms, sfree: terms -> producer) and NT
// terms buffers (tfull: terms -> chain, tfree: chain -> terms).
constexpr int kWsTermWarps = 4;
constexpr int kWsThreads = 32 * (2 + kWsTermWarps);
constexpr int kTermBytes = 2 * kBoxBytes;   // delta | k = (gamma*lambda*c)*nn

constexpr int kWsOutSlots = 2;   // output boxes in flight behind the TMA stores
template <int NST, int NT>
constexpr int tma2d_ws_smem_bytes()
{
    return NST * kStageBytes + NT * kTermBytes + kWsOutSlots * kBoxBytes + (2 * NST + 2 * NT) * 8 + NT * 4 + 64 + 1024;
}

__device__ __forceinline__ bool mbar_wait_thread(uint32_t bar, uint32_t parity)
{
    uint32_t ok = mbar_try_wait(bar, parity);
    if (!ok) {
        const unsigned long long t0 = global_ns();
        uint32_t polls = 0;
        while (!ok && polls < kWaitLimit) {
            ok = mbar_try_wait(bar, parity);
            if (!ok && ((++polls & 15u) == 0u) && global_ns() - t0 > kWaitLimitNs) break;
        }
    }
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float lds32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lds32u(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void sts32u(uint32_t addr, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

template <int NST, int NT, bool EPI>
__global__ void __launch_bounds__(kWsThreads)
puff_adv_tma2d_ws_kernel(const __grid_constant__ CUtensorMap tm_v,
                         const __grid_constant__ CUtensorMap tm_r,
                         const __grid_constant__ CUtensorMap tm_d,
                         const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_a,
                         const float* __restrict__ raw_v, const float* __restrict__ raw_r,
                         const float* __restrict__ raw_d, const float* __restrict__ raw_w,
                         const float* adv_in, float* __restrict__ seg_abs_sum, float gamma, float lambda,
                         float rho_clip, float c_clip, long long num_segments, int horizon, int num_tiles,
                         int group)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t term_base = base + NST * kStageBytes;
    const uint32_t out_base = term_base + NT * kTermBytes;
    const uint32_t bar_full = out_base + kWsOutSlots * kBoxBytes;
    const uint32_t bar_sfree = bar_full + 8 * NST;
    const uint32_t bar_tfull = bar_sfree + 8 * NST;
    const uint32_t bar_tfree = bar_tfull + 8 * NT;
    const uint32_t flag_base = bar_tfree + 8 * NT;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                         static_cast<int>(gridDim.x);
    const int nchunks = (horizon + kChunkCols - 1) / kChunkCols;
    const int total = my_tiles * nchunks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_sfree + 8 * s, kWsTermWarps);
        }
        for (int b = 0; b < NT; ++b) {
            mbar_init(bar_tfull + 8 * b, kWsTermWarps);
            mbar_init(bar_tfree + 8 * b, 1);
            sts32u(flag_base + 4 * b, 0u);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    const float gl = __fmul_rn(gamma, lambda);
    bool failed = false;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            prefetch_tensormap(&tm_v);
            prefetch_tensormap(&tm_r);
            prefetch_tensormap(&tm_d);
            prefetch_tensormap(&tm_w);
            // Loads are issued in groups of `group` consecutive chunks (NST % group == 0):
            // the producer waits until all their stages are free and then issues them back
            // to back, so that DRAM sees group*128 contiguous bytes of every row at once.
            int k = 0, c = nchunks - 1, s = 0, round = 0;
            for (int i = 0; i < total && !failed; i += group) {
                const int n = total - i < group ? total - i : group;
                if (round > 0) {
                    for (int j = 0; j < n; ++j) {
                        if (!mbar_wait_thread(bar_sfree + 8 * (s + j), static_cast<uint32_t>(round - 1) & 1u)) {
                            failed = true;
                            break;
                        }
                    }
                    if (failed) break;
                }
                for (int j = 0; j < n; ++j) {
                    const int tile = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
                    const uint32_t st = base + s * kStageBytes;
                    const uint32_t bar = bar_full + 8 * s;
                    const int x = c * kChunkCols, y = tile * kTileRows;
                    mbar_expect_tx(bar, kStageBytes);
                    tma_load_2d(st + 0 * kBoxBytes, &tm_v, x, y, bar);
                    tma_load_2d(st + 1 * kBoxBytes, &tm_r, x, y, bar);
                    tma_load_2d(st + 2 * kBoxBytes, &tm_d, x, y, bar);
                    tma_load_2d(st + 3 * kBoxBytes, &tm_w, x, y, bar);
                    if (--c < 0) {
                        c = nchunks - 1;
                        ++k;
                    }
                    if (++s == NST) {
                        s = 0;
                        ++round;
                    }
                }
            }
            if (failed) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
        }
    } else if (warp >= 2) {
        // ------------------------------- terms --------------------------------
        const int tt = (warp - 2) * 32 + lane;   // 0..127
        const int row = tt >> 2;                  // row of the tile
        const int g = tt & 3;                     // which 8 columns of the chunk
        const uint32_t rsw = static_cast<uint32_t>(row) & 7u;
        const uint32_t off0 = static_cast<uint32_t>(row) * 128u + (((2u * g) ^ rsw) << 4);
        const uint32_t off1 = static_cast<uint32_t>(row) * 128u + (((2u * g + 1u) ^ rsw) << 4);
        const uint32_t offn = static_cast<uint32_t>(row) * 128u + ((((2u * g + 2u) & 7u) ^ rsw) << 4);
        float first_v = 0.0f, first_r = 0.0f, first_d = 0.0f;   // column 0 of the previous (later) chunk
        int c = nchunks - 1, s = 0, b = 0;
        uint32_t sround = 0, bround = 0;
        for (int i = 0; i < total; ++i) {
            if (c == nchunks - 1) {   // tile start: nothing carries over
                first_v = 0.0f;
                first_r = 0.0f;
                first_d = 0.0f;
            }
            if (!mbar_wait_warp(bar_full + 8 * s, sround & 1u)) {
                failed = true;
                break;
            }
            if (bround > 0 && !mbar_wait_warp(bar_tfree + 8 * b, (bround - 1) & 1u)) {
                failed = true;
                break;
            }
            const uint32_t st = base + s * kStageBytes;
            float v[9], r[9], d[9], w[8];
            {
                const float4 a0 = lds128(st + 0 * kBoxBytes + off0), a1 = lds128(st + 0 * kBoxBytes + off1);
                v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
                const float4 b0 = lds128(st + 1 * kBoxBytes + off0), b1 = lds128(st + 1 * kBoxBytes + off1);
                r[0] = b0.x; r[1] = b0.y; r[2] = b0.z; r[3] = b0.w; r[4] = b1.x; r[5] = b1.y; r[6] = b1.z; r[7] = b1.w;
                const float4 c0 = lds128(st + 2 * kBoxBytes + off0), c1 = lds128(st + 2 * kBoxBytes + off1);
                d[0] = c0.x; d[1] = c0.y; d[2] = c0.z; d[3] = c0.w; d[4] = c1.x; d[5] = c1.y; d[6] = c1.z; d[7] = c1.w;
                const float4 e0 = lds128(st + 3 * kBoxBytes + off0), e1 = lds128(st + 3 * kBoxBytes + off1);
                w[0] = e0.x; w[1] = e0.y; w[2] = e0.z; w[3] = e0.w; w[4] = e1.x; w[5] = e1.y; w[6] = e1.z; w[7] = e1.w;
            }
            // column 8g+8: the next unit of the same row, or (g == 3) the carried column
            const float nv_s = lds32(st + 0 * kBoxBytes + offn);
            const float nr_s = lds32(st + 1 * kBoxBytes + offn);
            const float nd_s = lds32(st + 2 * kBoxBytes + offn);
            const float nv_c = __shfl_sync(0xffffffffu, first_v, (lane & ~3));
            const float nr_c = __shfl_sync(0xffffffffu, first_r, (lane & ~3));
            const float nd_c = __shfl_sync(0xffffffffu, first_d, (lane & ~3));
            v[8] = g == 3 ? nv_c : nv_s;
            r[8] = g == 3 ? nr_c : nr_s;
            d[8] = g == 3 ? nd_c : nd_s;
            first_v = v[0];
            first_r = r[0];
            first_d = d[0];
            const int col0 = c * kChunkCols + 8 * g;
            float dl[8], kk[8];
            uint32_t nonbin = 0u;
            if (col0 + 8 < horizon) {
                // all eight columns have a step: the f32x2 forms of the same IEEE operations,
                // two steps per instruction.  Steps (j, j+1) with odd j take their t+1
                // operands (j+1, j+2) from aligned register pairs of the 128-bit loads.
                const float2 neg1 = make_float2(-1.0f, -1.0f), one2 = make_float2(1.0f, 1.0f);
                const float2 gamma2 = make_float2(gamma, gamma), gl2 = make_float2(gl, gl);
#pragma unroll
                for (int j = 1; j < 7; j += 2) {
                    const float2 dn = make_float2(d[j + 1], d[j + 2]);
                    const float2 nn2 = __ffma2_rn(dn, neg1, one2);   // 1 - d: exact product, one rounding
                    const float2 t2 = __fadd2_rn(make_float2(r[j + 1], r[j + 2]),
                                                 __fmul2_rn(__fmul2_rn(gamma2, make_float2(v[j + 1], v[j + 2])), nn2));
                    const float2 td2 = make_float2(__fsub_rn(t2.x, v[j]), __fsub_rn(t2.y, v[j + 1]));
                    const float2 rho2 = make_float2(fminf(w[j], rho_clip), fminf(w[j + 1], rho_clip));
                    const float2 c2 = make_float2(fminf(w[j], c_clip), fminf(w[j + 1], c_clip));
                    const float2 d2 = __fmul2_rn(rho2, td2);
                    const float2 k2 = __fmul2_rn(__fmul2_rn(gl2, c2), nn2);
                    const float2 q2 = __fmul2_rn(dn, nn2);
                    nonbin |= __float_as_uint(q2.x) | __float_as_uint(q2.y);
                    dl[j] = d2.x;
                    dl[j + 1] = d2.y;
                    kk[j] = k2.x;
                    kk[j + 1] = k2.y;
                }
#pragma unroll
                for (int j = 0; j < 8; j += 7) {   // steps 0 and 7
                    float dj, gj, nj;
                    adv_terms(v[j], w[j], v[j + 1], r[j + 1], d[j + 1], gamma, gl, rho_clip, c_clip, dj, gj, nj);
                    dl[j] = dj;
                    kk[j] = __fmul_rn(gj, nj);
                    nonbin |= __float_as_uint(__fmul_rn(d[j + 1], nj));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool valid = col0 + j < horizon - 1;
                    float dj, gj, nj;
                    adv_terms(v[j], w[j], v[j + 1], r[j + 1], d[j + 1], gamma, gl, rho_clip, c_clip, dj, gj, nj);
                    dl[j] = valid ? dj : 0.0f;
                    kk[j] = valid ? __fmul_rn(gj, nj) : 0.0f;
                    nonbin |= valid ? __float_as_uint(__fmul_rn(d[j + 1], nj)) : 0u;
                }
            }
            const uint32_t tb = term_base + b * kTermBytes;
            sts128(tb + 0 * kBoxBytes + off0, make_float4(dl[0], dl[1], dl[2], dl[3]));
            sts128(tb + 0 * kBoxBytes + off1, make_float4(dl[4], dl[5], dl[6], dl[7]));
            sts128(tb + 1 * kBoxBytes + off0, make_float4(kk[0], kk[1], kk[2], kk[3]));
            sts128(tb + 1 * kBoxBytes + off1, make_float4(kk[4], kk[5], kk[6], kk[7]));
            if ((nonbin << 1) != 0u) sts32u(flag_base + 4 * b, 1u);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_tfull + 8 * b);
                mbar_arrive(bar_sfree + 8 * s);
            }
            if (--c < 0) c = nchunks - 1;
            if (++s == NST) {
                s = 0;
                ++sround;
            }
            if (++b == NT) {
                b = 0;
                ++bround;
            }
        }
        if (failed && lane == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    } else {
        // ------------------------------- chain --------------------------------
        if (lane == 0) prefetch_tensormap(&tm_a);
        const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
        const uint32_t sw = static_cast<uint32_t>(lane) & 7u;
        float a_run = 0.0f, abs_run = 0.0f, keep_last = 0.0f;
        int k = 0, c = nchunks - 1, b = 0, oslot = 0;
        uint32_t bround = 0;
        for (int i = 0; i < total; ++i) {
            const int tile = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
            if (c == nchunks - 1) {   // tile start
                const long long row = static_cast<long long>(tile) * kTileRows + lane;
                keep_last = (adv_in != nullptr && row < num_segments) ? adv_in[row * horizon + horizon - 1] : 0.0f;
                a_run = 0.0f;
                abs_run = 0.0f;
            }
            if (!mbar_wait_warp(bar_tfull + 8 * b, bround & 1u)) {
                failed = true;
                break;
            }
            const uint32_t tb = term_base + b * kTermBytes;
            float dl[32], kk[32], out[32];
#pragma unroll
            for (int u = 7; u >= 0; --u) {
                const uint32_t off = row_off + ((static_cast<uint32_t>(u) ^ sw) << 4);
                const float4 x = lds128(tb + 0 * kBoxBytes + off);
                const float4 y = lds128(tb + 1 * kBoxBytes + off);
                dl[4 * u] = x.x; dl[4 * u + 1] = x.y; dl[4 * u + 2] = x.z; dl[4 * u + 3] = x.w;
                kk[4 * u] = y.x; kk[4 * u + 1] = y.y; kk[4 * u + 2] = y.z; kk[4 * u + 3] = y.w;
            }
            const uint32_t flag = lds32u(flag_base + 4 * b);
            // the terms buffer is free as soon as every lane holds its values
            __syncwarp();
            if (lane == 0) {
                if (flag != 0u) sts32u(flag_base + 4 * b, 0u);
                mbar_arrive(bar_tfree + 8 * b);
            }
            const int cbase = c * kChunkCols;
            const float a_in = a_run;
            bool literal = flag != 0u;
            float abs_chunk = 0.0f;
            if (!literal) {
#pragma unroll
                for (int j = 31; j >= 0; --j) {
                    a_run = __fadd_rn(dl[j], __fmul_rn(kk[j], a_run));
                    out[j] = a_run;
                }
                abs_chunk = abs_tree32(out);
                literal = __any_sync(0xffffffffu, !(__fadd_rn(fabsf(a_in), abs_chunk) <= 1e30f));
            }
            if (literal) {   // rare: the reference's literal order, operands straight from global memory
                a_run = a_in;
                const long long row = static_cast<long long>(tile) * kTileRows + lane;
                const bool in_rows = row < num_segments;
                const long long ro = (in_rows ? row : 0) * horizon;
#pragma unroll
                for (int j = 31; j >= 0; --j) {
                    const int t = cbase + j;
                    if (in_rows && t < horizon - 1)
                        a_run = adv_step(__ldg(raw_v + ro + t), __ldg(raw_w + ro + t), __ldg(raw_v + ro + t + 1),
                                         __ldg(raw_r + ro + t + 1), __ldg(raw_d + ro + t + 1), a_run, gamma, gl,
                                         rho_clip, c_clip);
                    out[j] = a_run;
                }
                abs_chunk = abs_tree32(out);
            }
            if (EPI) abs_run = __fadd_rn(abs_run, abs_chunk);
            const uint32_t ob = out_base + oslot * kBoxBytes;
            if (lane == 0) bulk_wait_read<kWsOutSlots - 1>();   // the store that last used this box has read it
            __syncwarp();
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t off = row_off + ((static_cast<uint32_t>(u) ^ sw) << 4);
                float4 a4 = make_float4(out[4 * u], out[4 * u + 1], out[4 * u + 2], out[4 * u + 3]);
                if (cbase + 4 * u + 3 == horizon - 1) a4.w = keep_last;
                sts128(ob + off, a4);
            }
            if (EPI && c == 0) {
                const long long row = static_cast<long long>(tile) * kTileRows + lane;
                if (row < num_segments) seg_abs_sum[row] = abs_run;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(&tm_a, cbase, tile * kTileRows, ob);
                bulk_commit();
            }
            if (--c < 0) {
                c = nchunks - 1;
                ++k;
            }
            if (++b == NT) {
                b = 0;
                ++bround;
            }
            if (++oslot == kWsOutSlots) oslot = 0;
        }
        if (lane == 0) {
            // the stores only have to be done reading shared memory before the CTA exits;
            // their global writes complete with the grid
            bulk_wait_read<0>();
            if (failed) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
        }
    }
}

// ---------------------------------------------------------------------------
// bulk1d: serial, dense tiles of `tile_rows` whole rows fetched by 1-D bulk copies
// ---------------------------------------------------------------------------
// For H % 4 != 0 the row pitch is not a multiple of 16 bytes and no 2-D tensor
// map exists, but a tile of whole rows is one contiguous span per array;
// tile_rows is a multiple of 4, so every tile starts on a 16-byte boundary for
// any H.  (The last tile of a buffer may have a byte size that is not a
// multiple of 16: it is fetched with plain loads.)
//
// One CTA of four warps per tile, one stage of shared memory (v | r | d | w,
// dense, pitch H); several CTAs per SM overlap each other's phases:
//   1. thread 0 issues four cp.async.bulk copies, everybody waits on the mbarrier
//   2. terms, all 128 threads over the flat tile in units of four elements:
//      delta and k = (gamma*lambda*c)*nn of every step go to registers; after one
//      barrier (every raw operand has been read) they are written as interleaved
//      (delta, k) pairs over the d | w region
//   3. chain, warp 0: lane r walks row r with one 64-bit shared load per step,
//      A = delta + k*A, A written into the v region (stride H words: conflict-free
//      for odd H).  A non-binary nn or advantages near the overflow range send the
//      tile down the reference's literal order, operands straight from global memory
//   4. copy-out, all threads: coalesced 128-bit stores that skip column H-1
constexpr int kB1Threads = 128;
constexpr int kB1MaxUnits = 9;                                   // units of four elements per thread
constexpr int kB1MaxElems = kB1Threads * kB1MaxUnits * 4;         // elements per tile (72 KB of stage)

__global__ void __launch_bounds__(kB1Threads)
puff_adv_bulk1d_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                       const float* __restrict__ dones, const float* __restrict__ importance,
                       float* __restrict__ advantages, float* __restrict__ seg_abs_sum, float gamma,
                       float lambda, float rho_clip, float c_clip, long long num_segments,
                       int horizon, int tile_rows, long long num_tiles, int zero_last)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    float* const smem_f = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
    const int tid = threadIdx.x;
    const int tile_elems = tile_rows * horizon;
    const uint32_t arr_pitch = (static_cast<uint32_t>(tile_elems) * 4u + 15u) & ~15u;   // bytes, 16-byte aligned
    const uint32_t bar = base + 4u * arr_pitch;
    float* const sv = smem_f;
    float* const sr = sv + arr_pitch / 4;
    float* const sd = sr + arr_pitch / 4;
    float* const swt = sd + arr_pitch / 4;

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    const float gl = __fmul_rn(gamma, lambda);
    const float* const src[4] = {values, rewards, dones, importance};
    uint32_t parity = 0u;
    bool failed = false;

    for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const long long rem = num_segments - tile * tile_rows;
        const int rows = static_cast<int>(rem < tile_rows ? rem : tile_rows);
        const int n_el = rows * horizon;
        const uint32_t bytes = static_cast<uint32_t>(n_el) * 4u;
        const long long goff = tile * tile_elems;
        // ---- 1. fetch ----
        // bulk copies for the 16-byte multiple of the span (all of it, except in a last tile
        // whose row count makes the byte size ragged), plain loads for the up to three
        // trailing floats of each array
        {
            const uint32_t bulk_bytes = bytes & ~15u;
            if (bulk_bytes != 0u) {
                if (tid == 0) {
                    mbar_expect_tx(bar, 4u * bulk_bytes);
                    for (int a = 0; a < 4; ++a) bulk_load_1d(base + a * arr_pitch, src[a] + goff, bulk_bytes, bar);
                }
            }
            const int first_tail = static_cast<int>(bulk_bytes >> 2);
            if (tid < 4 * (n_el - first_tail)) {   // at most 12 threads
                const int a = tid / (n_el - first_tail), e = first_tail + tid % (n_el - first_tail);
                (smem_f + (a * arr_pitch) / 4)[e] = __ldg(src[a] + goff + e);
            }
            if (bulk_bytes != 0u) {
                if (!mbar_wait_thread(bar, parity)) failed = true;
                parity ^= 1u;
            }
            if (__syncthreads_or(failed)) {
                failed = true;
                break;
            }
        }
        // ---- 2. terms ----
        // a thread owns units of four consecutive elements (one 16-byte unit per array);
        // the operand at e+4 comes from the next unit
        uint32_t nonbin = 0u;
        const int n_grp = (n_el + 3) >> 2;
        const int grp_stride_cols = (4 * kB1Threads) % horizon;
        float4 dl4[kB1MaxUnits], kk4[kB1MaxUnits];
        {
            int col_g = (4 * tid) % horizon;   // column of the first element of this thread's next unit
#pragma unroll
            for (int u = 0; u < kB1MaxUnits; ++u) {
                const int grp = u * kB1Threads + tid;
                const int e = grp << 2;
                float dl[4] = {0.0f, 0.0f, 0.0f, 0.0f}, kk[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (grp < n_grp) {
                    // the arrays are padded to 16 bytes, so a unit that straddles n_el is readable
                    const float4 v4 = *reinterpret_cast<const float4*>(sv + e);
                    const float4 r4 = *reinterpret_cast<const float4*>(sr + e);
                    const float4 d4 = *reinterpret_cast<const float4*>(sd + e);
                    const float4 w4 = *reinterpret_cast<const float4*>(swt + e);
                    const bool more = e + 4 < n_el;
                    const float vn = more ? sv[e + 4] : 0.0f;
                    const float rn = more ? sr[e + 4] : 0.0f;
                    const float dn = more ? sd[e + 4] : 0.0f;
                    const float v[5] = {v4.x, v4.y, v4.z, v4.w, vn};
                    const float r[5] = {r4.x, r4.y, r4.z, r4.w, rn};
                    const float d[5] = {d4.x, d4.y, d4.z, d4.w, dn};
                    const float w[4] = {w4.x, w4.y, w4.z, w4.w};
                    int col = col_g;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool valid = (col < horizon - 1) && (e + j < n_el);   // then e+j+1 is in the same row
                        float dj, gj, nj;
                        adv_terms(v[j], w[j], v[j + 1], r[j + 1], d[j + 1], gamma, gl, rho_clip, c_clip, dj, gj, nj);
                        dl[j] = valid ? dj : 0.0f;
                        kk[j] = valid ? __fmul_rn(gj, nj) : 0.0f;
                        nonbin |= valid ? __float_as_uint(__fmul_rn(d[j + 1], nj)) : 0u;
                        col = col + 1 == horizon ? 0 : col + 1;
                    }
                }
                dl4[u] = make_float4(dl[0], dl[1], dl[2], dl[3]);
                kk4[u] = make_float4(kk[0], kk[1], kk[2], kk[3]);
                col_g += grp_stride_cols;
                if (col_g >= horizon) col_g -= horizon;
            }
        }
        __syncthreads();   // every raw operand of the tile has been read
        float2* const st = reinterpret_cast<float2*>(sd);   // (delta, k) pairs over the d | w region
#pragma unroll
        for (int u = 0; u < kB1MaxUnits; ++u) {
            const int grp = u * kB1Threads + tid;
            const int e = grp << 2;
            if (grp < n_grp) {
                *reinterpret_cast<float4*>(st + e) = make_float4(dl4[u].x, kk4[u].x, dl4[u].y, kk4[u].y);
                *reinterpret_cast<float4*>(st + e + 2) = make_float4(dl4[u].z, kk4[u].z, dl4[u].w, kk4[u].w);
            }
        }
        const bool any_nonbin = __syncthreads_or((nonbin << 1) != 0u);
        // ---- 3. chain ----
        if (tid < 32) {
            const int lane = tid;
            const int ro = lane * horizon;
            const bool mine = lane < rows;
            float a_run = 0.0f, abs_run = 0.0f;
            bool literal = any_nonbin;
            if (!literal) {
                if (mine) {
                    int t = horizon - 2;
                    for (; t >= 7; t -= 8) {   // eight steps' operands first, then the dependent part
                        float2 p8[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) p8[j] = st[ro + t - j];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            a_run = __fadd_rn(p8[j].x, __fmul_rn(p8[j].y, a_run));
                            sv[ro + t - j] = a_run;
                            abs_run = __fadd_rn(abs_run, fabsf(a_run));
                        }
                    }
                    for (; t >= 0; --t) {
                        const float2 pr = st[ro + t];
                        a_run = __fadd_rn(pr.x, __fmul_rn(pr.y, a_run));
                        sv[ro + t] = a_run;
                        abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    }
                }
                // the running sum of |A| bounds every |A| of the row
                literal = __any_sync(0xffffffffu, !(abs_run <= 1e30f));
            }
            if (literal) {   // rare: the reference's literal order, operands straight from global memory
                a_run = 0.0f;
                abs_run = 0.0f;
                if (mine) {
                    const long long gro = goff + ro;
                    for (int t = horizon - 2; t >= 0; --t) {
                        a_run = adv_step(__ldg(values + gro + t), __ldg(importance + gro + t), __ldg(values + gro + t + 1),
                                         __ldg(rewards + gro + t + 1), __ldg(dones + gro + t + 1), a_run, gamma, gl,
                                         rho_clip, c_clip);
                        sv[ro + t] = a_run;
                        abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    }
                }
            }
            if (mine && seg_abs_sum != nullptr) seg_abs_sum[tile * tile_rows + lane] = abs_run;
        }
        __syncthreads();
        // ---- 4. copy-out (advantages are in the v region), column H-1 of every row skipped ----
        {
            float* const g = advantages + goff;
            const int n4 = n_el >> 2;   // the tile starts on a 16-byte boundary
            int col = (4 * tid) % horizon;
            for (int e4 = tid; e4 < n4; e4 += kB1Threads) {
                const int e = e4 << 2;
                const float4 a4 = *reinterpret_cast<const float4*>(sv + e);
                if (col + 4 < horizon) {
                    *reinterpret_cast<float4*>(g + e) = a4;
                } else {
                    const float av[4] = {a4.x, a4.y, a4.z, a4.w};
                    int cj = col;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (cj != horizon - 1) g[e + j] = av[j];
                        else if (zero_last) g[e + j] = 0.0f;
                        cj = cj + 1 == horizon ? 0 : cj + 1;
                    }
                }
                col += grp_stride_cols;
                if (col >= horizon) col -= horizon;
            }
            for (int e = (n4 << 2) + tid; e < n_el; e += kB1Threads) {
                if (e % horizon != horizon - 1) g[e] = sv[e];
                else if (zero_last) g[e] = 0.0f;
            }
        }
        // the stage is refilled by the async proxy next
        fence_proxy_async();
        __syncthreads();
    }
    if (failed && tid == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
}

// ---------------------------------------------------------------------------
// bulk1d, warp-specialised: the odd-horizon counterpart of the tma2d pipeline
// ---------------------------------------------------------------------------
// The same split by dependency as puff_adv_tma2d_ws_kernel, on dense tiles of `tile_rows`
// whole rows (a contiguous span per array, see bulk1d above); eleven warps:
//   warp 0       producer: four cp.async.bulk copies per tile into a 2-deep ring of raw
//                stages (plus plain loads of the up to three ragged floats per array)
//   warps 3..10  terms: stream over the flat tile in units of four elements and write
//                (delta, k) pairs into one of two terms buffers; afterwards they copy the
//                finished advantages of the previous tile out to global memory with
//                coalesced 128-bit stores that skip column H-1
//   warps 1, 2   chain: warp b owns terms buffer b (every other tile); lane r walks row r
//                in place, A = delta + k*A stored over k; literal order from global memory
//                when a non-binary nn was flagged or the advantages near the overflow range
// One CTA per SM; tiles are pipelined inside it, so the kernel streams at buffer sizes
// where the one-stage bulk1d kernel is still phase-bound.
constexpr int kB1wStages = 2;
constexpr int kB1wTerms = 2;            // terms buffers = chain warps
constexpr int kB1wTermWarps = 8;
constexpr int kB1wTermThreads = 32 * kB1wTermWarps;
constexpr int kB1wThreads = 32 * (1 + kB1wTerms + kB1wTermWarps);

__global__ void __launch_bounds__(kB1wThreads)
puff_adv_bulk1d_ws_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                          const float* __restrict__ dones, const float* __restrict__ importance,
                          float* __restrict__ advantages, float* __restrict__ seg_abs_sum, float gamma,
                          float lambda, float rho_clip, float c_clip, long long num_segments,
                          int horizon, int tile_rows, long long num_tiles, int zero_last)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    uint8_t* const smem_al = smem_raw + (base - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tile_elems = tile_rows * horizon;
    const uint32_t arr_pitch = (static_cast<uint32_t>(tile_elems) * 4u + 15u) & ~15u;   // one raw array of a stage
    const uint32_t stage_bytes = 4u * arr_pitch;
    const uint32_t term_bytes = 2u * arr_pitch;                                          // (delta, k) pairs
    const uint32_t term_base = kB1wStages * stage_bytes;
    const uint32_t bar_off = term_base + kB1wTerms * term_bytes;
    const uint32_t bar_full = base + bar_off;
    const uint32_t bar_sfree = bar_full + 8 * kB1wStages;
    const uint32_t bar_tfull = bar_sfree + 8 * kB1wStages;
    const uint32_t bar_cdone = bar_tfull + 8 * kB1wTerms;
    const uint32_t flag_base = bar_cdone + 8 * kB1wTerms;

    const long long my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kB1wStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_sfree + 8 * s, kB1wTermWarps);
        }
        for (int b = 0; b < kB1wTerms; ++b) {
            mbar_init(bar_tfull + 8 * b, kB1wTermWarps);
            mbar_init(bar_cdone + 8 * b, 1);
            sts32u(flag_base + 4 * b, 0u);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    const float gl = __fmul_rn(gamma, lambda);
    bool failed = false;
    auto rows_of = [&](long long tile) {
        const long long rem = num_segments - tile * tile_rows;
        return static_cast<int>(rem < tile_rows ? rem : tile_rows);
    };

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const float* const src[4] = {values, rewards, dones, importance};
            for (long long n = 0; n < my_tiles; ++n) {
                const int s = static_cast<int>(n % kB1wStages);
                const uint32_t round = static_cast<uint32_t>(n / kB1wStages);
                if (round > 0 && !mbar_wait_thread(bar_sfree + 8 * s, (round - 1) & 1u)) {
                    failed = true;
                    break;
                }
                const long long tile = blockIdx.x + n * gridDim.x;
                const int n_el = rows_of(tile) * horizon;
                const long long goff = tile * tile_elems;
                const uint32_t bulk_bytes = (static_cast<uint32_t>(n_el) * 4u) & ~15u;
                float* const stage_f = reinterpret_cast<float*>(smem_al + s * stage_bytes);
                // ragged floats first: the arrive below publishes them together with the bulk bytes
                for (int e = static_cast<int>(bulk_bytes >> 2); e < n_el; ++e)
                    for (int a = 0; a < 4; ++a) (stage_f + a * (arr_pitch / 4))[e] = __ldg(src[a] + goff + e);
                const uint32_t bar = bar_full + 8 * s;
                if (bulk_bytes != 0u) {
                    mbar_expect_tx(bar, 4u * bulk_bytes);
                    for (int a = 0; a < 4; ++a)
                        bulk_load_1d(base + s * stage_bytes + a * arr_pitch, src[a] + goff, bulk_bytes, bar);
                } else {
                    mbar_arrive(bar);
                }
            }
            if (failed) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
        }
    } else if (warp > kB1wTerms) {
        // --------------------------- terms + copy-out --------------------------
        const int tt = (warp - 1 - kB1wTerms) * 32 + lane;   // 0 .. kB1wTermThreads-1
        const int unit_stride_cols = (4 * kB1wTermThreads) % horizon;
        auto copy_out = [&](long long n) {       // advantages of tile n sit in the .y of its pairs
            const int b = static_cast<int>(n % kB1wTerms);
            const long long tile = blockIdx.x + n * gridDim.x;
            const int n_el = rows_of(tile) * horizon;
            const float2* const tp = reinterpret_cast<const float2*>(smem_al + term_base + b * term_bytes);
            float* const g = advantages + tile * tile_elems;
            // unit by unit, the same units this thread fills in the terms pass: a thread only
            // ever overwrites pairs whose advantages it has itself written out
            const int n_grp = (n_el + 3) >> 2;
            int col = (4 * tt) % horizon;
            for (int e4 = tt; e4 < n_grp; e4 += kB1wTermThreads) {
                const int e = e4 << 2;
                const float4 p0 = *reinterpret_cast<const float4*>(tp + e);
                const float4 p1 = *reinterpret_cast<const float4*>(tp + e + 2);
                const float av[4] = {p0.y, p0.w, p1.y, p1.w};
                if (col + 4 < horizon && e + 4 <= n_el) {
                    *reinterpret_cast<float4*>(g + e) = make_float4(av[0], av[1], av[2], av[3]);
                } else {
                    int cj = col;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (e + j < n_el) {
                            if (cj != horizon - 1) g[e + j] = av[j];
                            else if (zero_last) g[e + j] = 0.0f;
                        }
                        cj = cj + 1 == horizon ? 0 : cj + 1;
                    }
                }
                col += unit_stride_cols;
                if (col >= horizon) col -= horizon;
            }
        };
        for (long long n = 0; n < my_tiles; ++n) {
            const int s = static_cast<int>(n % kB1wStages), b = static_cast<int>(n % kB1wTerms);
            if (!mbar_wait_warp(bar_full + 8 * s, static_cast<uint32_t>(n / kB1wStages) & 1u)) {
                failed = true;
                break;
            }
            const long long tile = blockIdx.x + n * gridDim.x;
            const int n_el = rows_of(tile) * horizon;
            const int n_grp = (n_el + 3) >> 2;
            const float* const sv = reinterpret_cast<const float*>(smem_al + s * stage_bytes);
            const float* const sr = sv + arr_pitch / 4;
            const float* const sd = sr + arr_pitch / 4;
            const float* const swt = sd + arr_pitch / 4;
            float2* const tp = reinterpret_cast<float2*>(smem_al + term_base + b * term_bytes);
            uint32_t nonbin = 0u;
            int col_g = (4 * tt) % horizon;
            for (int grp = tt; grp < n_grp; grp += kB1wTermThreads) {
                const int e = grp << 2;
                const float4 v4 = *reinterpret_cast<const float4*>(sv + e);
                const float4 r4 = *reinterpret_cast<const float4*>(sr + e);
                const float4 d4 = *reinterpret_cast<const float4*>(sd + e);
                const float4 w4 = *reinterpret_cast<const float4*>(swt + e);
                const bool more = e + 4 < n_el;
                const float v[5] = {v4.x, v4.y, v4.z, v4.w, more ? sv[e + 4] : 0.0f};
                const float r[5] = {r4.x, r4.y, r4.z, r4.w, more ? sr[e + 4] : 0.0f};
                const float d[5] = {d4.x, d4.y, d4.z, d4.w, more ? sd[e + 4] : 0.0f};
                const float w[4] = {w4.x, w4.y, w4.z, w4.w};
                float dl[4], kk[4];
                int col = col_g;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool valid = (col < horizon - 1) && (e + j < n_el);   // then e+j+1 is in the same row
                    float dj, gj, nj;
                    adv_terms(v[j], w[j], v[j + 1], r[j + 1], d[j + 1], gamma, gl, rho_clip, c_clip, dj, gj, nj);
                    dl[j] = valid ? dj : 0.0f;
                    kk[j] = valid ? __fmul_rn(gj, nj) : 0.0f;
                    nonbin |= valid ? __float_as_uint(__fmul_rn(d[j + 1], nj)) : 0u;
                    col = col + 1 == horizon ? 0 : col + 1;
                }
                *reinterpret_cast<float4*>(tp + e) = make_float4(dl[0], kk[0], dl[1], kk[1]);
                *reinterpret_cast<float4*>(tp + e + 2) = make_float4(dl[2], kk[2], dl[3], kk[3]);
                col_g += unit_stride_cols;
                if (col_g >= horizon) col_g -= horizon;
            }
            if ((nonbin << 1) != 0u) sts32u(flag_base + 4 * b, 1u);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_tfull + 8 * b);
                mbar_arrive(bar_sfree + 8 * s);
            }
            // the previous tile has been chained meanwhile: write it out
            if (n > 0) {
                const int pb = static_cast<int>((n - 1) % kB1wTerms);
                if (!mbar_wait_warp(bar_cdone + 8 * pb, static_cast<uint32_t>((n - 1) / kB1wTerms) & 1u)) {
                    failed = true;
                    break;
                }
                copy_out(n - 1);
            }
        }
        if (!failed && my_tiles > 0) {
            const long long n = my_tiles - 1;
            if (mbar_wait_warp(bar_cdone + 8 * static_cast<int>(n % kB1wTerms), static_cast<uint32_t>(n / kB1wTerms) & 1u))
                copy_out(n);
            else
                failed = true;
        }
        if (failed && lane == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    } else {
        // ------------------------------- chain --------------------------------
        for (long long n = warp - 1; n < my_tiles; n += kB1wTerms) {
            const int b = warp - 1;
            if (!mbar_wait_warp(bar_tfull + 8 * b, static_cast<uint32_t>(n / kB1wTerms) & 1u)) {
                failed = true;
                break;
            }
            const long long tile = blockIdx.x + n * gridDim.x;
            const int rows = rows_of(tile);
            float2* const tp = reinterpret_cast<float2*>(smem_al + term_base + b * term_bytes);
            const uint32_t flag = lds32u(flag_base + 4 * b);
            __syncwarp();
            if (lane == 0 && flag != 0u) sts32u(flag_base + 4 * b, 0u);
            const int ro = lane * horizon;
            const bool mine = lane < rows;
            float a_run = 0.0f, abs_run = 0.0f;
            bool literal = flag != 0u;
            if (!literal) {
                if (mine) {
                    int t = horizon - 2;
                    for (; t >= 7; t -= 8) {   // eight steps' operands first, then the dependent part
                        float2 p8[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) p8[j] = tp[ro + t - j];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            a_run = __fadd_rn(p8[j].x, __fmul_rn(p8[j].y, a_run));
                            tp[ro + t - j].y = a_run;
                            abs_run = __fadd_rn(abs_run, fabsf(a_run));
                        }
                    }
                    for (; t >= 0; --t) {
                        const float2 pr = tp[ro + t];
                        a_run = __fadd_rn(pr.x, __fmul_rn(pr.y, a_run));
                        tp[ro + t].y = a_run;
                        abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    }
                }
                literal = __any_sync(0xffffffffu, !(abs_run <= 1e30f));   // the sum bounds every |A| of the row
            }
            if (literal) {   // rare: the reference's literal order, operands straight from global memory
                a_run = 0.0f;
                abs_run = 0.0f;
                if (mine) {
                    const long long gro = tile * tile_elems + ro;
                    for (int t = horizon - 2; t >= 0; --t) {
                        a_run = adv_step(__ldg(values + gro + t), __ldg(importance + gro + t), __ldg(values + gro + t + 1),
                                         __ldg(rewards + gro + t + 1), __ldg(dones + gro + t + 1), a_run, gamma, gl,
                                         rho_clip, c_clip);
                        tp[ro + t].y = a_run;
                        abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    }
                }
            }
            if (mine && seg_abs_sum != nullptr) seg_abs_sum[tile * tile_rows + lane] = abs_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_cdone + 8 * b);
        }
        if (failed && lane == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    }
}

// ---------------------------------------------------------------------------
// scan: NT threads per row, 4 steps per thread, affine-pair scan of the carries
// ---------------------------------------------------------------------------
// A_t = delta_t + k_t * A_{t+1} with k_t = ((gamma*lambda)*c_t)*nn_t.  Thread j
// of a pass owns the unit of four columns G-1-j counted from the end of the
// row, so the suffix scan in time is an inclusive prefix scan over j.  The
// composed pair (K, D) of a unit maps the advantage entering it (column 4g+4)
// to the one leaving it (column 4g): A_out = D + K * A_in.  After the scan each
// thread knows its own A_in and replays its four steps in the reference's
// operation order, so only the carry-in differs from the serial result.
template <bool VEC>
__global__ void __launch_bounds__(1024)
puff_adv_scan_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                     const float* __restrict__ dones, const float* __restrict__ importance,
                     float* __restrict__ advantages, float* __restrict__ seg_abs_sum, float gamma,
                     float lambda, float rho_clip, float c_clip, long long num_segments, int horizon,
                     int zero_last)
{
    __shared__ float s_k[32], s_d[32], s_abs[32];
    __shared__ float s_carry;
    const int tid = threadIdx.x;
    const int nt = blockDim.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int nwarps = nt >> 5;
    const float gl = __fmul_rn(gamma, lambda);
    const int units = (horizon + 3) >> 2;          // units of 4 columns per row
    const int passes = (units + nt - 1) / nt;

    for (long long row = blockIdx.x; row < num_segments; row += gridDim.x) {
        const long long ro = row * horizon;
        const float* const v = values + ro;
        const float* const r = rewards + ro;
        const float* const d = dones + ro;
        const float* const w = importance + ro;
        float* const a = advantages + ro;
        float a_pass = 0.0f;      // advantage entering this pass (from later columns)
        float abs_acc = 0.0f;     // thread 0 only
        if (zero_last && tid == 0) a[horizon - 1] = 0.0f;

        for (int p = 0; p < passes; ++p) {
            const int j = p * nt + tid;
            const int g = units - 1 - j;
            const bool live = g >= 0;
            const int col0 = g << 2;
            float vv[5], rr[5], dd[5], ww[4];   // index i <-> column col0+i
#pragma unroll
            for (int i = 0; i < 5; ++i) {
                vv[i] = 0.0f;
                rr[i] = 0.0f;
                dd[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) ww[i] = 0.0f;
            if (live) {
                if (VEC) {   // horizon % 4 == 0 and 16-byte aligned bases
                    const float4 v4 = __ldg(reinterpret_cast<const float4*>(v + col0));
                    const float4 r4 = __ldg(reinterpret_cast<const float4*>(r + col0));
                    const float4 d4 = __ldg(reinterpret_cast<const float4*>(d + col0));
                    const float4 w4 = __ldg(reinterpret_cast<const float4*>(w + col0));
                    vv[0] = v4.x; vv[1] = v4.y; vv[2] = v4.z; vv[3] = v4.w;
                    rr[0] = r4.x; rr[1] = r4.y; rr[2] = r4.z; rr[3] = r4.w;
                    dd[0] = d4.x; dd[1] = d4.y; dd[2] = d4.z; dd[3] = d4.w;
                    ww[0] = w4.x; ww[1] = w4.y; ww[2] = w4.z; ww[3] = w4.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (col0 + i < horizon) {
                            vv[i] = __ldg(v + col0 + i);
                            rr[i] = __ldg(r + col0 + i);
                            dd[i] = __ldg(d + col0 + i);
                            ww[i] = __ldg(w + col0 + i);
                        }
                    }
                }
                if (col0 + 4 < horizon) {
                    vv[4] = __ldg(v + col0 + 4);
                    rr[4] = __ldg(r + col0 + 4);
                    dd[4] = __ldg(d + col0 + 4);
                }
            }
            // local composition over the (up to) four steps, latest column first
            float K = 1.0f, D = 0.0f;
            float dl[4], kk[4];
#pragma unroll
            for (int i = 3; i >= 0; --i) {
                const bool step = live && (col0 + i + 1 < horizon);   // t <= H-2
                const float nn = __fsub_rn(1.0f, dd[i + 1]);
                const float rho = fminf(ww[i], rho_clip);
                const float c = fminf(ww[i], c_clip);
                const float td = __fsub_rn(__fadd_rn(rr[i + 1], __fmul_rn(__fmul_rn(gamma, vv[i + 1]), nn)), vv[i]);
                dl[i] = step ? __fmul_rn(rho, td) : 0.0f;
                kk[i] = step ? __fmul_rn(__fmul_rn(gl, c), nn) : 1.0f;
                D = fmaf(kk[i], D, dl[i]);
                K = kk[i] * K;
            }
            // inclusive prefix scan over j inside the warp
            float Ki = K, Di = D;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float Kp = __shfl_up_sync(0xffffffffu, Ki, o);
                const float Dp = __shfl_up_sync(0xffffffffu, Di, o);
                if (lane >= o) {
                    Di = fmaf(Ki, Dp, Di);
                    Ki = Ki * Kp;
                }
            }
            // exclusive prefix inside the warp
            float Ke = __shfl_up_sync(0xffffffffu, Ki, 1);
            float De = __shfl_up_sync(0xffffffffu, Di, 1);
            if (lane == 0) {
                Ke = 1.0f;
                De = 0.0f;
            }
            float a_in;
            if (nwarps > 1) {
                if (lane == 31) {
                    s_k[warp] = Ki;
                    s_d[warp] = Di;
                }
                __syncthreads();
                if (warp == 0) {
                    float Kw = lane < nwarps ? s_k[lane] : 1.0f;
                    float Dw = lane < nwarps ? s_d[lane] : 0.0f;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const float Kp = __shfl_up_sync(0xffffffffu, Kw, o);
                        const float Dp = __shfl_up_sync(0xffffffffu, Dw, o);
                        if (lane >= o) {
                            Dw = fmaf(Kw, Dp, Dw);
                            Kw = Kw * Kp;
                        }
                    }
                    // A leaving warp `lane` = Dw + Kw * a_pass: store it, the next warp enters with it
                    s_d[lane] = fmaf(Kw, a_pass, Dw);
                }
                __syncthreads();
                const float a_warp_in = warp == 0 ? a_pass : s_d[warp - 1];
                a_in = fmaf(Ke, a_warp_in, De);
                if (tid == 0) s_carry = s_d[nwarps - 1];
            } else {
                a_in = fmaf(Ke, a_pass, De);
                const float a_out = fmaf(Ki, a_pass, Di);
                if (tid == 31) s_carry = a_out;
            }
            // replay in the reference's operation order
            float a_run = a_in, abs_loc = 0.0f;
            float out[4];
#pragma unroll
            for (int i = 3; i >= 0; --i) {
                const bool step = live && (col0 + i + 1 < horizon);
                if (step) {
                    a_run = adv_step(vv[i], ww[i], vv[i + 1], rr[i + 1], dd[i + 1], a_run, gamma, gl,
                                     rho_clip, c_clip);
                    abs_loc += fabsf(a_run);
                }
                out[i] = a_run;
            }
            if (live) {
                if (VEC && col0 + 4 < horizon) {
                    *reinterpret_cast<float4*>(a + col0) = make_float4(out[0], out[1], out[2], out[3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (col0 + i + 1 < horizon) a[col0 + i] = out[i];
                }
            }
            if (seg_abs_sum != nullptr) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) abs_loc += __shfl_xor_sync(0xffffffffu, abs_loc, o);
                if (lane == 0) s_abs[warp] = abs_loc;
            }
            __syncthreads();   // s_carry, s_abs visible; s_k / s_d reusable
            a_pass = s_carry;
            if (seg_abs_sum != nullptr && tid == 0)
                for (int i = 0; i < nwarps; ++i) abs_acc += s_abs[i];
            __syncthreads();
        }
        if (seg_abs_sum != nullptr && tid == 0) seg_abs_sum[row] = abs_acc;
    }
}

// ---------------------------------------------------------------------------
// generic: serial, one thread per row, plain global loads
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
puff_adv_generic_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                        const float* __restrict__ dones, const float* __restrict__ importance,
                        float* __restrict__ advantages, float* __restrict__ seg_abs_sum, float gamma,
                        float lambda, float rho_clip, float c_clip, long long num_segments,
                        long long horizon, int zero_last)
{
    const float gl = __fmul_rn(gamma, lambda);
    for (long long row = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
         row < num_segments; row += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long ro = row * horizon;
        float a_run = 0.0f, abs_run = 0.0f;
        float v_n = __ldg(values + ro + horizon - 1);
        for (long long t = horizon - 2; t >= 0; --t) {
            const float v_t = __ldg(values + ro + t);
            a_run = adv_step(v_t, __ldg(importance + ro + t), v_n, __ldg(rewards + ro + t + 1),
                             __ldg(dones + ro + t + 1), a_run, gamma, gl, rho_clip, c_clip);
            abs_run = __fadd_rn(abs_run, fabsf(a_run));
            advantages[ro + t] = a_run;
            v_n = v_t;
        }
        if (zero_last) advantages[ro + horizon - 1] = 0.0f;
        if (seg_abs_sum != nullptr) seg_abs_sum[row] = abs_run;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    int max_smem_optin = 0;
    cudaError_t err = cudaSuccess;
    bool ready = false;
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
    if (!d.ready) {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!d.ready) {
            cudaError_t e1 = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
            cudaError_t e2 = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
            cudaError_t e3 = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
            d.err = e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3);
            if (d.err == cudaSuccess) {
                // opt in to large dynamic shared memory once per device
                set_tma2d_attrs<2>();
                set_tma2d_attrs<3>();
                set_tma2d_attrs<4>();
                set_tma2d_ws_attrs<2, 2>();
                set_tma2d_ws_attrs<3, 2>();
                set_tma2d_ws_attrs<4, 2>();
                set_tma2d_ws_attrs<6, 2>();
                cudaFuncSetAttribute(puff_adv_bulk1d_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, d.max_smem_optin);
                cudaFuncSetAttribute(puff_adv_bulk1d_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, d.max_smem_optin);
                d.err = cudaGetLastError();
            }
            d.ready = (d.err == cudaSuccess);
        }
    }
    if (d.err != cudaSuccess) {
        *code = static_cast<int>(d.err);
        return nullptr;
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
    long long rows = -1, horizon = -1;
    CUtensorMap tm[5];
};

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
                                                           "PUFF_ADV_SCAN_THREADS"};
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

template <int NST>
static cudaError_t launch_tma2d(const MapSet& m, const float* adv_in, float* seg_abs_sum, float gamma, float lambda, float rho_clip,
                                float c_clip, long long rows, int horizon, int grid, int tiles, cudaStream_t st)
{
    if (seg_abs_sum != nullptr)
        puff_adv_tma2d_kernel<NST, true><<<grid, 32, tma2d_smem_bytes<NST>(), st>>>(
            m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], adv_in, seg_abs_sum, gamma, lambda, rho_clip, c_clip,
            rows, horizon, tiles);
    else
        puff_adv_tma2d_kernel<NST, false><<<grid, 32, tma2d_smem_bytes<NST>(), st>>>(
            m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], adv_in, nullptr, gamma, lambda, rho_clip, c_clip,
            rows, horizon, tiles);
    return cudaGetLastError();
}

template <int NST, int NT>
static cudaError_t launch_tma2d_ws(const MapSet& m, const float* adv_in, float* seg_abs_sum, float gamma, float lambda, float rho_clip,
                                   float c_clip, long long rows, int horizon, int grid, int tiles, cudaStream_t st)
{
    int group = tune(PUFF_TUNE_LOAD_GROUP, NST % 2 == 0 ? 2 : 1);
    if (group < 1 || NST % group != 0) group = 1;
    if (seg_abs_sum != nullptr)
        puff_adv_tma2d_ws_kernel<NST, NT, true><<<grid, kWsThreads, tma2d_ws_smem_bytes<NST, NT>(), st>>>(
            m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], m.ptr[0], m.ptr[1], m.ptr[2], m.ptr[3], adv_in, seg_abs_sum, gamma, lambda, rho_clip, c_clip,
            rows, horizon, tiles, group);
    else
        puff_adv_tma2d_ws_kernel<NST, NT, false><<<grid, kWsThreads, tma2d_ws_smem_bytes<NST, NT>(), st>>>(
            m.tm[0], m.tm[1], m.tm[2], m.tm[3], m.tm[4], m.ptr[0], m.ptr[1], m.ptr[2], m.ptr[3], adv_in, nullptr, gamma, lambda, rho_clip, c_clip,
            rows, horizon, tiles, group);
    return cudaGetLastError();
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
    for (int i = 0; i < 4; ++i) {
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

// Warp-specialised bulk1d: two raw stages and two terms buffers, 48 bytes of shared memory
// per element of a tile; the largest of 32/16/8/4 rows that fits, 0 if none does
static int bulk1d_ws_tile_rows(long long horizon, int max_smem, size_t* smem_bytes)
{
    const int cand[4] = {32, 16, 8, 4};
    for (int i = 0; i < 4; ++i) {
        const size_t arr = (static_cast<size_t>(cand[i]) * horizon * 4 + 15) & ~static_cast<size_t>(15);
        const size_t need = (kB1wStages * 4 + kB1wTerms * 2) * arr + 8 * (2 * kB1wStages + 2 * kB1wTerms) + 4 * kB1wTerms + 64 + 128;
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

extern "C" int puff_advantage_sm100_launch_ex(const float* values, const float* rewards, const float* dones,
                                              const float* importance, float* advantages, float* seg_abs_sum,
                                              float gamma, float lambda, float rho_clip, float c_clip,
                                              long long num_segments, long long horizon, int variant,
                                              unsigned flags, void* cuda_stream)
{
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
        // long rows with too few segments to give every SM a few rows: scan
        const bool few_rows = num_segments < static_cast<long long>(dev->sm_count) * 24;
        if (variant == PUFF_VARIANT_AUTO && can_scan && few_rows && horizon >= 512)
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
        static thread_local MapSet cache;
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
            bool hit = cache.rows == rows && cache.horizon == horizon;
            for (int i = 0; i < 5 && hit; ++i) hit = cache.ptr[i] == p[i];
            if (!hit) {
                cache.rows = -1;
                for (int i = 0; i < 5; ++i)
                    if (!make_map(&cache.tm[i], p[i], rows, horizon, horizon)) return PUFF_ERR_DRIVER;
                for (int i = 0; i < 5; ++i) cache.ptr[i] = p[i];
                cache.rows = rows;
                cache.horizon = horizon;
            }
            const long long tiles = (rows + kTileRows - 1) / kTileRows;
            float* abs_p = seg_abs_sum != nullptr ? seg_abs_sum + r0 : nullptr;
            // Large buffers: the warp-specialised kernel.  Measured on 131072 x 256: four raw
            // stages whose loads are issued two chunks at a time, two terms buffers, two CTAs
            // per SM (more CTAs per SM lowered the achieved DRAM rate).  Buffers of only a few
            // chunks per SM (8192 x 64 and smaller) finish sooner on the single-warp kernel,
            // whose pipeline has fewer hops.
            // PUFF_TUNE_WS_STAGES: 0 = single-warp, N = warp-specialised with N raw stages (2, 3, 4, 6).
            const long long work_items = tiles * ((horizon + kChunkCols - 1) / kChunkCols);
            const int ws = tune(PUFF_TUNE_WS_STAGES, work_items >= 8LL * dev->sm_count ? 4 : 0);
            if (ws != 0) {
                const int wnst = ws <= 2 ? 2 : ws == 3 ? 3 : ws <= 5 ? 4 : 6;
                const int smem = wnst * kStageBytes + 2 * kTermBytes + kWsOutSlots * kBoxBytes + 2048;
                int per_sm = (dev->max_smem_optin + 1024) / (smem + 1024);
                if (per_sm > 2) per_sm = 2;
                { const int o = tune(PUFF_TUNE_CTAS_PER_SM, 0); if (o > 0) per_sm = o < 3 ? o : 3; }
                if (per_sm < 1) per_sm = 1;
                const long long mg = static_cast<long long>(dev->sm_count) * per_sm;
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
        // measured at H = 127: the pipeline wins from a few thousand tiles on (131072 rows:
        // 66 us against 72 us); at 10007 rows the one-stage kernel is ahead (10.6 against 12.5 us)
        const long long ws_tiles = ws_rows > 0 ? (num_segments + ws_rows - 1) / ws_rows : 0;
        const int use_ws = ws_rows > 0 ? tune(PUFF_TUNE_WS_STAGES, ws_tiles >= 8LL * dev->sm_count ? 1 : 0) : 0;
        if (use_ws != 0) {
            const long long tiles = (num_segments + ws_rows - 1) / ws_rows;
            const long long max_grid = dev->sm_count;
            const int grid = static_cast<int>(tiles < max_grid ? tiles : max_grid);
            puff_adv_bulk1d_ws_kernel<<<grid, kB1wThreads, ws_smem, st>>>(values, rewards, dones, importance, advantages,
                                                                         seg_abs_sum, gamma, lambda, rho_clip, c_clip,
                                                                         num_segments, static_cast<int>(horizon), ws_rows,
                                                                         tiles, zero_last);
        } else {
        const long long tiles = (num_segments + bulk_rows - 1) / bulk_rows;
        int per_sm = static_cast<int>(static_cast<size_t>(dev->max_smem_optin + 1024) / (bulk_smem + 1024));
        per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
        const long long max_grid = static_cast<long long>(dev->sm_count) * per_sm;
        const int grid = static_cast<int>(tiles < max_grid ? tiles : max_grid);
        puff_adv_bulk1d_kernel<<<grid, kB1Threads, bulk_smem, st>>>(values, rewards, dones, importance, advantages,
                                                                    seg_abs_sum, gamma, lambda, rho_clip, c_clip,
                                                                    num_segments, static_cast<int>(horizon), bulk_rows, tiles, zero_last);
        }
        err = cudaGetLastError();
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
    } else if (kernel == PUFF_KERNEL_SCAN) {
        const long long units = (horizon + 3) / 4;
        // 512 threads at most: with ~60 registers per thread two such CTAs share an SM,
        // so 256 rows of 4096 columns run as one wave (measured 7.4 us against 9.1 us with 1024)
        int nt = 32;
        while (nt < 512 && nt < units) nt <<= 1;
        {
            const int o = tune(PUFF_TUNE_SCAN_THREADS, 0);
            if (o >= 32 && o <= 1024 && (o & (o - 1)) == 0) nt = o;
        }
        const long long max_grid = static_cast<long long>(dev->sm_count) * (2048 / nt) ;
        const int grid = static_cast<int>(num_segments < max_grid ? num_segments : max_grid);
        if (aligned16 && horizon % 4 == 0)
            puff_adv_scan_kernel<true><<<grid, nt, 0, st>>>(values, rewards, dones, importance, advantages, seg_abs_sum,
                                                            gamma, lambda, rho_clip, c_clip, num_segments, static_cast<int>(horizon), zero_last);
        else
            puff_adv_scan_kernel<false><<<grid, nt, 0, st>>>(values, rewards, dones, importance, advantages, seg_abs_sum,
                                                             gamma, lambda, rho_clip, c_clip, num_segments, static_cast<int>(horizon), zero_last);
        err = cudaGetLastError();
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
    } else {
        const long long blocks = (num_segments + 127) / 128;
        const long long max_grid = static_cast<long long>(dev->sm_count) * 16;
        const int grid = static_cast<int>(blocks < max_grid ? blocks : max_grid);
        puff_adv_generic_kernel<<<grid, 128, 0, st>>>(values, rewards, dones, importance, advantages, seg_abs_sum,
                                                      gamma, lambda, rho_clip, c_clip, num_segments, horizon, zero_last);
        err = cudaGetLastError();
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
}

extern "C" int puff_advantage_sm100_device_status(void)
{
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    int h = 0;
    e = cudaMemcpyFromSymbol(&h, g_device_status, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (h != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    }
    return h;
}

extern "C" int puff_advantage_sm100_set_tuning(int knob, int value)
{
    if (knob < 0 || knob >= PUFF_TUNE_COUNT) return PUFF_ERR_VARIANT;
    tune_init();
    return g_tune[knob].exchange(value < 0 ? -1 : value, std::memory_order_relaxed);
}

extern "C" const char* puff_advantage_sm100_version(void) { return "0.1"; }
