// Device-side building blocks shared by the advantage kernels (sm_100a): constants of
// the tiling, the recurrence step in the reference's operation order, PTX wrappers for
// mbarriers / TMA / bulk copies, and the per-chunk routines of the TMA-tiled kernels.
// Included by puff_advantage_sm100.cu only (it defines a __device__ variable).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/puff_advantage.h"
#include "puff_launch.cuh"

namespace puff {

// Device-side status word: PUFF_ERR_DEVICE_WAIT when a bounded wait gave up.
__device__ int g_device_status = 0;

// Optional per-CTA timeline (compile with -DPUFF_TIMELINE): clock64 stamps at the phase boundaries
// of the small-buffer kernels, read back with puff_advantage_sm100_timeline().  Stamp 0 (CTA start)
// and stamp 10 (CTA end) also record %globaltimer, in slots 12 and 14, so that the host can turn
// cycles into nanoseconds on a time line common to all CTAs.  A stamp is a one-lane branch: the warp
// may stay split behind it, and a split warp was measured to run a dependent chain at 37-40 cycles
// a step instead of 19, so latency-critical code behind a stamp starts with __syncwarp().
// Compiled out of release builds.
#ifdef PUFF_TIMELINE
constexpr int kTimelineSlots = 16;
constexpr int kTimelineCtas = 2048;
__device__ unsigned long long g_timeline[kTimelineCtas * kTimelineSlots];
#define PUFF_STAMP(slot)                                                                         \
    do {                                                                                         \
        if ((threadIdx.x & 31) == 0 && blockIdx.x < kTimelineCtas) {                             \
            if ((slot) == 0 || (slot) == 10) {                                                   \
                unsigned long long t_;                                                           \
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                           \
                g_timeline[blockIdx.x * kTimelineSlots + 12 + ((slot) == 10 ? 2 : 0)] = t_;      \
            }                                                                                    \
            g_timeline[blockIdx.x * kTimelineSlots + (slot)] = static_cast<unsigned long long>(clock64()); \
        }                                                                                        \
    } while (0)
// cycle accounting of a warp's loop phases: PUFF_TICK(acc) adds the cycles since the previous
// tick to acc; PUFF_PUT(slot, acc) stores a total
#define PUFF_TICK_DECL long long tick_prev_ = clock64()
#define PUFF_TICK(acc)                          \
    do {                                        \
        const long long now_ = clock64();       \
        (acc) += now_ - tick_prev_;             \
        tick_prev_ = now_;                      \
    } while (0)
#define PUFF_PUT(slot, acc)                                                                                       \
    do {                                                                                                          \
        if ((threadIdx.x & 31) == 0 && blockIdx.x < kTimelineCtas)                                                \
            g_timeline[blockIdx.x * kTimelineSlots + (slot)] = static_cast<unsigned long long>(acc);             \
    } while (0)
#else
#define PUFF_STAMP(slot) do { } while (0)
#define PUFF_TICK_DECL do { } while (0)
#define PUFF_TICK(acc) do { } while (0)
#define PUFF_PUT(slot, acc) do { } while (0)
#endif

// Index checks of debug builds (compile with -DPUFF_DEBUG_BOUNDS): every global-memory index a
// kernel forms is compared with the extent of its array.  A bad index records
// PUFF_ERR_DEVICE_BOUNDS in the status word and the access is skipped (loads yield 0); nothing
// traps.  Release builds compile the checks out.
#ifdef PUFF_DEBUG_BOUNDS
__device__ __forceinline__ bool idx_ok(long long i, long long n)
{
    if (i >= 0 && i < n) return true;
    atomicExch(&g_device_status, PUFF_ERR_DEVICE_BOUNDS);
    return false;
}
#else
__device__ __forceinline__ constexpr bool idx_ok(long long, long long) { return true; }
#endif
__device__ __forceinline__ float ldg_chk(const float* base, long long i, long long n)
{
    return idx_ok(i, n) ? __ldg(base + i) : 0.0f;
}
// plain (coherent) load: for memory the same kernel also writes
__device__ __forceinline__ float ld_chk(const float* base, long long i, long long n)
{
    return idx_ok(i, n) ? base[i] : 0.0f;
}
__device__ __forceinline__ float4 ldg4_chk(const float* base, long long i, long long n)
{
    return (idx_ok(i, n) && idx_ok(i + 3, n)) ? __ldg(reinterpret_cast<const float4*>(base + i))
                                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}
__device__ __forceinline__ void stg_chk(float* base, long long i, long long n, float v)
{
    if (idx_ok(i, n)) base[i] = v;
}
__device__ __forceinline__ void stg4_chk(float* base, long long i, long long n, float4 v)
{
    if (idx_ok(i, n) && idx_ok(i + 3, n)) *reinterpret_cast<float4*>(base + i) = v;
}
// a TMA box may hang over the tensor's edge (it is clipped or zero-filled there), but its
// origin must lie inside [0, width) x [0, rows)
__device__ __forceinline__ bool box_ok(int x, int y, int width, long long rows)
{
    return idx_ok(x, width) && idx_ok(y, rows);
}

constexpr int kTileRows = 32;              // segments per warp tile
constexpr int kChunkCols = 32;             // columns per TMA box (128 bytes)
constexpr int kBoxBytes = kTileRows * kChunkCols * 4;   // 4096
constexpr int kStageBytes = 4 * kBoxBytes;              // v, r, d, w
// The serial kernels run the chain as A = delta + k*A with k = ((gamma*lambda)*c)*nn, while the
// reference evaluates (((gamma*lambda)*c)*A)*nn.  For nn in {0, 1} the two agree bit for bit unless
// the inner product ((gamma*lambda)*c)*A overflows while nn == 0 (the reference then yields
// inf*0 = NaN, the packed form 0).  A chunk therefore stays on the packed form only while every
// |(gamma*lambda)*c| <= kPackedMaxGain and every |A| <= kPackedMaxAdv, whose product is below
// FLT_MAX; anything else is recomputed in the reference's literal order.
constexpr float kPackedMaxGain = 1e8f;
constexpr float kPackedMaxAdv = 1e30f;
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
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
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


// single-thread wait, plain arrive and 32-bit shared accesses (warp-specialised kernels)
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

// Shared-memory accesses of the chain loops.  No "memory" clobber: the compiler may move them
// across ordinary arithmetic and across each other's neighbours, which is what lets the loads of
// the next batch of steps issue under the dependent multiply-adds of the current one.  They stay
// ordered among themselves and against every barrier, fence and mbarrier operation (all volatile
// asm), and a store of A[t] can never pass the load of step t's operands: it needs their value.
__device__ __forceinline__ float2 lds64_chain(uint32_t addr)
{
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32_chain(uint32_t addr, float v)
{
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v));
}

// One row's recurrence A = delta + k*A over steps t = n_steps-1 .. 0 out of (delta, k) pairs in
// shared memory: pair t at pairs + 8*t, A[t] stored to out + out_stride*t (out_stride 4: a dense
// float row; 8 with out = pairs + 4: over the k of its own pair).  Batches of eight steps, the
// next batch's pairs loaded before the current batch's dependent chain runs.
__device__ __forceinline__ void chain_pairs_row(uint32_t pairs, uint32_t out, uint32_t out_stride, int n_steps,
                                                float& a_run, float& abs_run)
{
    int t = n_steps - 1;
    float2 cur[8];
    if (t >= 7) {
#pragma unroll
        for (int j = 0; j < 8; ++j) cur[j] = lds64_chain(pairs + 8u * static_cast<uint32_t>(t - j));
    }
    while (t >= 7) {
        float2 nxt[8];
        const bool more = t - 8 >= 7;
        if (more) {
#pragma unroll
            for (int j = 0; j < 8; ++j) nxt[j] = lds64_chain(pairs + 8u * static_cast<uint32_t>(t - 8 - j));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            a_run = __fadd_rn(cur[j].x, __fmul_rn(cur[j].y, a_run));
            sts32_chain(out + out_stride * static_cast<uint32_t>(t - j), a_run);
            abs_run = __fadd_rn(abs_run, fabsf(a_run));
        }
        if (more) {
#pragma unroll
            for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
        }
        t -= 8;
    }
    for (; t >= 0; --t) {
        const float2 pr = lds64_chain(pairs + 8u * static_cast<uint32_t>(t));
        a_run = __fadd_rn(pr.x, __fmul_rn(pr.y, a_run));
        sts32_chain(out + out_stride * static_cast<uint32_t>(t), a_run);
        abs_run = __fadd_rn(abs_run, fabsf(a_run));
    }
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
// (nn is not exactly 0 or 1), a gain (gamma*lambda)*c beyond kPackedMaxGain, or advantages
// beyond kPackedMaxAdv.
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
    float gain = 0.0f;   // largest |(gamma*lambda)*c| of the chunk (a NaN shows up in A instead)
    const float a_in = a_run;
    // step 31 alone (its t+1 operands are the carried ones); masked at the end of a row
    {
        float d, g, n;
        adv_terms(vc[31], wc[31], vc[32], rc[32], dc[32], gamma, gl, rho_clip, c_clip, d, g, n);
        gain = fmaxf(gain, fabsf(g));
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
        const float2 g2 = __fmul2_rn(gl2, c2);
        const float2 k2 = __fmul2_rn(g2, nn2);
        const float2 q2 = __fmul2_rn(dn, nn2);
        gain = fmaxf(gain, fmaxf(fabsf(g2.x), fabsf(g2.y)));
        nonbin |= __float_as_uint(q2.x) | __float_as_uint(q2.y);
        dl[j] = d2.x;
        dl[j + 1] = d2.y;
        kk[j] = k2.x;
        kk[j + 1] = k2.y;
    }
    {
        float d, g, n;
        adv_terms(vc[0], wc[0], vc[1], rc[1], dc[1], gamma, gl, rho_clip, c_clip, d, g, n);
        gain = fmaxf(gain, fabsf(g));
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
    const bool ok = ((nonbin << 1) == 0u) && (big <= kPackedMaxAdv) && (gain <= kPackedMaxGain);
    return __all_sync(0xffffffffu, ok);
}

}  // namespace puff
