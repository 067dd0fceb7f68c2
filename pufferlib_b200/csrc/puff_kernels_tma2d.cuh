// TMA-tiled serial advantage kernels for H % 4 == 0: single-warp and warp-specialised forms.
// Included by puff_advantage_sm100.cu after puff_device.cuh.
#pragma once
#include "puff_device.cuh"

namespace puff {

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
    PUFF_STAMP(0);   // CTA start
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
        for (int s = 0; s < NST; ++s) mbar_init(bar_base + 8 * s, 1);
        fence_mbar_init();
        fence_proxy_async();
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_r);
        prefetch_tensormap(&tm_d);
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_a);
    }
    __syncwarp();
    PUFF_STAMP(1);   // set-up done
    pdl_wait();   // nothing above reads or writes a tensor
    PUFF_STAMP(2);   // predecessor complete

    // work item -> (tile k of this CTA, chunk c); chunks of a tile run from the last column
    // block down.  The issuing lane keeps its own running (k, c, stage) of the next item to
    // load, so that nothing but the TMA instructions stands between launch and first bytes.
    // (Spreading the boxes of an item over four lanes, or the first ring-full of items over as
    // many lanes, was measured: slower and no faster respectively.)
    int ld_k = 0, ld_c = nchunks - 1, ld_s = 0, ld_i = 0;
    auto issue_next = [&]() {
        const int tile = static_cast<int>(blockIdx.x) + ld_k * static_cast<int>(gridDim.x);
        const uint32_t st = base + ld_s * kStageBytes;
        const uint32_t bar = bar_base + 8 * ld_s;
        int x = ld_c * kChunkCols;
        int y = tile * kTileRows;
        if (!box_ok(x, y, horizon, num_segments)) x = y = 0;   // debug builds: recorded, and a valid box is read instead
        mbar_expect_tx(bar, kStageBytes);
        tma_load_2d(st + 0 * kBoxBytes, &tm_v, x, y, bar);
        tma_load_2d(st + 1 * kBoxBytes, &tm_r, x, y, bar);
        tma_load_2d(st + 2 * kBoxBytes, &tm_d, x, y, bar);
        tma_load_2d(st + 3 * kBoxBytes, &tm_w, x, y, bar);
        if (--ld_c < 0) {
            ld_c = nchunks - 1;
            ++ld_k;
        }
        if (++ld_s == NST) ld_s = 0;
        ++ld_i;
    };

    if (lane == 0) {
        const int pre = total < NST ? total : NST;
        for (int i = 0; i < pre; ++i) issue_next();
    }
    pdl_launch_dependents();
    PUFF_STAMP(3);   // first loads issued

    const float gl = __fmul_rn(gamma, lambda);
    const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
    const uint32_t sw = static_cast<uint32_t>(lane) & 7u;

    float a_run = 0.0f, abs_run = 0.0f;
    float nv = 0.0f, nr = 0.0f, nd = 0.0f;   // values/rewards/dones at column t+1 across units
    float keep_last = 0.0f;                  // the caller's advantages[row, H-1]
    float keep_next = 0.0f;                  // the same for the next tile, fetched one tile ahead
    if (adv_in != nullptr && my_tiles > 0) {
        const long long row = static_cast<long long>(blockIdx.x) * kTileRows + lane;
        if (row < num_segments) keep_next = ld_chk(adv_in, row * horizon + horizon - 1, num_segments * horizon);
    }
    int k = 0, c = nchunks - 1, s = 0;
    uint32_t parity = 0;
    bool failed = false;

    for (int i = 0; i < total; ++i) {
        if (c == nchunks - 1) {   // new tile
            keep_last = keep_next;
            keep_next = 0.0f;
            if (adv_in != nullptr && k + 1 < my_tiles) {
                const long long row = (static_cast<long long>(blockIdx.x) + static_cast<long long>(k + 1) * gridDim.x) * kTileRows + lane;
                if (row < num_segments) keep_next = ld_chk(adv_in, row * horizon + horizon - 1, num_segments * horizon);
            }
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
        if (i < 2) PUFF_STAMP(4 + 3 * i);   // data of item i arrived
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
            if (row < num_segments) stg_chk(seg_abs_sum, row, num_segments, abs_run);
        }
        // generic-proxy reads of the stage and writes of the output box are
        // ordered before the async-proxy operations issued below
        if (i < 2) PUFF_STAMP(5 + 3 * i);   // item i computed
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            if (box_ok(cbase, tile * kTileRows, horizon, num_segments)) tma_store_2d(&tm_a, cbase, tile * kTileRows, ob);
            bulk_commit();
            if (ld_i < total) issue_next();
        }
        if (i < 2) PUFF_STAMP(6 + 3 * i);   // item i's store issued
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
    PUFF_STAMP(10);   // stores have left shared memory
}


// ---------------------------------------------------------------------------
// tma2d, warp-specialised: one CTA per tile stream, seven warps with three roles
// ---------------------------------------------------------------------------
// A lone warp per tile cannot issue instructions fast enough to keep up with
// HBM once the pipeline is deep (measured: one such warp per SM is compute
// bound at about a third of the bandwidth).  Here the work of a 32x32 chunk is
// split by dependency instead:
//   warp 0      producer: waits for a free stage, issues the four TMA loads
//   warps 2,3,4,6  terms: 128 threads, 8 columns of one row each, read the raw
//                         boxes and write delta and k = (gamma*lambda*c)*nn of
//                         every step into a terms buffer (same swizzled layout);
//                         columns without a step get delta = k = 0
//   warp 1      chain:    lane r walks row r's 32 steps from the terms buffer,
//                         A = delta + k*A, stores the advantages by TMA.  When the
//                         terms warps flagged a non-binary nn or a gain beyond
//                         kPackedMaxGain, or A exceeds kPackedMaxAdv, it redoes the
//                         chunk in the reference's literal order straight from global
//                         memory (rare, slow)
//   warp 5      idle:     warps are dealt to the SM's four schedulers round robin, so
//                         an idle warp 5 leaves the scheduler of warp 1 to the chain
//                         warps of the SM's two CTAs (measured 1.6 % faster)
// Rings: NST raw stages (full: TMA -> terms, sfree: terms -> producer) and NT
// terms buffers (tfull: terms -> chain, tfree: chain -> terms).
constexpr int kWsTermWarps = 4;
constexpr int kWsThreads = 32 * (3 + kWsTermWarps);   // warp 5 idles: see the role table
constexpr int kTermBytes = 2 * kBoxBytes;   // delta | k = (gamma*lambda*c)*nn

constexpr int kWsOutSlots = 4;   // output boxes in flight behind the TMA stores
template <int NST, int NT>
constexpr int tma2d_ws_smem_bytes()
{
    return NST * kStageBytes + NT * kTermBytes + kWsOutSlots * kBoxBytes + (2 * NST + 2 * NT) * 8 + NT * 4 + 64 + 1024;
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
    if (warp == 0) PUFF_STAMP(0);

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
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_r);
        prefetch_tensormap(&tm_d);
        prefetch_tensormap(&tm_w);
    }
    if (warp == 0) PUFF_STAMP(1);
    __syncthreads();
    pdl_wait();   // nothing above reads or writes a tensor
    pdl_launch_dependents();
    if (warp == 0) PUFF_STAMP(2);

    const float gl = __fmul_rn(gamma, lambda);
    bool failed = false;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            // (The first ring-full issued by one lane of each of four WARPS, one array each, was
            // measured as well: 1024 x 64 3.30 -> 3.25 us, 8192 x 64 4.68 -> 4.60, but 8192 x 128
            // 6.65 -> 6.94 and 16384 x 64 6.84 -> 7.12; not kept.)
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
                    int x = c * kChunkCols, y = tile * kTileRows;
                    if (!box_ok(x, y, horizon, num_segments)) x = y = 0;   // debug builds: recorded, a valid box is read instead
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
    } else if (warp == 5) {
        // idle: warps are dealt to the SM's four schedulers round robin, so this keeps the
        // scheduler of the chain warp (warp 1) free of a terms warp
    } else if (warp >= 2) {
        // ------------------------------- terms --------------------------------
        const int tt = (warp == 6 ? 3 : warp - 2) * 32 + lane;   // 0..127
        const int row = tt >> 2;                  // row of the tile
        const int g = tt & 3;                     // which 8 columns of the chunk
        const uint32_t rsw = static_cast<uint32_t>(row) & 7u;
        const uint32_t off0 = static_cast<uint32_t>(row) * 128u + (((2u * g) ^ rsw) << 4);
        const uint32_t off1 = static_cast<uint32_t>(row) * 128u + (((2u * g + 1u) ^ rsw) << 4);
        float first_v = 0.0f, first_r = 0.0f, first_d = 0.0f;   // column 0 of the previous (later) chunk
        int c = nchunks - 1, s = 0, b = 0;
        uint32_t sround = 0, bround = 0;
        [[maybe_unused]] long long cy_twait = 0, cy_twork = 0;
        PUFF_TICK_DECL;
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
            PUFF_TICK(cy_twait);
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
            // column 8g+8: column 0 of the next lane's eight, or (g == 3) column 0 of the
            // previous (later) chunk, which the row's g == 0 lane carries
            {
                const int src = g == 3 ? (lane & ~3) : lane + 1;
                v[8] = __shfl_sync(0xffffffffu, g == 0 ? first_v : v[0], src);
                r[8] = __shfl_sync(0xffffffffu, g == 0 ? first_r : r[0], src);
                d[8] = __shfl_sync(0xffffffffu, g == 0 ? first_d : d[0], src);
            }
            first_v = v[0];
            first_r = r[0];
            first_d = d[0];
            const int col0 = c * kChunkCols + 8 * g;
            float dl[8], kk[8];
            uint32_t nonbin = 0u;
            float gain = 0.0f;   // largest |(gamma*lambda)*c| of this thread's steps
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
#pragma unroll
                for (int j = 0; j < 8; j += 7) {   // steps 0 and 7
                    float dj, gj, nj;
                    adv_terms(v[j], w[j], v[j + 1], r[j + 1], d[j + 1], gamma, gl, rho_clip, c_clip, dj, gj, nj);
                    dl[j] = dj;
                    kk[j] = __fmul_rn(gj, nj);
                    gain = fmaxf(gain, fabsf(gj));
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
                    gain = valid ? fmaxf(gain, fabsf(gj)) : gain;
                    nonbin |= valid ? __float_as_uint(__fmul_rn(d[j + 1], nj)) : 0u;
                }
            }
            const uint32_t tb = term_base + b * kTermBytes;
            sts128(tb + 0 * kBoxBytes + off0, make_float4(dl[0], dl[1], dl[2], dl[3]));
            sts128(tb + 0 * kBoxBytes + off1, make_float4(dl[4], dl[5], dl[6], dl[7]));
            sts128(tb + 1 * kBoxBytes + off0, make_float4(kk[0], kk[1], kk[2], kk[3]));
            sts128(tb + 1 * kBoxBytes + off1, make_float4(kk[4], kk[5], kk[6], kk[7]));
            if ((nonbin << 1) != 0u || !(gain <= kPackedMaxGain)) sts32u(flag_base + 4 * b, 1u);
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
            PUFF_TICK(cy_twork);
        }
        if (warp == 2) {
            PUFF_PUT(9, cy_twait);
            PUFF_PUT(10, cy_twork);
        }
        if (failed && lane == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    } else {
        // ------------------------------- chain --------------------------------
        if (lane == 0) prefetch_tensormap(&tm_a);
        const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
        const uint32_t sw = static_cast<uint32_t>(lane) & 7u;
        float a_run = 0.0f, abs_run = 0.0f, keep_last = 0.0f;
        // The caller's advantages[row, H-1] of a tile is fetched one tile ahead: the value is
        // needed within the tile's first item, and a DRAM round trip under load is longer than
        // several items of this warp's work.
        float keep_next = 0.0f;
        if (adv_in != nullptr && my_tiles > 0) {
            const long long row = static_cast<long long>(blockIdx.x) * kTileRows + lane;
            if (row < num_segments) keep_next = ld_chk(adv_in, row * horizon + horizon - 1, num_segments * horizon);
        }
        int k = 0, c = nchunks - 1, b = 0, oslot = 0;
        uint32_t bround = 0;
        // The TMA store of an item is issued one item late, behind the shared-memory loads of
        // the next item, so that the proxy fence and the store issue overlap their latency.
        bool pend = false;
        int pend_x = 0, pend_y = 0;
        uint32_t pend_ob = 0;
        [[maybe_unused]] long long cy_wait = 0, cy_load = 0, cy_chain = 0, cy_store = 0;
        PUFF_TICK_DECL;
        for (int i = 0; i < total; ++i) {
            const int tile = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
            if (c == nchunks - 1) {   // tile start
                keep_last = keep_next;
                keep_next = 0.0f;
                if (adv_in != nullptr && k + 1 < my_tiles) {
                    const long long row = (static_cast<long long>(tile) + gridDim.x) * kTileRows + lane;
                    if (row < num_segments) keep_next = ld_chk(adv_in, row * horizon + horizon - 1, num_segments * horizon);
                }
                a_run = 0.0f;
                abs_run = 0.0f;
            }
            if (!mbar_wait_warp(bar_tfull + 8 * b, bround & 1u)) {
                failed = true;
                break;
            }
            PUFF_TICK(cy_wait);
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
            if (pend) fence_proxy_async();   // the previous item's output box, written by every lane
            // the terms buffer is free as soon as every lane holds its values
            __syncwarp();
            if (lane == 0) {
                if (pend) {
                    if (box_ok(pend_x, pend_y, horizon, num_segments)) tma_store_2d(&tm_a, pend_x, pend_y, pend_ob);
                    bulk_commit();
                }
                if (flag != 0u) sts32u(flag_base + 4 * b, 0u);
                mbar_arrive(bar_tfree + 8 * b);
                // with at most kWsOutSlots-1 stores still reading, this item's output box is free
                bulk_wait_read<kWsOutSlots - 1>();
            }
            PUFF_TICK(cy_load);
            const int cbase = c * kChunkCols;
            const float a_in = a_run;
            bool literal = flag != 0u;
            float abs_chunk = 0.0f;
            if (!literal) {
                // sum of |A| on two side chains that issue in the shadow of the recurrence's
                // dependent multiply-add (fixed order: odd and even columns, then their sum)
                float s_odd = 0.0f, s_even = 0.0f;
#pragma unroll
                for (int j = 31; j >= 0; j -= 2) {
                    a_run = __fadd_rn(dl[j], __fmul_rn(kk[j], a_run));
                    out[j] = a_run;
                    s_odd = __fadd_rn(s_odd, fabsf(a_run));
                    a_run = __fadd_rn(dl[j - 1], __fmul_rn(kk[j - 1], a_run));
                    out[j - 1] = a_run;
                    s_even = __fadd_rn(s_even, fabsf(a_run));
                }
                abs_chunk = __fadd_rn(s_odd, s_even);
                literal = __any_sync(0xffffffffu, !(__fadd_rn(fabsf(a_in), abs_chunk) <= kPackedMaxAdv));
            }
            if (literal) {   // rare: the reference's literal order, operands straight from global memory
                a_run = a_in;
                const long long row = static_cast<long long>(tile) * kTileRows + lane;
                const bool in_rows = row < num_segments;
                const long long ro = (in_rows ? row : 0) * horizon;
                const long long total_elems = num_segments * horizon;
#pragma unroll
                for (int j = 31; j >= 0; --j) {
                    const int t = cbase + j;
                    if (in_rows && t < horizon - 1)
                        a_run = adv_step(ldg_chk(raw_v, ro + t, total_elems), ldg_chk(raw_w, ro + t, total_elems),
                                         ldg_chk(raw_v, ro + t + 1, total_elems), ldg_chk(raw_r, ro + t + 1, total_elems),
                                         ldg_chk(raw_d, ro + t + 1, total_elems), a_run, gamma, gl, rho_clip, c_clip);
                    out[j] = a_run;
                }
                abs_chunk = abs_tree32(out);
            }
            if (EPI) abs_run = __fadd_rn(abs_run, abs_chunk);
            PUFF_TICK(cy_chain);
            const uint32_t ob = out_base + oslot * kBoxBytes;
            __syncwarp();   // lane 0 has seen this item's output box free (above)
            if (cbase + kChunkCols >= horizon) {   // the chunk that holds column H-1: it goes back unchanged
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (cbase + 4 * u + 3 == horizon - 1) out[4 * u + 3] = keep_last;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t off = row_off + ((static_cast<uint32_t>(u) ^ sw) << 4);
                sts128(ob + off, make_float4(out[4 * u], out[4 * u + 1], out[4 * u + 2], out[4 * u + 3]));
            }
            if (EPI && c == 0) {
                const long long row = static_cast<long long>(tile) * kTileRows + lane;
                if (row < num_segments) stg_chk(seg_abs_sum, row, num_segments, abs_run);
            }
            pend = true;
            pend_x = cbase;
            pend_y = tile * kTileRows;
            pend_ob = ob;
            if (--c < 0) {
                c = nchunks - 1;
                ++k;
            }
            if (++b == NT) {
                b = 0;
                ++bround;
            }
            if (++oslot == kWsOutSlots) oslot = 0;
            PUFF_TICK(cy_store);
        }
        PUFF_PUT(4, cy_wait);
        PUFF_PUT(5, cy_load);
        PUFF_PUT(6, cy_chain);
        PUFF_PUT(7, cy_store);
        PUFF_PUT(8, total);
        if (pend && !failed) {   // the last item's store
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                if (box_ok(pend_x, pend_y, horizon, num_segments)) tma_store_2d(&tm_a, pend_x, pend_y, pend_ob);
                bulk_commit();
            }
        }
        if (lane == 0) {
            // the stores only have to be done reading shared memory before the CTA exits;
            // their global writes complete with the grid
            bulk_wait_read<0>();
            if (failed) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
        }
    }
}

}  // namespace puff
