// Serial advantage kernels for H % 4 != 0 on dense row tiles fetched by 1-D bulk copies: one-stage and warp-specialised forms.
// Included by puff_advantage_sm100.cu after puff_device.cuh.
#pragma once
#include "puff_device.cuh"

namespace puff {

// ---------------------------------------------------------------------------
// bulk1d: serial, dense tiles of `tile_rows` whole rows fetched by 1-D bulk copies
// ---------------------------------------------------------------------------
// For H % 4 != 0 the row pitch is not a multiple of 16 bytes and no 2-D tensor
// map exists, but a tile of whole rows is one contiguous span per array;
// tile_rows is a multiple of 4, so every tile starts on a 16-byte boundary for
// any H.  (The last tile of a buffer may have a byte size that is not a
// multiple of 16: it is fetched with plain loads.)
//
// A team of threads per tile -- one of the CTA's four warps (8-row tiles, H <= 144) or the
// whole CTA (up to 32 rows) -- with one stage of shared memory (v | r | d | w, dense, pitch H);
// the teams of an SM overlap each other's phases:
//   1. one thread issues four cp.async.bulk copies, the team waits on its mbarrier
//   2. terms, all threads of the team over the flat tile in units of four elements:
//      delta and k = (gamma*lambda*c)*nn of every step go to registers; after one
//      barrier (every raw operand has been read) they are written as interleaved
//      (delta, k) pairs over the d | w region
//   3. chain, the team's first warp: lane r walks row r with one 64-bit shared load per step,
//      A = delta + k*A, A written into the v region (stride H words: conflict-free
//      for odd H).  A non-binary nn or advantages near the overflow range send the
//      tile down the reference's literal order, operands straight from global memory
//   4. write-out: the finished tile is dense in the v region and contiguous in global memory,
//      so it leaves through ONE 1-D bulk store issued by thread 0 (a memory system that is busy
//      reading takes plain stores slowly: the 128-bit stores this replaces took 1 us per tile).
//      The store covers column H-1 as well: lane r reads its row's advantages[H-1] while the
//      tile's inputs are in flight and the store writes that value back (0 when the op owns
//      the column)
constexpr int kB1Threads = 128;
constexpr int kB1MaxUnits = 9;                                   // units of four elements per thread
constexpr int kB1MaxElems = kB1Threads * kB1MaxUnits * 4;         // elements per tile (72 KB of stage)
constexpr int kB1WarpMaxElems = 32 * kB1MaxUnits * 4;             // ... per tile of a warp-sized team

// TEAM threads work on one tile: the whole CTA (TEAM = 128, one tile per CTA and pass), or each
// of its four warps on a tile of its own (TEAM = 32: four times as many, four times smaller
// tiles with a stage, an mbarrier and a bulk store each).  The warps of a CTA then run the
// phases below independently -- no CTA-wide barrier inside the loop -- so one warp's chain
// overlaps another's fetch and terms, and the four chains of a CTA sit on four different
// schedulers.  Measured against one tile per CTA: 10007 x 127 9.55 against 9.92 us, 8192 x 91
// 6.37 against 6.61, 5000 x 127 6.81 against 7.04 (two pairs of warps on 16-row tiles: level
// with four warps).  The chains then run at ~35 cycles a step instead of 19 -- four times as
// many chain warps, each a quarter full, share the issue slots -- which is what keeps the gain
// at 4 %.
template <int TEAM>
__device__ __forceinline__ void b1_team_sync()
{
    if (TEAM == 32) __syncwarp();
    else __syncthreads();
}
template <int TEAM>
__device__ __forceinline__ bool b1_team_or(bool pred)
{
    if (TEAM == 32) return __any_sync(0xffffffffu, pred) != 0;
    return __syncthreads_or(pred) != 0;
}

template <int TEAM>
__global__ void __launch_bounds__(kB1Threads)
puff_adv_bulk1d_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                       const float* __restrict__ dones, const float* __restrict__ importance,
                       float* __restrict__ advantages, float* __restrict__ seg_abs_sum, float gamma,
                       float lambda, float rho_clip, float c_clip, long long num_segments,
                       int horizon, int tile_rows, long long num_tiles, int zero_last)
{
    if (threadIdx.x == 0) PUFF_STAMP(0);   // CTA start
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    float* const smem_f = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
    constexpr int kTeams = kB1Threads / TEAM;
    const int tid = threadIdx.x % TEAM;      // thread of the team
    const int team = threadIdx.x / TEAM;
    const int tile_elems = tile_rows * horizon;
    const uint32_t arr_pitch = (static_cast<uint32_t>(tile_elems) * 4u + 15u) & ~15u;   // bytes, 16-byte aligned
    const uint32_t team_bytes = 4u * arr_pitch;                                          // one stage: v | r | d | w
    const uint32_t stage = base + team * team_bytes;
    const uint32_t bar = base + kTeams * team_bytes + 8u * team;
    float* const sv = smem_f + team * (team_bytes / 4);
    float* const sr = sv + arr_pitch / 4;
    float* const sd = sr + arr_pitch / 4;
    float* const swt = sd + arr_pitch / 4;

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
    if (threadIdx.x == 0) PUFF_STAMP(1);   // set-up done
    pdl_wait();   // nothing above reads or writes a tensor
    pdl_launch_dependents();
    if (threadIdx.x == 0) PUFF_STAMP(2);   // predecessor complete

    const float gl = __fmul_rn(gamma, lambda);
    const float* const src[4] = {values, rewards, dones, importance};
    uint32_t parity = 0u;
    bool failed = false;

    const long long first_tile = static_cast<long long>(blockIdx.x) * kTeams + team;
    if (TEAM < kB1Threads && threadIdx.x == 0) {
        // The first tiles of the four warps are requested by ONE thread, in warp order: the copies
        // then complete in that order, a quarter of the CTA's bytes apart, and each warp starts
        // on its tile while the later ones are still in flight.
        for (int w = 0; w < kTeams; ++w) {
            const long long t = static_cast<long long>(blockIdx.x) * kTeams + w;
            if (t >= num_tiles) break;
            const long long rem = num_segments - t * tile_rows;
            const int n_el = static_cast<int>(rem < tile_rows ? rem : tile_rows) * horizon;
            const uint32_t bulk_bytes = (static_cast<uint32_t>(n_el) * 4u) & ~15u;
            const long long goff = t * tile_elems;
            if (bulk_bytes == 0u) continue;
            const long long from = idx_ok(goff + n_el - 1, num_segments * horizon) ? goff : 0;
            const uint32_t wbar = base + kTeams * team_bytes + 8u * w;
            mbar_expect_tx(wbar, 4u * bulk_bytes);
            for (int a = 0; a < 4; ++a)
                bulk_load_1d(base + w * team_bytes + a * arr_pitch, src[a] + from, bulk_bytes, wbar);
        }
    }
    for (long long tile = first_tile; tile < num_tiles; tile += static_cast<long long>(gridDim.x) * kTeams) {
        const long long rem = num_segments - tile * tile_rows;
        const int rows = static_cast<int>(rem < tile_rows ? rem : tile_rows);
        const int n_el = rows * horizon;
        const uint32_t bytes = static_cast<uint32_t>(n_el) * 4u;
        const long long goff = tile * tile_elems;
        const long long total_elems = num_segments * horizon;
        float keep_last = 0.0f;   // warp 0, lane = row
        // ---- 1. fetch ----
        // bulk copies for the 16-byte multiple of the span (all of it, except in a last tile
        // whose row count makes the byte size ragged), plain loads for the up to three
        // trailing floats of each array
        {
            const uint32_t bulk_bytes = bytes & ~15u;
            if (bulk_bytes != 0u && !(TEAM < kB1Threads && tile == first_tile)) {
                if (tid == 0) {
                    // debug builds: a span that leaves the arrays is recorded, and the first rows are read instead
                    const long long from = idx_ok(goff + n_el - 1, total_elems) ? goff : 0;
                    bulk_wait_read<0>();   // the previous tile's store has read the v region
                    mbar_expect_tx(bar, 4u * bulk_bytes);
                    for (int a = 0; a < 4; ++a) bulk_load_1d(stage + a * arr_pitch, src[a] + from, bulk_bytes, bar);
                }
            }
            // the caller's advantages[row, H-1], for the write-out (requested now, used after the chain)
            if (tid < rows && !zero_last) keep_last = ld_chk(advantages, goff + static_cast<long long>(tid) * horizon + horizon - 1, total_elems);
            const int first_tail = static_cast<int>(bulk_bytes >> 2);
            if (bulk_bytes == 0u && tid == 0) bulk_wait_read<0>();
            if (bulk_bytes == 0u) b1_team_sync<TEAM>();   // (a tile of one to three floats: plain loads only)
            if (tid < 4 * (n_el - first_tail)) {   // at most 12 threads
                const int a = tid / (n_el - first_tail), e = first_tail + tid % (n_el - first_tail);
                (sv + (a * arr_pitch) / 4)[e] = ldg_chk(src[a], goff + e, total_elems);
            }
            if (bulk_bytes != 0u) {
                if (!mbar_wait_thread(bar, parity)) failed = true;
                parity ^= 1u;
            }
            if (threadIdx.x == 0 && tile == first_tile) PUFF_STAMP(3);   // first tile: thread 0 saw the data
            if (b1_team_or<TEAM>(failed)) {
                failed = true;
                break;
            }
            if (threadIdx.x == 0 && tile == first_tile) PUFF_STAMP(4);   // ... and so did everybody
        }
        // ---- 2. terms ----
        // a thread owns units of four consecutive elements (one 16-byte unit per array);
        // the operand at e+4 comes from the next unit
        uint32_t nonbin = 0u;
        float gain = 0.0f;   // largest |(gamma*lambda)*c| of this thread's steps
        const int n_grp = (n_el + 3) >> 2;
        const int grp_stride_cols = (4 * TEAM) % horizon;
        float4 dl4[kB1MaxUnits], kk4[kB1MaxUnits];
        {
            int col_g = (4 * tid) % horizon;   // column of the first element of this thread's next unit
#pragma unroll
            for (int u = 0; u < kB1MaxUnits; ++u) {
                const int grp = u * TEAM + tid;
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
                        gain = valid ? fmaxf(gain, fabsf(gj)) : gain;
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
        b1_team_sync<TEAM>();   // every raw operand of the tile has been read
        if (threadIdx.x == 0 && tile == first_tile) PUFF_STAMP(5);   // terms in registers
        float2* const st = reinterpret_cast<float2*>(sd);   // (delta, k) pairs over the d | w region
#pragma unroll
        for (int u = 0; u < kB1MaxUnits; ++u) {
            const int grp = u * TEAM + tid;
            const int e = grp << 2;
            if (grp < n_grp) {
                *reinterpret_cast<float4*>(st + e) = make_float4(dl4[u].x, kk4[u].x, dl4[u].y, kk4[u].y);
                *reinterpret_cast<float4*>(st + e + 2) = make_float4(dl4[u].z, kk4[u].z, dl4[u].w, kk4[u].w);
            }
        }
        const bool any_nonbin = b1_team_or<TEAM>((nonbin << 1) != 0u || !(gain <= kPackedMaxGain));
        if (threadIdx.x == 0 && tile == first_tile) PUFF_STAMP(6);   // pairs in shared memory
        // ---- 3. chain ----
        if (tid < 32) {
            const int lane = tid;
            const int ro = lane * horizon;
            const bool mine = lane < rows;
            float a_run = 0.0f, abs_run = 0.0f;
            bool literal = any_nonbin;
            // a warp that a one-lane branch above left split runs the dependent chain twice as slowly
            __syncwarp();
            [[maybe_unused]] const long long chain_t0 = clock64();
            if (!literal) {
                if (mine) {
                    // plain accesses, scheduled by the compiler (measured no slower here than the
                    // explicit prefetch of chain_pairs_row): 18-20 cycles a step
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
                literal = __any_sync(0xffffffffu, !(abs_run <= kPackedMaxAdv));
            }
            if (threadIdx.x < 32 && tile == first_tile) PUFF_PUT(8, clock64() - chain_t0);   // cycles of the first tile's chain loop
            if (literal) {   // rare: the reference's literal order, operands straight from global memory
                a_run = 0.0f;
                abs_run = 0.0f;
                if (mine) {
                    const long long gro = goff + ro;
                    for (int t = horizon - 2; t >= 0; --t) {
                        a_run = adv_step(ldg_chk(values, gro + t, total_elems), ldg_chk(importance, gro + t, total_elems),
                                         ldg_chk(values, gro + t + 1, total_elems), ldg_chk(rewards, gro + t + 1, total_elems),
                                         ldg_chk(dones, gro + t + 1, total_elems), a_run, gamma, gl, rho_clip, c_clip);
                        sv[ro + t] = a_run;
                        abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    }
                }
            }
            if (mine && seg_abs_sum != nullptr) stg_chk(seg_abs_sum, tile * tile_rows + lane, num_segments, abs_run);
            // ---- 4. write-out ----
            if (mine) sv[ro + horizon - 1] = keep_last;
            fence_proxy_async();
            __syncwarp();
            const uint32_t out_bytes = bytes & ~15u;
            if (lane == 0) {
                if (out_bytes != 0u && idx_ok(goff + n_el - 1, total_elems))
                    bulk_store_1d(advantages + goff, smem_u32(sv), out_bytes);
                bulk_commit();
            }
            for (int e = static_cast<int>(out_bytes >> 2) + lane; e < n_el; e += 32)   // ragged last tile
                stg_chk(advantages, goff + e, total_elems, sv[e]);
        }
        // every generic access to the stage is ordered before the async-proxy refill of the next tile
        fence_proxy_async();
        b1_team_sync<TEAM>();
        if (threadIdx.x == 0 && tile == first_tile) PUFF_STAMP(7);   // chain done, store issued
    }
    if (tid == 0) bulk_wait_read<0>();   // the last store has left shared memory
    if (failed && tid == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    if (threadIdx.x == 0) PUFF_STAMP(10);
}

// ---------------------------------------------------------------------------
// bulk1d, warp-specialised: the odd-horizon counterpart of the tma2d pipeline
// ---------------------------------------------------------------------------
// The same split by dependency as puff_adv_tma2d_ws_kernel, on dense tiles of `tile_rows`
// whole rows (a contiguous span per array, see bulk1d above); eleven warps:
//   warp 0       producer: four cp.async.bulk copies per tile into a 2-deep ring of raw
//                stages (plus plain loads of the up to three ragged floats per array)
//   warps 3..10  terms: stream over the flat tile in units of four elements and write
//                (delta, k) pairs into one of two terms buffers
//   warps 1, 2   chain: warp b owns terms buffer b and output buffer b (every other tile);
//                lane r walks row r, A = delta + k*A, into a dense [rows][H] output tile that
//                leaves through ONE 1-D bulk store (a whole tile is contiguous in global
//                memory).  The store covers column H-1 as well, so the lane first reads its
//                row's advantages[H-1] and the store writes that value back (or 0 when the
//                op owns the column).  Literal order from global memory when a non-binary nn
//                was flagged or the advantages near the overflow range.
// (Cycle accounting of an earlier form, in which the terms warps wrote the tiles out with plain
// 128-bit stores, showed them spending as long in those stores as in the terms: a memory system
// that is busy reading takes plain stores slowly, and the raw stages were held up behind them.)
// One CTA per SM; tiles are pipelined inside it, so the kernel streams at buffer sizes
// where the one-stage bulk1d kernel is still phase-bound.  Measured at 131072 x 127 with the
// ring depth as a template parameter: two stages of 32 rows 55.0 us, three of 24 rows 61.5,
// four of 16 rows 79.8, two of 16 rows 80.0 -- a tile's way through terms and chain takes
// about as long whatever its height, so the tallest tile that fits wins.
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
    // Logical warp: 0 producer, 1..2 chain, 3..10 terms.  Warps are dealt to the SM's four
    // schedulers round robin; physical warps 3 and 7 share one that no other warp of the
    // CTA uses, and the two chain warps get it.
    const int phys_warp = threadIdx.x >> 5;
    const int warp = phys_warp == 0 ? 0 : phys_warp == 3 ? 1 : phys_warp == 7 ? 2
                   : phys_warp < 3 ? phys_warp + 2 : phys_warp < 7 ? phys_warp + 1 : phys_warp;
    const int lane = threadIdx.x & 31;
    const int tile_elems = tile_rows * horizon;
    const uint32_t arr_pitch = (static_cast<uint32_t>(tile_elems) * 4u + 15u) & ~15u;   // one raw array of a stage
    const uint32_t stage_bytes = 4u * arr_pitch;
    const uint32_t term_bytes = 2u * arr_pitch;                                          // (delta, k) pairs
    const uint32_t term_base = kB1wStages * stage_bytes;
    const uint32_t out_base = term_base + kB1wTerms * term_bytes;                        // dense advantages, per chain warp
    const uint32_t bar_off = out_base + kB1wTerms * arr_pitch;
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
    pdl_wait();   // nothing above reads or writes a tensor
    pdl_launch_dependents();

    const float gl = __fmul_rn(gamma, lambda);
    const long long total_elems = num_segments * horizon;
    bool failed = false;
    auto rows_of = [&](long long tile) {
        const long long rem = num_segments - tile * tile_rows;
        return static_cast<int>(rem < tile_rows ? rem : tile_rows);
    };

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const float* const src[4] = {values, rewards, dones, importance};
            [[maybe_unused]] long long cy_pwait = 0, cy_pwork = 0;
            PUFF_TICK_DECL;
            for (long long n = 0; n < my_tiles; ++n) {
                const int s = static_cast<int>(n % kB1wStages);
                const uint32_t round = static_cast<uint32_t>(n / kB1wStages);
                PUFF_TICK(cy_pwork);
                if (round > 0 && !mbar_wait_thread(bar_sfree + 8 * s, (round - 1) & 1u)) {
                    failed = true;
                    break;
                }
                PUFF_TICK(cy_pwait);
                const long long tile = blockIdx.x + n * gridDim.x;
                const int n_el = rows_of(tile) * horizon;
                const long long goff = tile * tile_elems;
                const uint32_t bulk_bytes = (static_cast<uint32_t>(n_el) * 4u) & ~15u;
                float* const stage_f = reinterpret_cast<float*>(smem_al + s * stage_bytes);
                // ragged floats first: the arrive below publishes them together with the bulk bytes
                for (int e = static_cast<int>(bulk_bytes >> 2); e < n_el; ++e)
                    for (int a = 0; a < 4; ++a)
                        (stage_f + a * (arr_pitch / 4))[e] = ldg_chk(src[a], goff + e, total_elems);
                const uint32_t bar = bar_full + 8 * s;
                if (bulk_bytes != 0u) {
                    // debug builds: a span that leaves the arrays is recorded, and the first rows are read instead
                    const long long from = idx_ok(goff + n_el - 1, total_elems) ? goff : 0;
                    mbar_expect_tx(bar, 4u * bulk_bytes);
                    for (int a = 0; a < 4; ++a)
                        bulk_load_1d(base + s * stage_bytes + a * arr_pitch, src[a] + from, bulk_bytes, bar);
                } else {
                    mbar_arrive(bar);
                }
            }
            PUFF_PUT(0, cy_pwait);
            PUFF_PUT(1, my_tiles);
            if (failed) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
        }
    } else if (warp > kB1wTerms) {
        // --------------------------- terms + copy-out --------------------------
        const int tt = (warp - 1 - kB1wTerms) * 32 + lane;   // 0 .. kB1wTermThreads-1
        const int unit_stride_cols = (4 * kB1wTermThreads) % horizon;
        [[maybe_unused]] long long cy_tfullwait = 0, cy_terms = 0, cy_cwait = 0, cy_copy = 0;
        PUFF_TICK_DECL;
        for (long long n = 0; n < my_tiles; ++n) {
            const int s = static_cast<int>(n % kB1wStages), b = static_cast<int>(n % kB1wTerms);
            PUFF_TICK(cy_copy);
            if (!mbar_wait_warp(bar_full + 8 * s, static_cast<uint32_t>(n / kB1wStages) & 1u)) {
                failed = true;
                break;
            }
            PUFF_TICK(cy_tfullwait);
            // terms buffer b was last used by tile n - kB1wTerms: its chain must be through with it
            if (n >= kB1wTerms &&
                !mbar_wait_warp(bar_cdone + 8 * b, static_cast<uint32_t>(n / kB1wTerms - 1) & 1u)) {
                failed = true;
                break;
            }
            PUFF_TICK(cy_cwait);
            const long long tile = blockIdx.x + n * gridDim.x;
            const int n_el = rows_of(tile) * horizon;
            const int n_grp = (n_el + 3) >> 2;
            const float* const sv = reinterpret_cast<const float*>(smem_al + s * stage_bytes);
            const float* const sr = sv + arr_pitch / 4;
            const float* const sd = sr + arr_pitch / 4;
            const float* const swt = sd + arr_pitch / 4;
            float2* const tp = reinterpret_cast<float2*>(smem_al + term_base + b * term_bytes);
            uint32_t nonbin = 0u;
            float gain = 0.0f;   // largest |(gamma*lambda)*c| of this thread's steps
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
                    gain = valid ? fmaxf(gain, fabsf(gj)) : gain;
                    nonbin |= valid ? __float_as_uint(__fmul_rn(d[j + 1], nj)) : 0u;
                    col = col + 1 == horizon ? 0 : col + 1;
                }
                *reinterpret_cast<float4*>(tp + e) = make_float4(dl[0], kk[0], dl[1], kk[1]);
                *reinterpret_cast<float4*>(tp + e + 2) = make_float4(dl[2], kk[2], dl[3], kk[3]);
                col_g += unit_stride_cols;
                if (col_g >= horizon) col_g -= horizon;
            }
            if ((nonbin << 1) != 0u || !(gain <= kPackedMaxGain)) sts32u(flag_base + 4 * b, 1u);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_tfull + 8 * b);
                mbar_arrive(bar_sfree + 8 * s);
            }
            PUFF_TICK(cy_terms);
        }
        if (warp == kB1wTerms + 1) {
            PUFF_PUT(2, cy_tfullwait);
            PUFF_PUT(3, cy_terms);
            PUFF_PUT(4, cy_cwait);
            PUFF_PUT(5, cy_copy);
        }
        if (failed && lane == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    } else {
        // ------------------------------- chain --------------------------------
        [[maybe_unused]] long long cy_chwait = 0, cy_chwork = 0;
        PUFF_TICK_DECL;
        for (long long n = warp - 1; n < my_tiles; n += kB1wTerms) {
            const int b = warp - 1;
            PUFF_TICK(cy_chwork);
            if (!mbar_wait_warp(bar_tfull + 8 * b, static_cast<uint32_t>(n / kB1wTerms) & 1u)) {
                failed = true;
                break;
            }
            PUFF_TICK(cy_chwait);
            const long long tile = blockIdx.x + n * gridDim.x;
            const int rows = rows_of(tile);
            float2* const tp = reinterpret_cast<float2*>(smem_al + term_base + b * term_bytes);
            float* const ob = reinterpret_cast<float*>(smem_al + out_base + b * arr_pitch);
            const uint32_t flag = lds32u(flag_base + 4 * b);
            __syncwarp();
            if (lane == 0) {
                if (flag != 0u) sts32u(flag_base + 4 * b, 0u);
                bulk_wait_read<0>();   // this warp's previous store has read the output buffer
            }
            const int ro = lane * horizon;
            const bool mine = lane < rows;
            const long long goff = tile * tile_elems;
            // the caller's advantages[row, H-1] goes back unchanged (0 when the op owns the column)
            float keep_last = 0.0f;
            if (mine && !zero_last) keep_last = ld_chk(advantages, goff + ro + horizon - 1, total_elems);
            __syncwarp();
            float a_run = 0.0f, abs_run = 0.0f;
            bool literal = flag != 0u;
            if (!literal) {
                if (mine) chain_pairs_row(smem_u32(tp + ro), smem_u32(ob + ro), 4u, horizon - 1, a_run, abs_run);
                literal = __any_sync(0xffffffffu, !(abs_run <= kPackedMaxAdv));   // the sum bounds every |A| of the row
            }
            if (literal) {   // rare: the reference's literal order, operands straight from global memory
                a_run = 0.0f;
                abs_run = 0.0f;
                if (mine) {
                    const long long gro = tile * tile_elems + ro;
                    for (int t = horizon - 2; t >= 0; --t) {
                        a_run = adv_step(ldg_chk(values, gro + t, total_elems), ldg_chk(importance, gro + t, total_elems),
                                         ldg_chk(values, gro + t + 1, total_elems), ldg_chk(rewards, gro + t + 1, total_elems),
                                         ldg_chk(dones, gro + t + 1, total_elems), a_run, gamma, gl, rho_clip, c_clip);
                        ob[ro + t] = a_run;
                        abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    }
                }
            }
            if (mine) ob[ro + horizon - 1] = keep_last;
            if (mine && seg_abs_sum != nullptr) stg_chk(seg_abs_sum, tile * tile_rows + lane, num_segments, abs_run);
            // the output tile is complete: one bulk store for its 16-byte multiple, plain stores for
            // the up to three trailing floats of a ragged last tile
            fence_proxy_async();
            __syncwarp();
            const int n_el = rows * horizon;
            const uint32_t bulk_bytes = (static_cast<uint32_t>(n_el) * 4u) & ~15u;
            if (lane == 0) {
                mbar_arrive(bar_cdone + 8 * b);   // the pairs have been consumed
                if (bulk_bytes != 0u && idx_ok(goff + n_el - 1, total_elems))
                    bulk_store_1d(advantages + goff, smem_u32(ob), bulk_bytes);
                bulk_commit();
            }
            for (int e = static_cast<int>(bulk_bytes >> 2) + lane; e < n_el; e += 32)
                stg_chk(advantages, goff + e, total_elems, ob[e]);
        }
        if (lane == 0) bulk_wait_read<0>();   // the last store has left shared memory
        PUFF_TICK(cy_chwork);
        if (warp == 1) {
            PUFF_PUT(6, cy_chwait);
            PUFF_PUT(7, cy_chwork);
        }
        if (failed && lane == 0) atomicExch(&g_device_status, PUFF_ERR_DEVICE_WAIT);
    }
}

}  // namespace puff
