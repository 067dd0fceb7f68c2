// Affine-pair scan kernel (long rows, few segments) and the generic one-thread-per-row kernel.
// Included by puff_advantage_sm100.cu after puff_device.cuh.
#pragma once
#include "puff_device.cuh"

namespace puff {

// ---------------------------------------------------------------------------
// scan: NT threads per row, W = 4*UPT steps per thread, affine-pair scan of the carries
// ---------------------------------------------------------------------------
// A_t = delta_t + k_t * A_{t+1} with k_t = ((gamma*lambda)*c_t)*nn_t.  Thread j
// of a pass owns the unit of W columns G-1-j counted from the end of the
// row, so the suffix scan in time is an inclusive prefix scan over j.  The
// composed pair (K, D) of a unit maps the advantage entering it (column Wg+W)
// to the one leaving it (column Wg): A_out = D + K * A_in.  After the scan each
// thread knows its own A_in and replays its W steps in the reference's
// operation order, so only the carry-in differs from the serial result.
// UPT = 2 halves the number of passes (and of scans and barriers) of a long row and puts
// all of a thread's loads in flight at once.
template <bool VEC, int UPT>
__global__ void __launch_bounds__(1024 / UPT)
puff_adv_scan_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                     const float* __restrict__ dones, const float* __restrict__ importance,
                     float* __restrict__ advantages, float* __restrict__ seg_abs_sum, float gamma,
                     float lambda, float rho_clip, float c_clip, long long num_segments, int horizon,
                     int zero_last)
{
    constexpr int W = 4 * UPT;
    __shared__ float s_k[32], s_d[32], s_abs[32];
    __shared__ float s_carry;
    const int tid = threadIdx.x;
    const int nt = blockDim.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int nwarps = nt >> 5;
    const float gl = __fmul_rn(gamma, lambda);
    const int units = (horizon + W - 1) / W;       // units of W columns per row
    const int passes = (units + nt - 1) / nt;
    pdl_wait();
    pdl_launch_dependents();

    for (long long row = blockIdx.x; row < num_segments; row += gridDim.x) {
        const long long ro = row * horizon;
        const long long total_elems = num_segments * horizon;
        float a_pass = 0.0f;      // advantage entering this pass (from later columns)
        float abs_acc = 0.0f;     // thread 0 only
        float gain = 0.0f;        // largest |(gamma*lambda)*c| of this thread's steps
        float chk = 0.0f;         // sum of this thread's |A|: inf or NaN as soon as one of them is
        if (zero_last && tid == 0) stg_chk(advantages, ro + horizon - 1, total_elems, 0.0f);

        for (int p = 0; p < passes; ++p) {
            const int j = p * nt + tid;
            const int g = units - 1 - j;
            const bool live = g >= 0;
            const int col0 = g * W;
            float vv[W + 1], rr[W + 1], dd[W + 1], ww[W];   // index i <-> column col0+i
#pragma unroll
            for (int i = 0; i < W + 1; ++i) {
                vv[i] = 0.0f;
                rr[i] = 0.0f;
                dd[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < W; ++i) ww[i] = 0.0f;
            if (live) {
                if (VEC) {   // horizon % 4 == 0 and 16-byte aligned bases
#pragma unroll
                    for (int u = 0; u < UPT; ++u) {
                        if (col0 + 4 * u < horizon) {   // the last unit of a row may be half empty
                            const float4 v4 = ldg4_chk(values, ro + col0 + 4 * u, total_elems);
                            const float4 r4 = ldg4_chk(rewards, ro + col0 + 4 * u, total_elems);
                            const float4 d4 = ldg4_chk(dones, ro + col0 + 4 * u, total_elems);
                            const float4 w4 = ldg4_chk(importance, ro + col0 + 4 * u, total_elems);
                            vv[4 * u] = v4.x; vv[4 * u + 1] = v4.y; vv[4 * u + 2] = v4.z; vv[4 * u + 3] = v4.w;
                            rr[4 * u] = r4.x; rr[4 * u + 1] = r4.y; rr[4 * u + 2] = r4.z; rr[4 * u + 3] = r4.w;
                            dd[4 * u] = d4.x; dd[4 * u + 1] = d4.y; dd[4 * u + 2] = d4.z; dd[4 * u + 3] = d4.w;
                            ww[4 * u] = w4.x; ww[4 * u + 1] = w4.y; ww[4 * u + 2] = w4.z; ww[4 * u + 3] = w4.w;
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < W; ++i) {
                        if (col0 + i < horizon) {
                            vv[i] = ldg_chk(values, ro + col0 + i, total_elems);
                            rr[i] = ldg_chk(rewards, ro + col0 + i, total_elems);
                            dd[i] = ldg_chk(dones, ro + col0 + i, total_elems);
                            ww[i] = ldg_chk(importance, ro + col0 + i, total_elems);
                        }
                    }
                }
                if (col0 + W < horizon) {
                    vv[W] = ldg_chk(values, ro + col0 + W, total_elems);
                    rr[W] = ldg_chk(rewards, ro + col0 + W, total_elems);
                    dd[W] = ldg_chk(dones, ro + col0 + W, total_elems);
                }
            }
            // local composition over the (up to) W steps, latest column first
            float K = 1.0f, D = 0.0f;
#pragma unroll
            for (int i = W - 1; i >= 0; --i) {
                const bool step = live && (col0 + i + 1 < horizon);   // t <= H-2
                const float nn = __fsub_rn(1.0f, dd[i + 1]);
                const float rho = fminf(ww[i], rho_clip);
                const float c = fminf(ww[i], c_clip);
                const float td = __fsub_rn(__fadd_rn(rr[i + 1], __fmul_rn(__fmul_rn(gamma, vv[i + 1]), nn)), vv[i]);
                const float gc = __fmul_rn(gl, c);
                const float dl = step ? __fmul_rn(rho, td) : 0.0f;
                const float kk = step ? __fmul_rn(gc, nn) : 1.0f;
                gain = step ? fmaxf(gain, fabsf(gc)) : gain;
                D = fmaf(kk, D, dl);
                K = kk * K;
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
            chk += fabsf(a_in);
            float out[W];
#pragma unroll
            for (int i = W - 1; i >= 0; --i) {
                const bool step = live && (col0 + i + 1 < horizon);
                if (step) {
                    a_run = adv_step(vv[i], ww[i], vv[i + 1], rr[i + 1], dd[i + 1], a_run, gamma, gl,
                                     rho_clip, c_clip);
                    abs_loc += fabsf(a_run);
                }
                out[i] = a_run;
            }
            if (live) {
#pragma unroll
                for (int u = 0; u < UPT; ++u) {
                    if (VEC && col0 + 4 * u + 4 < horizon) {
                        stg4_chk(advantages, ro + col0 + 4 * u, total_elems,
                                 make_float4(out[4 * u], out[4 * u + 1], out[4 * u + 2], out[4 * u + 3]));
                    } else {
#pragma unroll
                        for (int i = 4 * u; i < 4 * u + 4; ++i)
                            if (col0 + i + 1 < horizon) stg_chk(advantages, ro + col0 + i, total_elems, out[i]);
                    }
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
            chk += abs_loc;   // after the warp reduction: lane sums, still inf / NaN when any |A| is
        }
        // Folding nn into k changes the result (not just its rounding) when ((gamma*lambda)*c)*A
        // overflows under nn == 0: the reference then carries NaN to the start of the row.  A row
        // with a gain beyond kPackedMaxGain or an advantage beyond kPackedMaxAdv is redone by one
        // thread in the reference's literal order (rare, slow).
        if (__syncthreads_or(!(gain <= kPackedMaxGain) || !(chk <= kPackedMaxAdv))) {
            if (tid == 0) {
                float a_run = 0.0f, abs_run = 0.0f;
                for (int t = horizon - 2; t >= 0; --t) {
                    a_run = adv_step(ldg_chk(values, ro + t, total_elems), ldg_chk(importance, ro + t, total_elems),
                                     ldg_chk(values, ro + t + 1, total_elems), ldg_chk(rewards, ro + t + 1, total_elems),
                                     ldg_chk(dones, ro + t + 1, total_elems), a_run, gamma, gl, rho_clip, c_clip);
                    abs_run = __fadd_rn(abs_run, fabsf(a_run));
                    stg_chk(advantages, ro + t, total_elems, a_run);
                }
                abs_acc = abs_run;
            }
        }
        if (seg_abs_sum != nullptr && tid == 0) stg_chk(seg_abs_sum, row, num_segments, abs_acc);
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
    pdl_wait();
    pdl_launch_dependents();
    for (long long row = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
         row < num_segments; row += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long ro = row * horizon;
        float a_run = 0.0f, abs_run = 0.0f;
        const long long total_elems = num_segments * horizon;
        float v_n = ldg_chk(values, ro + horizon - 1, total_elems);
        for (long long t = horizon - 2; t >= 0; --t) {
            const float v_t = ldg_chk(values, ro + t, total_elems);
            a_run = adv_step(v_t, ldg_chk(importance, ro + t, total_elems), v_n, ldg_chk(rewards, ro + t + 1, total_elems),
                             ldg_chk(dones, ro + t + 1, total_elems), a_run, gamma, gl, rho_clip, c_clip);
            abs_run = __fadd_rn(abs_run, fabsf(a_run));
            stg_chk(advantages, ro + t, total_elems, a_run);
            v_n = v_t;
        }
        if (zero_last) stg_chk(advantages, ro + horizon - 1, total_elems, 0.0f);
        if (seg_abs_sum != nullptr) stg_chk(seg_abs_sum, row, num_segments, abs_run);
    }
}

}  // namespace puff
