// Minibatch gather + advantage normalisation for the prioritised sampler (sm_100a).
//
// Replaces the eager torch sequence that follows the advantage op in the
// reference trainer (pufferlib/pufferl.py):
//     mb_prio       = (segments * prio_probs[idx, None]) ** -anneal_beta      :363
//     mb_values     = values[idx]                                              :373
//     mb_returns    = advantages[idx] + mb_values                              :374
//     mb_advantages = advantages[idx]                                          :375
//     adv = mb_prio * (adv - adv.mean()) / (adv.std() + 1e-8)                  :408-409
// (std is the unbiased one over all gathered elements, as torch.std.)
//
// Two launches: the first gathers the rows, writes values / returns / raw
// advantages and accumulates sum and sum of squares in fp64 (per-CTA partials
// in caller-owned scratch, fixed order); the second reduces the partials,
// forms mean and std, and writes the weighted, normalised advantages.  The raw
// rows it re-reads were written a few microseconds earlier and come from L2.
// Memory-bound gathers of whole rows: 8 bytes read and 12-16 written per
// gathered element.  (Both steps as ONE cooperative launch with a grid-wide
// barrier between them, the first rows kept in registers across it, measured
// 18.3 us where the two launches below, chained by programmatic dependent
// launch, take 15.5: 8192 of 131072 x 256 rows.)
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/puff_advantage.h"
#include "puff_launch.cuh"

namespace puff {
void count_launch();

constexpr int kMbThreads = 256;
constexpr int kMbMaxBlocks = 592;   // one wave: four CTAs of 256 threads on each of 148 SMs
constexpr int kMbCtasPerSm = 4;

__device__ int g_mb_bad_index = 0;

__device__ __forceinline__ void block_sum2(double& a, double& b, double* s_part)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        s_part[2 * warp] = a;
        s_part[2 * warp + 1] = b;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double ta = 0.0, tb = 0.0;
        for (int i = 0; i < (blockDim.x >> 5); ++i) {
            ta += s_part[2 * i];
            tb += s_part[2 * i + 1];
        }
        a = ta;
        b = tb;
    }
}

// one warp per gathered row; contiguous slab of rows per CTA
template <bool VEC>
__global__ void __launch_bounds__(kMbThreads, kMbCtasPerSm)
puff_mb_gather_kernel(const float* __restrict__ advantages, const float* __restrict__ values,
                      const long long* __restrict__ idx, float* __restrict__ mb_values,
                      float* __restrict__ mb_returns, float* __restrict__ mb_adv_raw,
                      double* __restrict__ partial, long long num_segments, long long horizon,
                      long long mb_segments)
{
    __shared__ double s_part[2 * kMbThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = kMbThreads / 32;
    const long long per = (mb_segments + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x;
    const long long hi = lo + per < mb_segments ? lo + per : mb_segments;
    double sum = 0.0, sq = 0.0;
    pdl_wait();
    pdl_launch_dependents();
    // two rows per warp and pass, so that a lane has four (VEC: 128-bit) loads in flight
    for (long long m0 = lo + warp; m0 < hi; m0 += 2 * nwarps) {
        const long long m1 = m0 + nwarps;
        const bool two = m1 < hi;
        const long long src0 = idx[m0], src1 = two ? idx[m1] : 0;
        const bool ok0 = src0 >= 0 && src0 < num_segments;
        const bool ok1 = !two || (src1 >= 0 && src1 < num_segments);
        if ((!ok0 || !ok1) && lane == 0) atomicExch(&g_mb_bad_index, 1);
        const float* a0 = advantages + (ok0 ? src0 : 0) * horizon;
        const float* v0 = values + (ok0 ? src0 : 0) * horizon;
        const float* a1 = advantages + (ok1 ? src1 : 0) * horizon;
        const float* v1 = values + (ok1 ? src1 : 0) * horizon;
        const long long o0 = m0 * horizon, o1 = (two ? m1 : m0) * horizon;
        if (VEC) {
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
            for (long long c = 4 * lane; c < horizon; c += 128) {
                float4 a4 = __ldg(reinterpret_cast<const float4*>(a0 + c));
                float4 v4 = __ldg(reinterpret_cast<const float4*>(v0 + c));
                float4 b4 = two ? __ldg(reinterpret_cast<const float4*>(a1 + c)) : zero4;
                float4 u4 = two ? __ldg(reinterpret_cast<const float4*>(v1 + c)) : zero4;
                if (!ok0) a4 = v4 = zero4;
                if (!ok1) b4 = u4 = zero4;
                *reinterpret_cast<float4*>(mb_values + o0 + c) = v4;
                *reinterpret_cast<float4*>(mb_returns + o0 + c) =
                    make_float4(__fadd_rn(a4.x, v4.x), __fadd_rn(a4.y, v4.y), __fadd_rn(a4.z, v4.z), __fadd_rn(a4.w, v4.w));
                *reinterpret_cast<float4*>(mb_adv_raw + o0 + c) = a4;
                sum += static_cast<double>(a4.x) + static_cast<double>(a4.y) + static_cast<double>(a4.z) + static_cast<double>(a4.w);
                sq += static_cast<double>(a4.x) * a4.x + static_cast<double>(a4.y) * a4.y +
                      static_cast<double>(a4.z) * a4.z + static_cast<double>(a4.w) * a4.w;
                if (two) {
                    *reinterpret_cast<float4*>(mb_values + o1 + c) = u4;
                    *reinterpret_cast<float4*>(mb_returns + o1 + c) =
                        make_float4(__fadd_rn(b4.x, u4.x), __fadd_rn(b4.y, u4.y), __fadd_rn(b4.z, u4.z), __fadd_rn(b4.w, u4.w));
                    *reinterpret_cast<float4*>(mb_adv_raw + o1 + c) = b4;
                    sum += static_cast<double>(b4.x) + static_cast<double>(b4.y) + static_cast<double>(b4.z) + static_cast<double>(b4.w);
                    sq += static_cast<double>(b4.x) * b4.x + static_cast<double>(b4.y) * b4.y +
                          static_cast<double>(b4.z) * b4.z + static_cast<double>(b4.w) * b4.w;
                }
            }
        } else {
            for (long long c = lane; c < horizon; c += 32) {
                const float av = ok0 ? __ldg(a0 + c) : 0.0f, vv = ok0 ? __ldg(v0 + c) : 0.0f;
                const float bv = (two && ok1) ? __ldg(a1 + c) : 0.0f, uv = (two && ok1) ? __ldg(v1 + c) : 0.0f;
                mb_values[o0 + c] = vv;
                mb_returns[o0 + c] = __fadd_rn(av, vv);
                mb_adv_raw[o0 + c] = av;
                sum += static_cast<double>(av);
                sq += static_cast<double>(av) * av;
                if (two) {
                    mb_values[o1 + c] = uv;
                    mb_returns[o1 + c] = __fadd_rn(bv, uv);
                    mb_adv_raw[o1 + c] = bv;
                    sum += static_cast<double>(bv);
                    sq += static_cast<double>(bv) * bv;
                }
            }
        }
    }
    block_sum2(sum, sq, s_part);
    if (threadIdx.x == 0) {
        partial[2 * blockIdx.x] = sum;
        partial[2 * blockIdx.x + 1] = sq;
    }
}

template <bool VEC>
__global__ void __launch_bounds__(kMbThreads, kMbCtasPerSm)
puff_mb_normalize_kernel(const float* __restrict__ mb_adv_raw, const float* __restrict__ prio_probs,
                         const long long* __restrict__ idx, const double* __restrict__ partial, int n_partial,
                         float* __restrict__ mb_adv_norm, float* __restrict__ mb_prio, float anneal_beta,
                         long long num_segments, long long prio_segments, long long horizon, long long mb_segments)
{
    __shared__ float s_mean, s_denom;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = kMbThreads / 32;
    const long long stride = static_cast<long long>(gridDim.x) * nwarps;
    long long m = blockIdx.x * static_cast<long long>(nwarps) + warp;
    pdl_wait();
    pdl_launch_dependents();
    // the warp's first row: its index and probability are requested before the reduction below,
    // so that their two dependent round trips run beside it
    long long src_row = m < mb_segments ? idx[m] : -1;
    bool ok = src_row >= 0 && src_row < num_segments;
    float p = ok ? __ldg(prio_probs + src_row) : 1.0f;
    // one warp of every CTA reduces the same few partials in the same order
    if (warp == 0) {
        double sum = 0.0, sq = 0.0;
        for (int i = lane; i < n_partial; i += 32) {
            sum += partial[2 * i];
            sq += partial[2 * i + 1];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
        }
        if (lane == 0) {
            const double n = static_cast<double>(mb_segments) * static_cast<double>(horizon);
            const double mean = sum / n;
            double var = (sq - sum * mean) / (n - 1.0);   // unbiased, as torch.std; n == 1 gives NaN there too
            if (var < 0.0) var = 0.0;
            s_mean = static_cast<float>(mean);
            s_denom = static_cast<float>(sqrt(var)) + 1e-8f;
        }
    }
    __syncthreads();
    const float mean = s_mean, denom = s_denom;
    while (m < mb_segments) {
        // the next row's index and probability, one row ahead
        const long long m_next = m + stride;
        const long long src_next = m_next < mb_segments ? idx[m_next] : -1;
        const bool ok_next = src_next >= 0 && src_next < num_segments;
        const float p_next = ok_next ? __ldg(prio_probs + src_next) : 1.0f;
        // (segments * p) ** -beta, evaluated in fp32 like the reference
        // prio_segments is the N of pufferl.py:363: the segment count the probabilities were
        // normalised over, which exceeds num_segments when this GPU holds one shard of them.
        // A row with a bad index gets weight 0, i.e. a zero row (its raw row is zero as well).
        const float prio = ok ? powf(static_cast<float>(prio_segments) * p, -anneal_beta) : 0.0f;
        if (lane == 0) mb_prio[m] = prio;
        const float* a = mb_adv_raw + m * horizon;
        float* o = mb_adv_norm + m * horizon;
        if (VEC) {
#pragma unroll 2
            for (long long c = 4 * lane; c < horizon; c += 128) {
                const float4 a4 = *reinterpret_cast<const float4*>(a + c);
                *reinterpret_cast<float4*>(o + c) =
                    ok ? make_float4(prio * (a4.x - mean) / denom, prio * (a4.y - mean) / denom,
                                     prio * (a4.z - mean) / denom, prio * (a4.w - mean) / denom)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        } else {
            for (long long c = lane; c < horizon; c += 32) o[c] = ok ? prio * (a[c] - mean) / denom : 0.0f;
        }
        m = m_next;
        src_row = src_next;
        ok = ok_next;
        p = p_next;
    }
}

// CTAs of the gather kernel (= partial sums): sixteen rows per CTA, two per warp and pass, at most one wave
static int mb_blocks(long long mb_segments)
{
    long long b = (mb_segments + 15) / 16;
    if (b < 1) b = 1;
    if (b > kMbMaxBlocks) b = kMbMaxBlocks;
    return static_cast<int>(b);
}
}  // namespace puff

using namespace puff;

extern "C" size_t puff_minibatch_sm100_scratch_bytes(long long mb_segments)
{
    if (mb_segments <= 0) return 16;
    return static_cast<size_t>(mb_blocks(mb_segments)) * 2 * sizeof(double);
}

extern "C" int puff_minibatch_sm100_gather(const float* advantages, const float* values, const float* prio_probs,
                                           const long long* idx, float* mb_values, float* mb_returns,
                                           float* mb_adv_raw, float* mb_adv_norm, float* mb_prio,
                                           float anneal_beta, long long num_segments, long long horizon,
                                           long long mb_segments, void* scratch, size_t scratch_bytes,
                                           void* cuda_stream)
{
    return puff_minibatch_sm100_gather_ex(advantages, values, prio_probs, idx, mb_values, mb_returns, mb_adv_raw,
                                          mb_adv_norm, mb_prio, anneal_beta, num_segments, num_segments, horizon,
                                          mb_segments, scratch, scratch_bytes, cuda_stream);
}

extern "C" int puff_minibatch_sm100_gather_ex(const float* advantages, const float* values, const float* prio_probs,
                                              const long long* idx, float* mb_values, float* mb_returns,
                                              float* mb_adv_raw, float* mb_adv_norm, float* mb_prio,
                                              float anneal_beta, long long num_segments, long long prio_segments,
                                              long long horizon, long long mb_segments, void* scratch,
                                              size_t scratch_bytes, void* cuda_stream)
{
    if (num_segments < 0 || horizon < 0 || mb_segments < 0 || prio_segments < num_segments) return PUFF_ERR_SHAPE;
    if (mb_segments == 0 || horizon == 0) return PUFF_OK;
    if (num_segments == 0) return PUFF_ERR_SHAPE;   // nothing to gather from
    if (advantages == nullptr || values == nullptr || prio_probs == nullptr || idx == nullptr ||
        mb_values == nullptr || mb_returns == nullptr || mb_adv_raw == nullptr || mb_adv_norm == nullptr ||
        mb_prio == nullptr)
        return PUFF_ERR_NULL;
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 7u) ||
        scratch_bytes < puff_minibatch_sm100_scratch_bytes(mb_segments))
        return PUFF_ERR_WORKSPACE;
    const void* fp[7] = {advantages, values, mb_values, mb_returns, mb_adv_raw, mb_adv_norm, prio_probs};
    bool vec = horizon % 4 == 0;
    for (int i = 0; i < 7; ++i) {
        const uintptr_t p = reinterpret_cast<uintptr_t>(fp[i]);
        if (p & 3u) return PUFF_ERR_ALIGN;
        if (i < 6 && (p & 15u)) vec = false;
    }
    if (reinterpret_cast<uintptr_t>(idx) & 7u) return PUFF_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int blocks = mb_blocks(mb_segments);
    double* partial = static_cast<double*>(scratch);
    // the first kernel of the call is launched plainly (what precedes it in the stream is not this
    // library's to know), the second programmatically behind the first
    if (vec)
        puff_mb_gather_kernel<true><<<blocks, kMbThreads, 0, st>>>(advantages, values, idx, mb_values, mb_returns,
                                                                   mb_adv_raw, partial, num_segments, horizon, mb_segments);
    else
        puff_mb_gather_kernel<false><<<blocks, kMbThreads, 0, st>>>(advantages, values, idx, mb_values, mb_returns,
                                                                    mb_adv_raw, partial, num_segments, horizon, mb_segments);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    long long nb = (mb_segments + 15) / 16;
    if (nb > kMbMaxBlocks) nb = kMbMaxBlocks;
    e = vec ? launch_neighbour(puff_mb_normalize_kernel<true>, static_cast<int>(nb), kMbThreads, 0, st, mb_adv_raw, prio_probs,
                            idx, partial, blocks, mb_adv_norm, mb_prio, anneal_beta, num_segments, prio_segments, horizon,
                            mb_segments)
            : launch_neighbour(puff_mb_normalize_kernel<false>, static_cast<int>(nb), kMbThreads, 0, st, mb_adv_raw, prio_probs,
                            idx, partial, blocks, mb_adv_norm, mb_prio, anneal_beta, num_segments, prio_segments, horizon,
                            mb_segments);
    count_launch();
    return static_cast<int>(e);
}

extern "C" int puff_minibatch_sm100_bad_index(void)
{
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    int h = 0;
    e = cudaMemcpyFromSymbol(&h, g_mb_bad_index, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (h != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_mb_bad_index, &zero, sizeof(int));
    }
    return h;
}
