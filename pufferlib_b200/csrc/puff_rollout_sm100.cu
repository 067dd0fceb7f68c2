// Rollout writer: one environment step into column `column` of the experience
// buffers that the advantage op reads (sm_100a).
//
// Replaces three of the eager column assignments of the reference's rollout loop
// (pufferlib/pufferl.py):
//     r = torch.clamp(r, -1, 1)                      :275
//     self.rewards[batch_rows, l]   = r              :294
//     self.terminals[batch_rows, l] = d.float()      :295
//     self.values[batch_rows, l]    = value.flatten():296
// for a contiguous block of rows (the reference's "fast path for fully
// vectorized envs", :282-283).  The buffers stay row-major [segments, horizon]
// -- the layout the advantage kernels are built around -- so every element is
// a 4-byte store at a stride of `horizon` floats; one launch instead of five.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/puff_advantage.h"

namespace puff {
void count_launch();

__global__ void __launch_bounds__(256)
puff_rollout_write_kernel(float* __restrict__ rewards, float* __restrict__ terminals, float* __restrict__ values,
                          const float* __restrict__ step_rewards, const unsigned char* __restrict__ step_dones,
                          const float* __restrict__ step_values, long long row_begin, long long num_rows,
                          long long column, long long horizon, float reward_clip)
{
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < num_rows;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long o = (row_begin + i) * horizon + column;
        float r = step_rewards[i];
        // torch.clamp keeps NaN; fminf/fmaxf would return the bound
        if (reward_clip > 0.0f && r == r) r = fminf(fmaxf(r, -reward_clip), reward_clip);
        rewards[o] = r;
        terminals[o] = step_dones[i] ? 1.0f : 0.0f;
        values[o] = step_values[i];
    }
}
}  // namespace puff

using namespace puff;

extern "C" int puff_rollout_sm100_write(float* rewards, float* terminals, float* values,
                                        const float* step_rewards, const unsigned char* step_dones,
                                        const float* step_values, long long row_begin, long long num_rows,
                                        long long column, long long num_segments, long long horizon,
                                        float reward_clip, void* cuda_stream)
{
    if (num_segments < 0 || horizon < 0 || num_rows < 0) return PUFF_ERR_SHAPE;
    if (row_begin < 0 || row_begin + num_rows > num_segments || column < 0 || column >= horizon) return PUFF_ERR_SHAPE;
    if (num_rows == 0) return PUFF_OK;
    if (rewards == nullptr || terminals == nullptr || values == nullptr || step_rewards == nullptr ||
        step_dones == nullptr || step_values == nullptr)
        return PUFF_ERR_NULL;
    const void* fp[5] = {rewards, terminals, values, step_rewards, step_values};
    for (int i = 0; i < 5; ++i)
        if (reinterpret_cast<uintptr_t>(fp[i]) & 3u) return PUFF_ERR_ALIGN;
    long long blocks = (num_rows + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    puff_rollout_write_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        rewards, terminals, values, step_rewards, step_dones, step_values, row_begin, num_rows, column, horizon,
        reward_clip);
    count_launch();
    return static_cast<int>(cudaGetLastError());
}
